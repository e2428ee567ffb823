// common.cuh -- shared device helpers for the sm_100a kernels: mbarrier, TMA, tcgen05/TMEM
// wrappers (inline PTX), shared-memory operand descriptors and the bounded-wait policy.
#pragma once
#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>

namespace ppml_b200 {

// ---------------------------------------------------------------------------------------------
// Status codes returned by the C-ABI (0 = launched).  1..6 keep the meaning the reference's
// launchers give them (src/cuda/MulMatQ8Kernel.cu:476-547): 1 bad args / unsupported, 2 K%32,
// 3 scratch alloc, 4 quantize launch, 5 weight type, 6 kernel launch.
// ---------------------------------------------------------------------------------------------
enum : int { ST_OK = 0, ST_BAD_ARGS = 1, ST_BAD_K = 2, ST_SCRATCH = 3, ST_QUANT = 4, ST_WTYPE = 5,
             ST_LAUNCH = 6, ST_UNSUPPORTED_PATH = 7, ST_DEVICE_ABORT = 8, ST_TOO_LARGE = 9 };

// Device error word: a kernel whose bounded wait ran out stores a non-zero code there and leaves
// early; ppml_b200_device_status() reads it.  Layout: [0] code, [1] where (role << 8 | site).
// The word lives in one translation unit; kernels get its device address as an argument.
int* device_error_ptr();

// ---------------------------------------------------------------------------------------------
// Generic PTX helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.b32 %0, 1, 0, P;\n\t}\n"
        : "=r"(pred));
    return pred != 0;
}

// ---- programmatic dependent launch ---------------------------------------------------------------
// A kernel launched with launch_pdl() may start (its CTAs become resident and run their prologue) while the kernel before it
// in the stream is still running; pdl_wait() blocks until that kernel has completed and its memory operations are visible,
// so everything after it keeps the stream's ordering.  Every kernel that is launched this way calls pdl_wait() before its
// first access to global memory.  pdl_launch_dependents() lets the next kernel of the stream begin launching early.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- mbarrier -------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_inval(uint32_t bar) {
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
#ifdef PPML_MBAR_TEST_WAIT
        "mbarrier.test_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
#else
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
#endif
        "selp.b32 %0, 1, 0, P;\n\t}\n"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Same test, but the hardware may keep the thread suspended for up to `ns` nanoseconds while the phase is
// incomplete: a waiting warp then takes far fewer issue slots from the warps that do the arithmetic.
__device__ __forceinline__ bool mbar_test_suspend(uint32_t bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, P;\n\t}\n"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(ns) : "memory");
    return ok != 0;
}

// Bounded wait.  Every spin in these kernels goes through here: after kWaitCycles clock cycles
// (or as soon as another thread of the CTA has given up) it records where it stopped,
// raises the CTA-wide abort flag and returns false; callers then leave their role loop and fall
// through to the common exit, which still frees TMEM.
constexpr long long kWaitCycles = 3000000000LL;   // about 1.5 s at the maximum SM clock

// The polling loop lives in a function of its own (not inlined): a wait that succeeds at once costs one
// instruction and a branch at the call site, and the loop, the clock reads and the abort path do not bloat
// every role loop.
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* cta_abort, int* err, int site) {
    const long long t0 = clock64();
    for (uint32_t it = 1;; ++it) {
        if (mbar_test(bar, parity)) return true;
        if ((it & 63u) == 0u) {
            if (*cta_abort) return false;
            if (clock64() - t0 > kWaitCycles) break;
        }
    }
    *cta_abort = 1;
    err[0] = ST_DEVICE_ABORT;
    err[1] = site;
    __threadfence();
    return false;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* cta_abort, int* err, int site) {
    if (mbar_test(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, cta_abort, err, site);
}

// Same policy for roles that usually wait long (producers running ahead of a slow consumer): backs
// off with nanosleep between polls so that the spinning does not take issue slots from the warps
// doing the arithmetic.
__device__ __forceinline__ bool mbar_wait_relaxed(uint32_t bar, uint32_t parity, volatile int* cta_abort, int* err, int site) {
    if (mbar_test(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t it = 1;; ++it) {
        __nanosleep(it < 8 ? 32 : 128);
        if (mbar_test(bar, parity)) return true;
        if ((it & 15u) == 0u) {
            if (*cta_abort) return false;
            if (clock64() - t0 > kWaitCycles) break;
        }
    }
    *cta_abort = 1;
    err[0] = ST_DEVICE_ABORT;
    err[1] = site;
    __threadfence();
    return false;
}

// ---- proxies / fences -------------------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() {      // generic-proxy smem writes -> async proxy
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- TMA (bulk tensor copies, no cluster forms) -----------------------------------------------
__device__ __forceinline__ void prefetch_tmap(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
// x = innermost coordinate (elements); the byte offset x*elem must be a multiple of 16.
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const void* tmap, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const void* tmap, uint32_t bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst_smem, const void* tmap, uint32_t bar, int x, int y, int z, int w) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

// Tiled bulk store shared -> global (bulk async-group completion): the box at `src_smem`, laid out as the tensor map's
// swizzle mode says, goes to coordinates (x, y, z); parts of the box outside the tensor are not written.  The writes to
// shared memory must have been made visible to the async proxy (fence_proxy_async_smem) before the issuing thread runs this.
__device__ __forceinline__ void tma_store_3d(const void* tmap, uint32_t src_smem, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(src_smem), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// waits until the bulk stores committed by this thread have finished reading shared memory (the buffers may be reused)
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// the same, but the most recently committed group may still be reading (two buffers used in turn)
__device__ __forceinline__ void bulk_wait_read_but_one() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
// waits until the bulk stores committed by this thread are complete
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Untiled bulk copy global -> shared (both addresses 16-byte aligned, size a multiple of 16), completion counted in
// bytes on the mbarrier.
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar) : "memory");
}

// ---- TMEM -------------------------------------------------------------------------------------
// One full warp allocates; ncols is a power of two in [32, 512]; the base address lands in smem.
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp gets lane (base+t), r[j] = column j.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
// Writes the same 32-bit value to 32 lanes x 32 consecutive columns (thread t -> lane base+t).
__device__ __forceinline__ void tmem_st32_fill(uint32_t taddr, uint32_t v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, "
        "%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};"
        ::"r"(taddr), "r"(v) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---- tcgen05.mma ------------------------------------------------------------------------------
// Instruction descriptor (32 bit): [4,6) D format (1 = f32, 2 = s32), [7,10) A format, [10,13) B format
// (f16 kinds: 0 f16, 1 bf16, 2 tf32; i8 kind: 1 = signed 8 bit), [15] A major, [16] B major
// (0 = K-major, 1 = MN-major), [17,23) N >> 3, [24,29) M >> 4.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t d_fmt, uint32_t a_fmt, uint32_t b_fmt,
                                                  uint32_t a_mn_major, uint32_t b_mn_major,
                                                  uint32_t M, uint32_t N) {
    return (d_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | (a_mn_major << 15) | (b_mn_major << 16) |
           ((N >> 3) << 17) | ((M >> 4) << 24);
}

// Shared-memory operand descriptor (64 bit): [0,14) start address >> 4, [16,30) leading byte
// offset >> 4, [32,46) stride byte offset >> 4, [46,48) version = 1, [61,64) layout
// (0 = no swizzle / interleaved, 2 = 128-byte swizzle over 16-byte chunks, 1 = 128-byte swizzle over
// 32-byte chunks: the layout of 32-bit operands whose row index is contiguous, 4 = 64-byte swizzle).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint32_t layout) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(layout & 7u) << 61;
    return d;
}
constexpr uint32_t kLayoutSW128 = 2;
constexpr uint32_t kLayoutSW128Base32 = 1;
constexpr uint32_t kLayoutSW64 = 4;           // 64-byte swizzle over 16-byte chunks: tiles whose rows are 64 bytes

enum class MmaKind { TF32, F16, I8 };

template <MmaKind KIND>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                     uint32_t accumulate) {
    if constexpr (KIND == MmaKind::TF32) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}\n"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
    } else if constexpr (KIND == MmaKind::F16) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}\n"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
    }
}

// Arrives (count 1) on the mbarrier once every tcgen05.mma issued so far by this thread is done.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Byte offset of 16-byte chunk `c` (0..7) of row `r` inside a K-major tile stored with the
// 128-byte swizzle: rows are 128 bytes, groups of 8 rows are 1024 bytes, chunk index XOR (row % 8).
// The tile base must be 1024-byte aligned.
__device__ __forceinline__ uint32_t sw128_off(uint32_t r, uint32_t c) {
    return (r >> 3) * 1024u + (r & 7u) * 128u + ((c ^ (r & 7u)) << 4);
}

// ---- shared-memory loads through 32-bit shared addresses (one address register, no generic-pointer math) ----
__device__ __forceinline__ float4 lds_f4(uint32_t saddr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(saddr));
    return v;
}
// the same with a compile-time byte offset folded into the instruction (no address arithmetic)
template <int OFF>
__device__ __forceinline__ float4 lds_f4_at(uint32_t saddr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4+%5];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(saddr), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ uint16_t lds_u16_at(uint32_t saddr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1+%2];" : "=h"(v) : "r"(saddr), "n"(OFF));
    return v;
}
// mbarrier arrive by the lane whose `lane` is 0, as one predicated instruction (no divergent region)
__device__ __forceinline__ void mbar_arrive_lane0(uint32_t bar, uint32_t lane) {
    asm volatile("{\n\t.reg .pred P;\n\tsetp.eq.u32 P, %1, 0;\n\t@P mbarrier.arrive.shared::cta.b64 _, [%0];\n\t}\n" ::"r"(bar), "r"(lane) : "memory");
}
__device__ __forceinline__ uint16_t lds_u16(uint32_t saddr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(saddr));
    return v;
}

// Regroups a 32 x 32 fp32 tile held one row per lane (lane r holds v[j] = element j of row r) for row-contiguous
// global accesses: afterwards lane l holds in v[8 s .. 8 s + 7] (s = 0..3) the elements 8 (l >> 3) .. 8 (l >> 3) + 7 of
// row (l & 7) + 8 s, so that an access with one 32-byte piece per lane covers eight whole 128-byte rows instead of
// touching 32 rows with 32 bytes each.  Two exchange steps: lane bit 3 + st pairs with the piece bit st (8 or 16 floats).
// All 32 lanes must call it.
__device__ __forceinline__ void rows_to_line_pieces(float (&v)[32], int lane) {
#pragma unroll
    for (int st = 0; st < 2; ++st) {
        const int bit = 8 << st;
        const bool up = (lane & bit) != 0;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            if ((j & bit) == 0) {
                // the lane with the bit clear keeps piece j and sends j + bit; its partner the reverse
                const float send = up ? v[j] : v[j + bit];
                const float got = __shfl_xor_sync(0xffffffffu, send, bit);
                if (up) v[j] = got; else v[j + bit] = got;
            }
        }
    }
}

// the activations of the reference's act_fwd_scalar (src/backend/CPUKernels.cpp:1903-1916), same formulas
__device__ __forceinline__ float act_scalar(int kind, float x) {
    switch (kind) {
        case 1: return 1.0f / (1.0f + expf(-x));
        case 2: return x / (1.0f + expf(-x));
        case 3: return 0.5f * x * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
        case 4: return tanhf(x);
        case 5: return x > 0.0f ? x : 0.0f;
        default: return x;
    }
}

// ---- packed fp32 pairs (one issue slot for two lanes of add / mul / fma) ------------------------
__device__ __forceinline__ uint64_t pack2(float a, float b) {
    uint64_t r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b)); return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& a, float& b) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t fadd2(uint64_t a, uint64_t b) {
    uint64_t r; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r;
}
__device__ __forceinline__ uint64_t fadd2_rz(uint64_t a, uint64_t b) {
    uint64_t r; asm("add.rz.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r;
}
__device__ __forceinline__ uint64_t fmul2(uint64_t a, uint64_t b) {
    uint64_t r; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r;
}
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c)); return r;
}

__device__ __forceinline__ float tf32_round(float x) {
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
    return __uint_as_float(u);
}

}  // namespace ppml_b200

// ---- host: launch with programmatic stream serialization (PPML_B200_PDL=0 switches it off) -----------------------------
#include <cstdlib>
#include <utility>
namespace ppml_b200 {
inline bool pdl_enabled() {
    static const bool on = [] { const char* e = std::getenv("PPML_B200_PDL"); return !(e && e[0] == '0'); }();
    return on;
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
}  // namespace ppml_b200
