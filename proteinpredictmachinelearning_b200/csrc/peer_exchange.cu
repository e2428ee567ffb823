// peer_exchange.cu -- the exchanges of the sharded block as single kernels over peer memory (NVLink / NVSwitch).
//
// When the activations of a block are cut into contiguous flat chunks over the GPUs of one box (one process per GPU),
// three things have to cross between ranks under the reference's flat-buffer semantics: a pair bias and the
// outer-product-mean's `right` operand are needed whole on every rank (all-gather), and the (n, l) transposes that the
// reference runs as permute copies (src/modules/Attention.cpp:489, :744) move every element to another rank's rows.
// Here each is ONE kernel: every rank pushes its part straight into the other ranks' buffers with plain stores to peer
// memory, between two flag rounds:
//   round 1 (before the stores)  "I have arrived": nobody overwrites a buffer a peer's earlier kernels may still read;
//   round 2 (after the stores)   "my part has landed": when the kernel ends, every rank's buffer is complete and local.
// Consumers then read local memory only -- no kernel of the library ever issues a load from peer memory, and TMA is never
// pointed at it.  There is no multicast and no in-switch reduction: plain st.global to mapped peer addresses.
//
// Flags are 32-bit epoch counters in peer-mapped memory, one row of 8 per exchange site and round; the epoch itself lives
// in device memory (it advances by one per launch), so a launch recorded in a CUDA graph stays valid when replayed.
// Every spin is bounded (about 1.5 s): a rank whose peers never arrive records ST_DEVICE_ABORT in the device error word
// and returns; nothing here can wait for another launch on the same GPU.
//
// Buffers and flags are shared through CUDA IPC (ppml_b200_peer_alloc / _export / _open): plain cudaMalloc'ed memory,
// mapped once at set-up.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstring>

#include "../../include/ppml_b200.h"
#include "kernels.h"

namespace ppml_b200 {

namespace {

constexpr int kMaxRanks = 8;
constexpr int kMaxSites = 16;

struct Peers { void* p[kMaxRanks]; };

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Device-resident state of one process: the epoch of every site and the counter that finds the last CTA of a launch.
__device__ uint32_t g_site_epoch[kMaxSites];
__device__ int g_cta_count[kMaxSites];

// flags layout (uint32): [site][round 0..1][kMaxRanks]
__device__ __forceinline__ uint32_t* flag_of(void* base, int site, int round, int from) {
    return static_cast<uint32_t*>(base) + (site * 2 + round) * kMaxRanks + from;
}

// Bounded wait until every rank's flag of (site, round) in this rank's own flag block has reached `epoch`.
// Called by one thread; returns false after the time limit (the error word is set).
__device__ bool wait_all(void* my_flags, int site, int round, int world, uint32_t epoch, int* err) {
    const long long t0 = clock64();
    for (int r = 0; r < world; ++r) {
        const uint32_t* f = flag_of(my_flags, site, round, r);
        uint32_t it = 0;
        while (static_cast<int32_t>(ld_acquire_sys(f) - epoch) < 0) {
            if ((++it & 255u) == 0u && clock64() - t0 > kWaitCycles) {
                err[0] = ST_DEVICE_ABORT; err[1] = 0x5000 + site * 16 + round * 8 + r;
                __threadfence();
                return false;
            }
        }
    }
    return true;
}

// Shared prologue / epilogue of the exchange kernels.
//   begin: thread 0 of CTA 0 tells every peer "rank arrived" (round 0); thread 0 of every CTA waits until all have.
//   end:   after this CTA's stores, the last CTA of the launch tells every peer "rank's part has landed" (round 1), waits
//          for all parts and advances the epoch.
__device__ bool exchange_begin(const Peers& flags, int site, int rank, int world, uint32_t epoch, int* err, int* ok_smem) {
    if (threadIdx.x == 0) {
        if (blockIdx.x == 0)
            for (int r = 0; r < world; ++r) st_release_sys(flag_of(flags.p[r], site, 0, rank), epoch);
        *ok_smem = wait_all(flags.p[rank], site, 0, world, epoch, err) ? 1 : 0;
    }
    __syncthreads();
    return *ok_smem != 0;
}

__device__ void exchange_end(const Peers& flags, int site, int rank, int world, uint32_t epoch, int* err) {
    __threadfence_system();                       // this thread's peer stores are visible system-wide
    __syncthreads();
    if (threadIdx.x == 0) {
        const int done = atomicAdd(&g_cta_count[site], 1);
        if (done == static_cast<int>(gridDim.x) - 1) {
            __threadfence_system();               // ... and so are those of the CTAs counted before this one
            for (int r = 0; r < world; ++r) st_release_sys(flag_of(flags.p[r], site, 1, rank), epoch);
            wait_all(flags.p[rank], site, 1, world, epoch, err);
            g_cta_count[site] = 0;
            g_site_epoch[site] = epoch;
            __threadfence();
        }
    }
}

// all-gather: this rank's n16 16-byte words go to word offset rank * n16 of every rank's buffer (its own included)
__global__ void __launch_bounds__(256)
peer_all_gather_kernel(const uint4* __restrict__ src, Peers dst, long long n16, int rank, int world, Peers flags, int site, int* err) {
    __shared__ int ok_s;
    const uint32_t epoch = g_site_epoch[site] + 1u;
    if (!exchange_begin(flags, site, rank, world, epoch, err, &ok_s)) return;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (int pr = 0; pr < world; ++pr) {
        const int peer = (rank + pr) % world;     // start with the own copy, then walk the ring: spreads the traffic
        uint4* out = static_cast<uint4*>(dst.p[peer]) + static_cast<long long>(rank) * n16;
        for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16; i += stride) out[i] = src[i];
    }
    exchange_end(flags, site, rank, world, epoch, err);
}

// (n, l) transpose of x [n_loc][L][C] (this rank's n range) into out [l_loc][world * n_loc][C] on the rank that owns l:
// row (n, l) of C floats goes to rank l / l_loc, row (l % l_loc, rank * n_loc + n).  c4 = C / 4.
__global__ void __launch_bounds__(256)
peer_transpose_kernel(const uint4* __restrict__ x, Peers out, int n_loc, int L, int c4, int rank, int world, Peers flags, int site, int* err) {
    __shared__ int ok_s;
    const uint32_t epoch = g_site_epoch[site] + 1u;
    if (!exchange_begin(flags, site, rank, world, epoch, err, &ok_s)) return;
    // a warp moves whole rows of c4 16-byte words: the destination of a row is found once per row with 32-bit arithmetic
    // (a division per 16-byte word, as first written, cost more than the copy), and four rows are in flight per warp
    const int l_loc = L / world;
    const int rows = n_loc * L;
    const long long n_all = static_cast<long long>(world) * n_loc;
    const int lane = threadIdx.x & 31;
    const int warps_total = static_cast<int>(gridDim.x) * (blockDim.x >> 5);
    const int warp_id = static_cast<int>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    constexpr int kRows = 4;
    auto dst_of = [&](int row) -> uint4* {
        const int n = row / L, l = row - n * L;
        const int peer = l / l_loc;
        return static_cast<uint4*>(out.p[peer]) + (static_cast<long long>(l - peer * l_loc) * n_all + rank * n_loc + n) * c4;
    };
    if (c4 <= 64) {
        for (int row = warp_id * kRows; row < rows; row += warps_total * kRows) {
            uint4 v[kRows][2];
#pragma unroll
            for (int r = 0; r < kRows; ++r)
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    const int c = lane + 32 * k;
                    if (row + r < rows && c < c4) v[r][k] = x[static_cast<long long>(row + r) * c4 + c];
                }
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                if (row + r >= rows) break;
                uint4* dst = dst_of(row + r);
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    const int c = lane + 32 * k;
                    if (c < c4) dst[c] = v[r][k];
                }
            }
        }
    } else {
        for (int row = warp_id; row < rows; row += warps_total) {
            uint4* dst = dst_of(row);
            for (int c = lane; c < c4; c += 32) dst[c] = x[static_cast<long long>(row) * c4 + c];
        }
    }
    exchange_end(flags, site, rank, world, epoch, err);
}

bool peers_ok(void* const* ptrs, int world) {
    if (!ptrs || world < 1 || world > kMaxRanks) return false;
    for (int r = 0; r < world; ++r) if (!ptrs[r] || (reinterpret_cast<uintptr_t>(ptrs[r]) & 15u)) return false;
    return true;
}

Peers as_peers(void* const* ptrs, int world) {
    Peers p{};
    for (int r = 0; r < world; ++r) p.p[r] = ptrs[r];
    return p;
}

}  // namespace

}  // namespace ppml_b200

using namespace ppml_b200;

extern "C" {

int ppml_b200_peer_flag_bytes(void) { return kMaxSites * 2 * kMaxRanks * 4; }

void* ppml_b200_peer_alloc(int64_t bytes) {
    void* p = nullptr;
    if (bytes <= 0 || cudaMalloc(&p, static_cast<size_t>(bytes)) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    if (cudaMemset(p, 0, static_cast<size_t>(bytes)) != cudaSuccess) { cudaGetLastError(); cudaFree(p); return nullptr; }
    cudaDeviceSynchronize();
    return p;
}
void ppml_b200_peer_free(void* p) { if (p) cudaFree(p); }

int ppml_b200_peer_export(void* p, void* handle64) {
    if (!p || !handle64) return ST_BAD_ARGS;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    if (cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), p) != cudaSuccess) { cudaGetLastError(); return ST_LAUNCH; }
    return ST_OK;
}
void* ppml_b200_peer_open(const void* handle64) {
    if (!handle64) return nullptr;
    void* p = nullptr;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return p;
}
void ppml_b200_peer_close(void* p) { if (p) cudaIpcCloseMemHandle(p); }

int ppml_b200_peer_all_gather(const void* src, void* const* dst_ptrs, int64_t bytes_per_rank, int rank, int world,
                              void* const* flag_ptrs, int site, void* stream) {
    if (!src || bytes_per_rank <= 0 || (bytes_per_rank & 15) || rank < 0 || rank >= world || site < 0 || site >= kMaxSites) return ST_BAD_ARGS;
    if ((reinterpret_cast<uintptr_t>(src) & 15u) || !peers_ok(dst_ptrs, world) || !peers_ok(flag_ptrs, world)) return ST_BAD_ARGS;
    int* err = device_error_ptr();
    if (!err) return ST_LAUNCH;
    const long long n16 = bytes_per_rank / 16;
    long long grid = (n16 + 255) / 256;
    const int cap = num_sms() / 2 > 0 ? num_sms() / 2 : 1;        // every CTA must be resident: it waits for the peers
    if (grid > cap) grid = cap;
    peer_all_gather_kernel<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(src), as_peers(dst_ptrs, world), n16, rank, world, as_peers(flag_ptrs, world), site, err);
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_LAUNCH;
}

int ppml_b200_peer_transpose(const float* x, void* const* out_ptrs, int n_loc, int L, int C, int rank, int world,
                             void* const* flag_ptrs, int site, void* stream) {
    if (!x || n_loc <= 0 || L <= 0 || C <= 0 || (C & 3) || rank < 0 || rank >= world || site < 0 || site >= kMaxSites) return ST_BAD_ARGS;
    if (L % world) return ST_BAD_ARGS;
    if ((reinterpret_cast<uintptr_t>(x) & 15u) || !peers_ok(out_ptrs, world) || !peers_ok(flag_ptrs, world)) return ST_BAD_ARGS;
    int* err = device_error_ptr();
    if (!err) return ST_LAUNCH;
    if (static_cast<long long>(n_loc) * L > 0x7fffffffLL) return ST_BAD_ARGS;
    const long long total = static_cast<long long>(n_loc) * L * (C / 4);
    long long grid = (total + 255) / 256;
    const int cap = num_sms() > 0 ? num_sms() : 1;
    if (grid > cap) grid = cap;
    peer_transpose_kernel<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint4*>(x), as_peers(out_ptrs, world), n_loc, L, C / 4, rank, world, as_peers(flag_ptrs, world), site, err);
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_LAUNCH;
}

}  // extern "C"
