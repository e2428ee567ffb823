// umma_gemm.cuh -- the tcgen05 contraction engine shared by mul_mat (tf32 / f16 / bf16), the
// outgoing triangle multiplication and the outer-product-mean.
//
//   D[b][m][n] = sum_k A[b][m][k] * B[b][n][k]          (both operands K-major, i.e. "NT")
//
// One persistent CTA per SM walks the (batch, m-tile, n-tile) list.  Per tile:
//   warp 0      TMA producer: 128 x 128-byte A tile and BN x 128-byte B tile per K step, 128-byte swizzle
//   warps 6-9   (tf32 with software rounding only) round the landed fp32 words to tf32 in place
//   warp 1      one elected thread issues tcgen05.mma (M = 128, N = BN, 32 bytes of K each) into TMEM
//   warps 2-5   epilogue: tcgen05.ld of the fp32 accumulators, scale / bias / clamp, stores
// TMEM holds two accumulators of BN columns so the epilogue of a tile overlaps the next tile's
// main loop.  Every wait is bounded (common.cuh).
#pragma once
#include "common.cuh"

namespace ppml_b200 {

// ROW_MAJOR_FUSED: row-major store with the fused neighbours of a Linear (LayerNorm algebra, activation, gate).  An epilogue
// of its own: compiled into the plain instance, that code slowed every HBM-bound product although it never ran there
// (24.2 -> 31.5 us at 65536 x 128 x 256 tf32, 69.9 -> 96.8 at 65536 x 128 x 1024).
enum class Epi { ROW_MAJOR, OPM_BLOCKED, ROW_MAJOR_FUSED };

struct GemmParams {
    int M, N, K;            // per-batch extents: rows of A, rows of B, contraction length
    int batch;
    int m_tiles, n_tiles;
    int flat_rows;          // 1 (batch 1, more row tiles than CTAs): every CTA takes an equal contiguous range of rows and walks
                            // it in tiles of 128, the last one partial (its other rows belong to the next CTA, which computes
                            // them again from its own start): no CTA has a whole tile more than another (3.46 tiles per CTA
                            // ran as 4 at M = 65536)
    int k_steps;            // ceil(K / elements per 128 bytes)
    float* C;
    long long ldc;          // row stride of C (elements)
    long long c_batch;      // batch stride of C (elements)
    const float* bias;      // [N] or null, added after alpha
    float alpha;            // scales the accumulator
    int clamp;              // 1: NaN -> 0 and clamp to +-1e4 (triangle multiplication)
    int vec_ok;             // 1: float4 stores are legal (alignment checked on the host)
    int opm_D, opm_L;       // OPM_BLOCKED: row = d1*L+i, col = d2*L+j -> ((d1*D+d2)*L+i)*L+j
    int ab_fmt;             // operand format of the f16 kind: 0 = fp16, 1 = bf16
    // fused neighbours of a Linear (all optional):
    //   ln_stats [M][2] = (mean, 1 / sqrt(var + eps)) of every row of A, ln_u [N]: the product ran on the raw rows with
    //   weights pre-scaled by gamma, and  out = rstd * (acc - mean * u[n]) + bias[n]  is LayerNorm(x) W^T + b
    //   gate [M][N] (row stride ldc), act: out = act(out) * gate  (the reference's OP_ACT_MUL on a Linear's output)
    const float* ln_stats;
    const float* ln_u;
    const float* gate;
    int act;                // 0 none, 1 sigmoid, 2 silu, 3 gelu (tanh form), 4 tanh, 5 relu
    int* err;               // device error word
};

constexpr int kGemmStageA = 128 * 128;          // bytes of one A tile
constexpr int kGemmMaxStages = 8;

template <int BN>
__host__ __device__ constexpr int gemm_stage_bytes() { return kGemmStageA + BN * 128; }

template <int BN>
__host__ __device__ constexpr int gemm_num_stages() {
    int s = (200 * 1024) / gemm_stage_bytes<BN>();
    return s > kGemmMaxStages ? kGemmMaxStages : s;
}

constexpr int kEpiStagePitch = 144;                       // bytes per staged row: 32 floats + 16 bytes of padding
constexpr int kEpiStageBytes = 32 * kEpiStagePitch;       // one warp's 32 x 32 transposition buffer
constexpr int kEpiBiasBytes = 2 * 256 * 4;                // one warp's copy of the tile's bias slice and of its u slice

// the activations of the reference's act_fwd_scalar (src/backend/CPUKernels.cpp:1903-1916), same formulas; sigmoid and
// SiLU (what the model's gates use) take the hardware exp2 / reciprocal approximations (about 2 ulp, far inside the 1e-3
// of the tf32 product they follow): expf and an IEEE division cost a dozen instructions per element
__device__ __forceinline__ float act_sigmoid_fast(float x) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * x));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return r;
}
__device__ __forceinline__ float act_apply(int kind, float x) {
    switch (kind) {
        case 1: return act_sigmoid_fast(x);
        case 2: return x * act_sigmoid_fast(x);
        case 3: return 0.5f * x * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
        case 4: return tanhf(x);
        case 5: return x > 0.0f ? x : 0.0f;
        default: return x;
    }
}

// dynamic smem: [stages x (A tile | B tile)] (1024-byte aligned), the barriers, then per epilogue warp a
// transposition buffer and a bias slice
template <int BN>
__host__ __device__ constexpr int gemm_smem_bytes() {
    return gemm_num_stages<BN>() * gemm_stage_bytes<BN>() + 1024 /*alignment slack*/ + 512 /*barriers*/ +
           4 * (kEpiStageBytes + kEpiBiasBytes);
}

// MNMAJOR: both operands are stored with the row index (m or n) contiguous and K strided (A[b][k][m],
// B[b][k][n]); the stage then holds boxes of 128 bytes of rows x BK k: 32 rows x 32 k in the 32-byte-chunk form
// of the 128-byte swizzle for fp32 operands, 64 rows x 64 k in the ordinary 128-byte swizzle for 16-bit ones.
template <MmaKind KIND, int BN, Epi EPI, bool CONVERT, bool MNMAJOR = false>
__global__ void __launch_bounds__(CONVERT ? 320 : 192, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmParams p) {
    constexpr int STAGES = gemm_num_stages<BN>();
    constexpr int STAGE_BYTES = gemm_stage_bytes<BN>();
    constexpr int ESIZE = (KIND == MmaKind::TF32) ? 4 : (KIND == MmaKind::F16 ? 2 : 1);
    constexpr int BK = 128 / ESIZE;                       // elements of K per stage
    constexpr uint32_t TMEM_COLS = 2 * BN;
    static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256, "UMMA N");

    constexpr bool kFused = EPI == Epi::ROW_MAJOR_FUSED;
    constexpr bool kRowMajor = EPI != Epi::OPM_BLOCKED;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
    // barrier slots (8 bytes each)
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kGemmMaxStages + s); };
    auto conv_bar = [&](int s) { return bar_base + 8u * (2 * kGemmMaxStages + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (3 * kGemmMaxStages + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (3 * kGemmMaxStages + 2 + a); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + STAGES * STAGE_BYTES + 8 * (3 * kGemmMaxStages + 4));
    volatile int* cta_abort = reinterpret_cast<volatile int*>(smem_gen + STAGES * STAGE_BYTES + 8 * (3 * kGemmMaxStages + 4) + 8);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
            mbar_init(conv_bar(s), 4);
        }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 4); }
        *cta_abort = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
        tmem_relinquish();
    }
    if (warp == 0 && lane == 0) { prefetch_tmap(&tmA); prefetch_tmap(&tmB); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int tiles_per_batch = p.m_tiles * p.n_tiles;
    const int total_tiles = tiles_per_batch * p.batch;
    // the k-th tile of this CTA: batch b, rows [row0, row_end) (row0 + 128 rows are loaded and multiplied), column tile nt
    const int flat_r0 = static_cast<int>(static_cast<long long>(p.M) * blockIdx.x / gridDim.x);
    const int flat_r1 = static_cast<int>(static_cast<long long>(p.M) * (blockIdx.x + 1) / gridDim.x);
    auto tile_at = [&](uint32_t k, int& b, int& row0, int& row_end, int& nt) -> bool {
        if (p.flat_rows) {
            const int im = static_cast<int>(k) / p.n_tiles;
            nt = static_cast<int>(k) - im * p.n_tiles;
            b = 0;
            row0 = flat_r0 + im * 128;
            row_end = min(flat_r1, row0 + 128);
            return row0 < flat_r1;
        }
        const long long t = blockIdx.x + static_cast<long long>(k) * gridDim.x;
        if (t >= total_tiles) return false;
        b = static_cast<int>(t / tiles_per_batch);
        const int r = static_cast<int>(t - static_cast<long long>(b) * tiles_per_batch);
        const int mt = r / p.n_tiles;
        nt = r - mt * p.n_tiles;
        row0 = mt * 128;
        row_end = min(p.M, row0 + 128);
        return true;
    };

    if (warp == 0) {
        // ------------------------------- TMA producer -------------------------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            int b, row0, row_end, nt;
            for (uint32_t tk = 0; ok && tile_at(tk, b, row0, row_end, nt); ++tk) {
                for (int ks = 0; ks < p.k_steps; ++ks, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, cta_abort, p.err, 0x101)) { ok = false; break; }
                    const uint32_t sa = smem_base + s * STAGE_BYTES;
                    mbar_arrive_expect_tx(full_bar(s), STAGE_BYTES);
                    if constexpr (!MNMAJOR) {
                        tma_load_3d(sa, &tmA, full_bar(s), ks * BK, row0, b);
                        tma_load_3d(sa + kGemmStageA, &tmB, full_bar(s), ks * BK, nt * BN, b);
                    } else {
                        // boxes of BK rows (inner, contiguous: 128 bytes) x BK k, one after the other
                        constexpr int kBox = BK * 128;
                        static_assert(BN % BK == 0, "row-contiguous operands: BN must be a multiple of the box width");
#pragma unroll
                        for (int i = 0; i < 128 / BK; ++i) tma_load_3d(sa + i * kBox, &tmA, full_bar(s), row0 + i * BK, ks * BK, b);
#pragma unroll
                        for (int i = 0; i < BN / BK; ++i) tma_load_3d(sa + kGemmStageA + i * kBox, &tmB, full_bar(s), nt * BN + i * BK, ks * BK, b);
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------- MMA issuer ---------------------------------
        if (lane == 0) {
            uint32_t idesc;
            if constexpr (KIND == MmaKind::I8) idesc = make_idesc(2, 1, 1, 0, 0, 128, BN);
            else if constexpr (KIND == MmaKind::TF32) idesc = make_idesc(1, 2, 2, MNMAJOR ? 1 : 0, MNMAJOR ? 1 : 0, 128, BN);
            else idesc = make_idesc(1, p.ab_fmt, p.ab_fmt, MNMAJOR ? 1 : 0, MNMAJOR ? 1 : 0, 128, BN);
            uint32_t it = 0, tile_i = 0;
            bool ok = true;
            int b_, row0_, row_end_, nt_;
            for (; ok && tile_at(tile_i, b_, row0_, row_end_, nt_); ++tile_i) {
                const int acc = tile_i & 1;
                const uint32_t acc_ph = (tile_i >> 1) & 1u;
                if (!mbar_wait(tempty_bar(acc), acc_ph ^ 1u, cta_abort, p.err, 0x201)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int ks = 0; ks < p.k_steps; ++ks, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!mbar_wait(CONVERT ? conv_bar(s) : full_bar(s), ph, cta_abort, p.err, 0x202)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_base + s * STAGE_BYTES;
                    if constexpr (!MNMAJOR) {
                        const uint64_t da = make_smem_desc(sa, 16, 1024, kLayoutSW128);
                        const uint64_t db = make_smem_desc(sa + kGemmStageA, 16, 1024, kLayoutSW128);
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            // 32 bytes of K per instruction: advance the start address by 2 x 16 bytes
                            umma<KIND>(d_tmem, da + 2u * kk, db + 2u * kk, idesc, (ks | kk) != 0 ? 1u : 0u);
                        }
                    } else {
                        // 32-bit operands with the row index contiguous: 128-byte swizzle over 32-byte chunks, whose
                        // atom is 4 k x 128 bytes.  Row blocks (32 rows) are 4096 bytes apart (leading offset),
                        // groups of 4 k are 512 bytes apart (stride offset); one instruction consumes 8 k = 1024 bytes.
                        // 16-bit operands: the ordinary 128-byte swizzle, atom 8 k x 128 bytes; row blocks (64 rows) 8192
                        // bytes apart, groups of 8 k 1024 bytes apart, one instruction consumes 16 k = 2048 bytes.
                        constexpr uint32_t kLbo = BK * 128, kSbo = (KIND == MmaKind::TF32) ? 512 : 1024;
                        constexpr uint32_t kLay = (KIND == MmaKind::TF32) ? kLayoutSW128Base32 : kLayoutSW128;
                        constexpr uint32_t kAdv = (KIND == MmaKind::TF32) ? 64u : 128u;
                        const uint64_t da = make_smem_desc(sa, kLbo, kSbo, kLay);
                        const uint64_t db = make_smem_desc(sa + kGemmStageA, kLbo, kSbo, kLay);
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk)
                            umma<KIND>(d_tmem, da + kAdv * kk, db + kAdv * kk, idesc, (ks | kk) != 0 ? 1u : 0u);
                    }
                    umma_commit(empty_bar(s));          // stage reusable once these MMAs have read it
                }
                if (ok) umma_commit(tfull_bar(acc));    // accumulator complete
            }
        }
        __syncwarp();
    } else if (warp < 6) {
        // ------------------------------- epilogue -----------------------------------
        // Each warp owns 32 accumulator rows (its TMEM lane quarter).  Per 32-column chunk: TMEM -> registers
        // (thread = row), scale / bias / clamp, then through a padded shared-memory buffer so that the global
        // stores are row-contiguous: eight lanes write one 128-byte row segment, four rows per instruction.
        const int q = warp & 3;                          // TMEM lane quarter this warp may touch
        const int ew = warp - 2;
        uint8_t* stage = smem_gen + STAGES * STAGE_BYTES + 512 + ew * (kEpiStageBytes + kEpiBiasBytes);
        float* bias_s = reinterpret_cast<float*>(stage + kEpiStageBytes);
        uint32_t tile_i = 0;
        bool ok = true;
        int b, trow0, row_end, nt;
        for (; ok && tile_at(tile_i, b, trow0, row_end, nt); ++tile_i) {
            const int acc = tile_i & 1;
            const uint32_t acc_ph = (tile_i >> 1) & 1u;
            const int col0 = nt * BN;
            __syncwarp();                                // every lane is done with the previous tile's bias slice
            if (p.bias != nullptr) {
                for (int j = lane; j < BN; j += 32) bias_s[j] = (col0 + j < p.N) ? p.bias[col0 + j] : 0.0f;
            } else {
                for (int j = lane; j < BN; j += 32) bias_s[j] = 0.0f;
            }
            float ln_mean = 0.0f, ln_rstd = 1.0f;
            if (kFused && p.ln_stats != nullptr) {
                for (int j = lane; j < BN; j += 32) bias_s[256 + j] = (col0 + j < p.N) ? p.ln_u[col0 + j] : 0.0f;
                const int rown = trow0 + q * 32 + lane;
                if (rown < p.M) {
                    const float2 st2 = *reinterpret_cast<const float2*>(p.ln_stats + 2 * (static_cast<long long>(b) * p.M + rown));
                    ln_mean = st2.x; ln_rstd = st2.y;
                }
            }
            __syncwarp();
            if (!mbar_wait(tfull_bar(acc), acc_ph, cta_abort, p.err, 0x301)) { ok = false; break; }
            tc_fence_after();
            const int row0 = trow0 + q * 32;
            // blocked store: (slab, position) of the warp's first row and of every chunk's first column, one division each;
            // the elements step from there (an integer division per stored element costs more than the store)
            int opm_d1 = 0, opm_i = 0;
            if constexpr (!kRowMajor) { opm_d1 = row0 / p.opm_L; opm_i = row0 - opm_d1 * p.opm_L; }
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                const int cbase = col0 + c * 32;
                if (cbase >= p.N) break;                 // uniform across the warp
                int opm_d2 = 0, opm_j = 0;
                if constexpr (!kRowMajor) { opm_d2 = cbase / p.opm_L; opm_j = cbase - opm_d2 * p.opm_L; }
                uint32_t v[32];
                tmem_ld32(tmem_base + acc * BN + c * 32 + (static_cast<uint32_t>(q * 32) << 16), v);
                tmem_ld_wait();
                float f[32];
#pragma unroll
                for (int j4 = 0; j4 < 8; ++j4) {
                    const float4 b4 = *reinterpret_cast<const float4*>(bias_s + c * 32 + j4 * 4);
                    f[j4 * 4 + 0] = fmaf(__uint_as_float(v[j4 * 4 + 0]), p.alpha, b4.x);
                    f[j4 * 4 + 1] = fmaf(__uint_as_float(v[j4 * 4 + 1]), p.alpha, b4.y);
                    f[j4 * 4 + 2] = fmaf(__uint_as_float(v[j4 * 4 + 2]), p.alpha, b4.z);
                    f[j4 * 4 + 3] = fmaf(__uint_as_float(v[j4 * 4 + 3]), p.alpha, b4.w);
                }
                if (kFused && p.ln_stats != nullptr) {
                    // f = alpha * acc + bias so far; the LayerNorm form is rstd * (alpha * acc - mean * u) + bias
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float bj = bias_s[c * 32 + j];
                        f[j] = fmaf(fmaf(-ln_mean, bias_s[256 + c * 32 + j], f[j] - bj), ln_rstd, bj);
                    }
                }
                if (p.clamp) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        float x = f[j];
                        x = (x == x) ? fminf(fmaxf(x, -1e4f), 1e4f) : 0.0f;
                        f[j] = x;
                    }
                }
                if (kFused && p.act != 0 && p.gate == nullptr) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) f[j] = act_apply(p.act, f[j]);
                }
                if (p.vec_ok) {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        *reinterpret_cast<float4*>(stage + lane * kEpiStagePitch + j * 16) =
                            make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]);
                    __syncwarp();
                    const int cc = lane & 7;             // 16-byte chunk inside the 128-byte row segment
                    const int col = cbase + cc * 4;
                    // blocked store: the address of this lane's first row, stepped by four rows per round
                    float* optr = nullptr;
                    int o_ii = 0;
                    if constexpr (!kRowMajor) {
                        const int L = p.opm_L, D = p.opm_D;
                        int d1 = opm_d1, d2 = opm_d2, jj = opm_j + cc * 4;
                        o_ii = opm_i + (lane >> 3);
                        while (o_ii >= L) { o_ii -= L; ++d1; }
                        while (jj >= L) { jj -= L; ++d2; }
                        optr = p.C + ((static_cast<long long>(d1) * D + d2) * L + o_ii) * L + jj;
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int rr = (lane >> 3) + 4 * i;
                        const int row = row0 + rr;
                        float4 val = *reinterpret_cast<const float4*>(stage + rr * kEpiStagePitch + cc * 16);
                        if (row < row_end && col < p.N) {    // vec_ok: N, ldc (or L) are multiples of 4
                            if constexpr (kRowMajor) {
                                if (kFused && p.gate != nullptr) {         // read with the same coalesced pattern as the store
                                    const float4 g4 = *reinterpret_cast<const float4*>(p.gate + static_cast<long long>(b) * p.c_batch +
                                                                                        static_cast<long long>(row) * p.ldc + col);
                                    val.x = act_apply(p.act, val.x) * g4.x; val.y = act_apply(p.act, val.y) * g4.y;
                                    val.z = act_apply(p.act, val.z) * g4.z; val.w = act_apply(p.act, val.w) * g4.w;
                                }
                                *reinterpret_cast<float4*>(p.C + static_cast<long long>(b) * p.c_batch +
                                                           static_cast<long long>(row) * p.ldc + col) = val;
                            } else {
                                *reinterpret_cast<float4*>(optr) = val;
                            }
                        }
                        if constexpr (!kRowMajor) {          // four rows on: L is a multiple of 4 here, so at most one slab boundary
                            const int L = p.opm_L;
                            optr += 4 * L; o_ii += 4;
                            if (o_ii >= L) { o_ii -= L; optr += static_cast<long long>(p.opm_D - 1) * L * L; }
                        }
                    }
                    __syncwarp();
                } else {
                    const int row = row0 + lane;
                    if (row < row_end) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int col = cbase + j;
                            if (col < p.N) {
                                if constexpr (kRowMajor) {
                                    const long long off = static_cast<long long>(b) * p.c_batch + static_cast<long long>(row) * p.ldc + col;
                                    p.C[off] = (kFused && p.gate != nullptr) ? act_apply(p.act, f[j]) * p.gate[off] : f[j];
                                } else {
                                    const int L = p.opm_L, D = p.opm_D;
                                    int d1 = opm_d1, ii = opm_i + lane, d2 = opm_d2, jj = opm_j + j;
                                    while (ii >= L) { ii -= L; ++d1; }
                                    while (jj >= L) { jj -= L; ++d2; }
                                    p.C[((static_cast<long long>(d1) * D + d2) * L + ii) * L + jj] = f[j];
                                }
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
        }
    } else {
        // ------------------------------- tf32 rounding (CONVERT only) ----------------
        if constexpr (CONVERT) {
            const int ctid = threadIdx.x - 6 * 32;       // 0..127
            uint32_t it = 0;
            bool ok = true;
            int b_, row0_, row_end_, nt_;
            for (uint32_t tk = 0; ok && tile_at(tk, b_, row0_, row_end_, nt_); ++tk) {
                for (int ks = 0; ks < p.k_steps; ++ks, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!mbar_wait(full_bar(s), ph, cta_abort, p.err, 0x401)) { ok = false; break; }
                    float4* st = reinterpret_cast<float4*>(smem_gen + s * STAGE_BYTES);
#pragma unroll 4
                    for (int i = ctid; i < STAGE_BYTES / 16; i += 128) {
                        float4 x = st[i];
                        x.x = tf32_round(x.x); x.y = tf32_round(x.y); x.z = tf32_round(x.z); x.w = tf32_round(x.w);
                        st[i] = x;
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(conv_bar(s));
                }
            }
        }
    }

    // common exit: all roles meet here (also after an aborted wait) before TMEM is released
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace ppml_b200
