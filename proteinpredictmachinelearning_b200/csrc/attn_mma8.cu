// Attention forward for head dim 8 (the extra-MSA blocks) on the warp-level tensor-core instruction
// mma.sync.m16n8k8 (tf32 operands, fp32 accumulation).  A head dim of 8 is exactly one k step of that instruction for
// the score product and one n tile for the P V product, so nothing is padded; the tcgen05 shapes (M = 128, N >= 16,
// operands in swizzled shared-memory tiles of at least 32 bytes per row) do not fit a contraction this short, and on
// CUDA cores the sixteen FMAs per (query, key) pair alone cost 0.24 ms at the extra-MSA size.
//
// A warp owns 32 query rows (two m tiles) of one (batch, head) and walks the keys in tiles of 64:
//   S = bias tile (the accumulator's start value) + Q K^T    8 n tiles x 2 m tiles, K fragments shared by the m tiles
//   online softmax in the accumulator layout (a row lives in the four lanes of a quad: two shuffles per row and tile)
//   O += P V                                                 P is the score fragment itself: with the keys of an n tile
//                                                            taken in the order (0, 2, 4, 6, 1, 3, 5, 7) the
//                                                            accumulator layout of S is the A layout of the product
//   l += P 1                                                 the row sums come from a product of the same fragment with ones
// With a bias shared by the batch (or none) a CTA of 8 warps works on four batch elements and 64 rows, so one staged bias
// tile serves four batch elements and one staged K / V tile two row groups; with a bias per batch element a CTA of 4 warps
// works on 128 rows of one batch element.  A CTA walks several consecutive row blocks; its copies run ahead across them.
// Q, K, V (fp32, 16-byte aligned rows) and the bias tile arrive by cp.async into two stages, laid out so that every
// fragment read is one conflict-free 4-byte (K, V) or 8-byte (bias) read per lane.  Arithmetic contract as the other
// attention kernels (masking, eps in the denominator, rows without a visible key, first-tile rule); Q, K and V are
// rounded to tf32 (half away from zero), P is cut to tf32 and its row sum taken from the cut values; softmax and
// accumulation are fp32.
#include "kernels.h"

#include <math_constants.h>

namespace ppml_b200 {
namespace {

__device__ __forceinline__ float ex2_approx(float x) {
    float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
    float y; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y;
}
// the tensor core reads the upper 19 bits of an operand: adding half an ulp of tf32 first makes that a rounding
__device__ __forceinline__ uint32_t tf32_bits(float x) { return __float_as_uint(x) + 0x1000u; }

__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async16(float* dst, const float* src, bool ok) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))),
                 "l"(src), "r"(ok ? 16 : 0) : "memory");
}
__device__ __forceinline__ void cp_async4(float* dst, const float* src, bool ok) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))),
                 "l"(src), "r"(ok ? 4 : 0) : "memory");
}

constexpr int kTile = 64;        // keys per step
constexpr int kPitch = 72;       // floats per staged bias row: 8-byte reads of a half-warp (4 rows x 4 lanes) hit 16 bank pairs
constexpr int kKV = kTile * 8;   // floats of one K (or V) tile

// NW warps per CTA, GB batch elements per CTA: 32 NW / GB query rows per CTA
template <int GB, int NW, int MT>
struct Shape {
    static constexpr int rows = 16 * MT * NW / GB;
    static constexpr int stage = rows * kPitch + 2 * GB * kKV;       // floats of one stage: bias rows, K tiles, V tiles
    static constexpr int qtile = 16 * MT * NW * 8;                        // floats of the Q rows of one row block
    static constexpr int smem_bytes = (2 * stage + qtile) * static_cast<int>(sizeof(float));
};

// GB: batch elements per CTA (4: warp w works on batch element w % 4 and the 32-row group w / 4; 1: the warps take
// 32-row groups of one batch element)
template <int GB, int NW, int MT>
__global__ void __launch_bounds__(32 * NW, GB == 4 ? (MT == 2 ? 16 : 24) / NW : 2)
attn_d8_mma_kernel(const float* __restrict__ Q, const float* __restrict__ K, const float* __restrict__ V,
                   const float* __restrict__ bias, float* __restrict__ O, float* __restrict__ LSE,
                   int B, int H, int L, int Lk, int causal, float scale, float eps, long long bias_batch_stride, int ft,
                   int bias_vec, int blocks_per_cta, const AttnLayout lay) {
    constexpr int NT = 32 * NW;
    constexpr int kRows = Shape<GB, NW, MT>::rows;                  // query rows per CTA
    constexpr int kBias = kRows * kPitch;
    constexpr int kStage = Shape<GB, NW, MT>::stage;
    constexpr float kLog2e = 1.4426950408889634f;
    extern __shared__ __align__(16) float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int bl = warp % GB, rg = warp / GB;                   // batch element and 32-row group of this warp
    const int hh = blockIdx.y;
    const int b0 = blockIdx.z * GB;
    const int b = b0 + bl;
    const bool b_ok = b < B;
    // this CTA's row blocks (kRows rows each): the copies run ahead across their boundaries
    const int n_blocks = (L + kRows - 1) / kRows;
    const int rb_begin = blockIdx.x * blocks_per_cta, rb_end = min(rb_begin + blocks_per_cta, n_blocks);
    if (rb_begin >= rb_end) return;
    const float* Bh = bias ? bias + static_cast<size_t>(GB == 1 ? b0 : 0) * bias_batch_stride +
                                 static_cast<size_t>(hh) * L * static_cast<size_t>(Lk) : nullptr;

    // rows of this thread in row block rb: index r = mi * 2 + hr -> row rb * kRows + rg * (16 * MT) + mi * 16 + hr * 8 + g
    int jmax[2 * MT];
    uint32_t qa[MT][4];
    float m[2 * MT], mfirst[2 * MT];
    float o[MT][4], lacc[MT][4];                       // lacc: row sums of P (every column of the fragment holds the sum)
    auto begin_block = [&](int rb) {
#pragma unroll
        for (int mi = 0; mi < MT; ++mi)
#pragma unroll
            for (int hr = 0; hr < 2; ++hr) {
                const int i = rb * kRows + rg * (16 * MT) + mi * 16 + hr * 8 + g;
                const bool ok = b_ok && i < L;
                jmax[mi * 2 + hr] = ok ? (causal ? min(i + 1, Lk) : Lk) : 0;
                const float* qp = smem + 2 * kStage + (bl * kRows + rg * (16 * MT) + mi * 16 + hr * 8 + g) * 8;     // staged, zero-filled
                qa[mi][hr] = tf32_bits(qp[t] * scale);                      // a0 / a1: channel t
                qa[mi][hr + 2] = tf32_bits(qp[t + 4] * scale);              // a2 / a3: channel t + 4
            }
#pragma unroll
        for (int r = 0; r < 2 * MT; ++r) { m[r] = -CUDART_INF_F; mfirst[r] = -CUDART_INF_F; }
        if (lay.gate && t == 0 && b_ok) {
            // the block's gate rows are read when it ends: bring them into L2 now
#pragma unroll
            for (int r = 0; r < 2 * MT; ++r) {
                const int i = rb * kRows + rg * (16 * MT) + (r >> 1) * 16 + (r & 1) * 8 + g;
                if (i < L) asm volatile("prefetch.global.L2 [%0];" ::"l"(lay.gate + b * lay.g_b + hh * lay.g_h + static_cast<long long>(i) * lay.g_l));
            }
        }
#pragma unroll
        for (int mi = 0; mi < MT; ++mi)
#pragma unroll
            for (int e = 0; e < 4; ++e) { o[mi][e] = 0.0f; lacc[mi][e] = 0.0f; }
    };
    // keys needed by any row of row block rb
    auto keys_of = [&](int rb) { return causal ? min(min(rb * kRows + kRows - 1, L - 1) + 1, Lk) : Lk; };

    // one stage: [bias rows][K of the GB batch elements][V of the GB batch elements]
    //   K tile: [n tile][channel half][key of the n tile][channel of the half]      -> fragment element = lane
    //   V tile: [n tile][key parity][key pair of the n tile][channel]               -> fragment element = t * 8 + g
    // what this thread copies per stage is fixed: key (tid % 128) / 2 and 16-byte half tid % 2 of the K and V tile of the
    // batch elements tid / 128, tid / 128 + NT / 128, ...; 16 bytes at column 4 (tid % 16) of the bias rows tid / 16,
    // tid / 16 + NT / 16, ...; with the first key tile of a row block, two 16-byte pieces of its Q rows
    const int ckey = (threadIdx.x & 127) >> 1, chalf = threadIdx.x & 1, cb = threadIdx.x >> 7;
    const int kdst = (((ckey >> 3) * 2 + chalf) * 8 + (ckey & 7)) * 4;
    const int vdst = (((ckey >> 3) * 2 + (ckey & 1)) * 4 + ((ckey & 7) >> 1)) * 8 + chalf * 4;
    const float* ksrc = K + (b0 + cb) * lay.k_b + hh * lay.k_h + ckey * lay.k_l + chalf * 4;
    const float* vsrc = V + (b0 + cb) * lay.v_b + hh * lay.v_h + ckey * lay.v_l + chalf * 4;
    const int brow = threadIdx.x >> 4, bcol = (threadIdx.x & 15) * 4;
    auto stage_in = [&](int rb, int j0, int buf) {
        float* st = smem + buf * kStage;
        const int row0 = rb * kRows;
        if (Bh) {
            if (bias_vec) {
                const float* bp = Bh + static_cast<size_t>(row0 + brow) * Lk + j0 + bcol;
                float* bd = st + brow * kPitch + bcol;
                const bool col_ok = j0 + bcol < Lk;                     // Lk is a multiple of 4 here
#pragma unroll
                for (int i = 0; i < kRows * 16 / NT; ++i) {
                    const bool ok = col_ok && row0 + brow + i * (NT / 16) < L;
                    cp_async16(bd + i * (NT / 16) * kPitch, ok ? bp : Bh, ok);
                    bp += (NT / 16) * static_cast<size_t>(Lk);
                }
            } else {
                for (int p = threadIdx.x; p < kRows * 64; p += NT) {
                    const int r = p >> 6, c = p & 63;
                    const bool ok = row0 + r < L && j0 + c < Lk;
                    cp_async4(st + r * kPitch + c, ok ? Bh + static_cast<size_t>(row0 + r) * Lk + j0 + c : Bh, ok);
                }
            }
        }
        const bool key_ok = j0 + ckey < Lk;
        const float* kp = ksrc + j0 * lay.k_l;
        const float* vp = vsrc + j0 * lay.v_l;
        if (NT <= 128 || cb < GB) {
#pragma unroll
            for (int bb = 0; bb < GB; bb += (NT + 127) / 128) {
                const bool ok = key_ok && b0 + cb + bb < B;
                cp_async16(st + kBias + (cb + bb) * kKV + kdst, ok ? kp : K, ok);
                cp_async16(st + kBias + (GB + cb + bb) * kKV + vdst, ok ? vp : V, ok);
                kp += ((NT + 127) / 128) * lay.k_b; vp += ((NT + 127) / 128) * lay.v_b;
            }
        }
        if (j0 == 0) {
            // the Q rows of the block: nobody reads the previous block's any more (they are in registers since its start)
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                const int p = threadIdx.x + i * NT, idx = p >> 1, half = p & 1, bb = idx / kRows, r = idx % kRows;
                const bool ok = b0 + bb < B && row0 + r < L;
                cp_async16(smem + 2 * kStage + idx * 8 + half * 4,
                           ok ? Q + (b0 + bb) * lay.q_b + hh * lay.q_h + static_cast<long long>(row0 + r) * lay.q_l + half * 4 : Q, ok);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    auto end_block = [&](int rb) {
        // the gate values first, all loads in flight together (the stores below could alias them for the compiler)
        float gv[2 * MT][2];
#pragma unroll
        for (int r = 0; r < 2 * MT; ++r) {
            const int i = rb * kRows + rg * (16 * MT) + (r >> 1) * 16 + (r & 1) * 8 + g;
            gv[r][0] = gv[r][1] = 0.0f;
            if (lay.gate && b_ok && i < L) {
                const float2* gp = reinterpret_cast<const float2*>(lay.gate + b * lay.g_b + hh * lay.g_h + static_cast<long long>(i) * lay.g_l + 2 * t);
                if ((reinterpret_cast<uintptr_t>(gp) & 7) == 0) { const float2 v = __ldg(gp); gv[r][0] = v.x; gv[r][1] = v.y; }
                else { gv[r][0] = __ldg(reinterpret_cast<const float*>(gp)); gv[r][1] = __ldg(reinterpret_cast<const float*>(gp) + 1); }
            }
        }
#pragma unroll
        for (int r = 0; r < 2 * MT; ++r) {
            const int mi = r >> 1, hr = r & 1;
            float l = lacc[mi][hr * 2];
            const int i = rb * kRows + rg * (16 * MT) + mi * 16 + hr * 8 + g;
            if (!b_ok || i >= L) continue;
            if (ft > 0 && mfirst[r] == -CUDART_INF_F) l = 0.0f;     // the reference's first key tile is fully masked: O = 0, LSE = -inf
            float inv = 0.0f, lse = -CUDART_INF_F;
            if (l > 0.0f) { inv = 1.0f / (l + eps); lse = m[r] + logf(l + eps); }
            float v0 = o[mi][hr * 2] * inv, v1 = o[mi][hr * 2 + 1] * inv;
            if (lay.gate) {
                if (lay.act == 1) {                                 // sigmoid: 1 / (1 + 2^(-x log2 e)) on the fast units
                    v0 *= rcp_approx(1.0f + ex2_approx(-gv[r][0] * kLog2e));
                    v1 *= rcp_approx(1.0f + ex2_approx(-gv[r][1] * kLog2e));
                } else {
                    v0 *= act_scalar(lay.act, gv[r][0]); v1 *= act_scalar(lay.act, gv[r][1]);
                }
            }
            float* op = O + b * lay.o_b + hh * lay.o_h + static_cast<long long>(i) * lay.o_l + 2 * t;
            if ((reinterpret_cast<uintptr_t>(op) & 7) == 0) *reinterpret_cast<float2*>(op) = make_float2(v0, v1);
            else { op[0] = v0; op[1] = v1; }
            if (LSE && t == 0) LSE[(static_cast<size_t>(b) * H + hh) * L + i] = lse;
        }
    };

    stage_in(rb_begin, 0, 0);
    for (int rb = rb_begin, j0 = 0, buf = 0;; buf ^= 1) {
        // the step after this one: the next key tile, or the first of the next row block
        const bool last_tile = j0 + kTile >= keys_of(rb);
        const int rb_next = last_tile ? rb + 1 : rb, j0_next = last_tile ? 0 : j0 + kTile;
        const float* st = smem + buf * kStage;
        const float* bs = st + (rg * (16 * MT) + g) * kPitch + 2 * t;
        const float* ks = st + kBias + bl * kKV + lane;
        const float* vs = st + kBias + (GB + bl) * kKV + t * 8 + g;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        // every thread has left the previous tile (whose stage the next copies overwrite) and sees this tile's copies
        __syncthreads();
        if (j0 == 0) begin_block(rb);
        if (rb_next < rb_end) stage_in(rb_next, j0_next, buf ^ 1);

        float s[MT][8][4];
#pragma unroll
        for (int mi = 0; mi < MT; ++mi)
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                if (Bh) {
                    const float2 lo = *reinterpret_cast<const float2*>(bs + (mi * 16) * kPitch + n * 8);
                    const float2 hi = *reinterpret_cast<const float2*>(bs + (mi * 16 + 8) * kPitch + n * 8);
                    s[mi][n][0] = lo.x; s[mi][n][1] = lo.y; s[mi][n][2] = hi.x; s[mi][n][3] = hi.y;
                } else {
                    s[mi][n][0] = s[mi][n][1] = s[mi][n][2] = s[mi][n][3] = 0.0f;
                }
            }
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            const uint32_t kb0 = tf32_bits(ks[(n * 2) * 32]), kb1 = tf32_bits(ks[(n * 2 + 1) * 32]);
#pragma unroll
            for (int mi = 0; mi < MT; ++mi) mma_tf32(s[mi][n], qa[mi], kb0, kb1);
        }
        // keys past the end (or past the diagonal) of a row; element e of an n tile: key j0 + n * 8 + 2 t + (e & 1)
        int jlow = jmax[0];
#pragma unroll
        for (int r = 1; r < 2 * MT; ++r) jlow = min(jlow, jmax[r]);
        if (j0 + kTile > jlow) {
#pragma unroll
            for (int mi = 0; mi < MT; ++mi)
#pragma unroll
                for (int n = 0; n < 8; ++n)
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (j0 + n * 8 + 2 * t + (e & 1) >= jmax[mi * 2 + (e >> 1)]) s[mi][n][e] = -CUDART_INF_F;
        }
        float alpha[2 * MT], nml2[2 * MT];
#pragma unroll
        for (int r = 0; r < 2 * MT; ++r) {
            const int mi = r >> 1, e0 = (r & 1) * 2;
            float mt = -CUDART_INF_F;
#pragma unroll
            for (int n = 0; n < 8; ++n) mt = fmaxf(mt, fmaxf(s[mi][n][e0], s[mi][n][e0 + 1]));
            mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 1));
            mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 2));
            if (j0 < ft) {                                     // the same for every lane
                if (j0 + kTile <= ft) {
                    mfirst[r] = fmaxf(mfirst[r], mt);
                } else {
                    float mf = -CUDART_INF_F;
#pragma unroll
                    for (int n = 0; n < 8; ++n)
#pragma unroll
                        for (int c = 0; c < 2; ++c)
                            if (j0 + n * 8 + 2 * t + c < ft) mf = fmaxf(mf, s[mi][n][e0 + c]);
                    mf = fmaxf(mf, __shfl_xor_sync(0xffffffffu, mf, 1));
                    mf = fmaxf(mf, __shfl_xor_sync(0xffffffffu, mf, 2));
                    mfirst[r] = fmaxf(mfirst[r], mf);
                }
            }
            const float m_new = fmaxf(m[r], mt);
            // nothing visible so far: alpha = 0 and every probability is 2^-inf = 0, the state stays empty
            alpha[r] = (m[r] == -CUDART_INF_F) ? 0.0f : ex2_approx((m[r] - m_new) * kLog2e);
            nml2[r] = (m_new == -CUDART_INF_F) ? 0.0f : -m_new * kLog2e;
            m[r] = m_new;
        }
#pragma unroll
        for (int mi = 0; mi < MT; ++mi)
#pragma unroll
            for (int n = 0; n < 8; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    s[mi][n][e] = ex2_approx(fmaf(s[mi][n][e], kLog2e, nml2[mi * 2 + (e >> 1)]));
#pragma unroll
        for (int mi = 0; mi < MT; ++mi) {
            o[mi][0] *= alpha[mi * 2]; o[mi][1] *= alpha[mi * 2];
            o[mi][2] *= alpha[mi * 2 + 1]; o[mi][3] *= alpha[mi * 2 + 1];
            lacc[mi][0] *= alpha[mi * 2]; lacc[mi][2] *= alpha[mi * 2 + 1];
        }
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            const uint32_t vb0 = tf32_bits(vs[(n * 2) * 32]), vb1 = tf32_bits(vs[(n * 2 + 1) * 32]);
#pragma unroll
            for (int mi = 0; mi < MT; ++mi) {
                // A fragment of P: (row g, key 2t), (row g + 8, key 2t), (row g, key 2t + 1), (row g + 8, key 2t + 1).  The
                // tensor core drops the low 13 bits of P; the row sum is taken from the same operand (a product with
                // ones), so numerator and denominator see the same P
                const uint32_t pa[4] = {__float_as_uint(s[mi][n][0]), __float_as_uint(s[mi][n][2]), __float_as_uint(s[mi][n][1]),
                                        __float_as_uint(s[mi][n][3])};
                mma_tf32(o[mi], pa, vb0, vb1);
                mma_tf32(lacc[mi], pa, 0x3f800000u, 0x3f800000u);
            }
        }
        if (last_tile) {
            end_block(rb);
            if (rb_next >= rb_end) break;
        }
        rb = rb_next; j0 = j0_next;
    }
}

template <int GB, int NW, int MT>
int launch_shape(const float* Q, const float* K, const float* V, const float* bias, float* O, float* LSE, int B, int H, int L,
                 int Lk, int causal, float scale, float eps, long long bias_batch_stride, int ft, int bias_vec, const AttnLayout& lay,
                 cudaStream_t st) {
    using S = Shape<GB, NW, MT>;
    static bool configured[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return ST_LAUNCH;
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(attn_d8_mma_kernel<GB, NW, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::smem_bytes) != cudaSuccess)
            return ST_LAUNCH;
        configured[dev] = true;
    }
    // a CTA takes several consecutive row blocks (its copies run ahead across them) as long as the grid keeps about eight
    // waves of CTAs
    const int n_blocks = (L + S::rows - 1) / S::rows, groups = (B + GB - 1) / GB;
    const long long ctas_wanted = 8LL * num_sms() * (GB == 4 ? (MT == 2 ? 16 : 24) / NW : 2);
    long long split = (ctas_wanted + static_cast<long long>(H) * groups - 1) / (static_cast<long long>(H) * groups);
    if (split > n_blocks) split = n_blocks;
    if (split < 1) split = 1;
    const int per_cta = static_cast<int>((n_blocks + split - 1) / split);
    dim3 grid((n_blocks + per_cta - 1) / per_cta, H, groups);
    attn_d8_mma_kernel<GB, NW, MT><<<grid, 32 * NW, S::smem_bytes, st>>>(Q, K, V, bias, O, LSE, B, H, L, Lk, causal, scale, eps,
                                                                    bias_batch_stride, ft, bias_vec, per_cta, lay);
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_LAUNCH;
}

}  // namespace

int launch_attn_d8_mma(const float* Q, const float* K, const float* V, const float* bias, float* O, float* LSE, int B, int H,
                       int L, int Lk, int d, int causal, float scale, float eps, long long bias_batch_stride, int ft,
                       const AttnLayout& lay, cudaStream_t st) {
    if (d != 8 || L < 16 || H > 65535) return ST_UNSUPPORTED_PATH;
    // 16-byte copies of the 32-byte Q / K / V rows
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (!al16(Q) || !al16(K) || !al16(V) ||
        ((lay.q_b | lay.q_h | lay.q_l | lay.k_b | lay.k_h | lay.k_l | lay.v_b | lay.v_h | lay.v_l) & 3) != 0) return ST_UNSUPPORTED_PATH;
    const bool shared = bias == nullptr || bias_batch_stride == 0;
    const int bias_vec = bias != nullptr && (Lk & 3) == 0 && (bias_batch_stride & 3) == 0 && al16(bias);
    if (shared && B >= 4) {
        if ((B + 3) / 4 > 65535) return ST_UNSUPPORTED_PATH;
        if (L > 32)
            return launch_shape<4, 8, 2>(Q, K, V, bias, O, LSE, B, H, L, Lk, causal, scale, eps, bias_batch_stride, ft, bias_vec, lay, st);
        return launch_shape<4, 4, 2>(Q, K, V, bias, O, LSE, B, H, L, Lk, causal, scale, eps, bias_batch_stride, ft, bias_vec, lay, st);
    }
    if (B > 65535) return ST_UNSUPPORTED_PATH;
    return launch_shape<1, 4, 2>(Q, K, V, bias, O, LSE, B, H, L, Lk, causal, scale, eps, bias_batch_stride, ft, bias_vec, lay, st);
}

}  // namespace ppml_b200
