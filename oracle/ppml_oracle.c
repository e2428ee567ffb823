/*
 * ppml_oracle.c -- CPU restatement of the reference's dense-contraction path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the product library links, loads or
 * calls this file; only the test-suite, the smoke check and the CPU-baseline
 * leg of the benchmark do, and there only as the checker / the timed baseline.
 *
 * Every function is a plain-C restatement of one reference routine; the
 * reference location (path inside the reference project : lines) is given in
 * the comment above it.  Loop order and the order of floating-point operations
 * follow the reference so that fp32 results agree to rounding.
 *
 * Parity status: pinned.  tests/test_oracle.py checks each function against
 * (1) the known-answer vectors of the reference's own unit tests
 *     (tests/test_cuda.cpp MulMat / OutProd) and
 * (2) fixtures produced by running the reference's unmodified CPU sources
 *     (compiled by oracle/Makefile into oracle/_ref/) on seeded inputs
 *     (tests/golden/*.npz, made by tests/golden/make_golden.py).
 * The Q8 mul_mat has no CPU kernel in the reference; its restatement follows
 * the CUDA kernel's arithmetic line by line and is pinned only through the
 * reference's host quantizers (bit-exact) and a dequantize-then-fp32 bound.
 *
 * Build: gcc -O2 -fPIC -shared -std=c99 -ffp-contract=off ppml_oracle.c -lm
 *        (-ffp-contract=off keeps a*b+c as two roundings like the reference's
 *        x86-64 -O2 build).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define QK 32

/* ------------------------------------------------------------------ */
/* fp16 <-> fp32, round-to-nearest-even, full subnormal/inf/nan support */
/* (semantics of include/ppml/HalfUtils.h:26-52 and of __float2half)   */
/* ------------------------------------------------------------------ */
static uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

uint16_t oracle_f32_to_f16(float f) {
    uint32_t x = f2u(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7fffffffu;
    if (ax > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);          /* NaN */
    if (ax >= 0x47800000u) {                                          /* >= 65536: may round to inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (ax >= 0x38800000u) {                                          /* normal half */
        uint32_t mant = ax & 0x7fffffu;
        uint32_t exp = (ax >> 23) - 112u;
        uint32_t h = (exp << 10) | (mant >> 13);
        uint32_t rem = mant & 0x1fffu;
        if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h++;       /* carry may reach inf: correct */
        return (uint16_t)(sign | h);
    }
    if (ax < 0x33000000u) return (uint16_t)sign;                      /* < 2^-25 -> 0 */
    {                                                                 /* subnormal half */
        uint32_t e = ax >> 23;                                        /* 102..112 */
        uint32_t mant = (ax & 0x7fffffu) | 0x800000u;
        uint32_t shift = 126u - e;                                    /* 14..24 */
        uint32_t h = mant >> shift;
        uint32_t rem = mant & ((1u << shift) - 1u);
        uint32_t half = 1u << (shift - 1u);
        if (rem > half || (rem == half && (h & 1u))) h++;
        return (uint16_t)(sign | h);
    }
}

float oracle_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t mant = h & 0x3ffu;
    if (exp == 0) {
        if (mant == 0) return u2f(sign);
        {
            float v = (float)mant * 5.9604644775390625e-8f;           /* 2^-24 */
            return sign ? -v : v;
        }
    }
    if (exp == 31) return u2f(sign | 0x7f800000u | (mant << 13));
    return u2f(sign | ((exp + 112u) << 23) | (mant << 13));
}

/* bf16 (new dtype, no reference counterpart): round-to-nearest-even */
uint16_t oracle_f32_to_bf16(float f) {
    uint32_t x = f2u(f);
    if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x40u);
    x += 0x7fffu + ((x >> 16) & 1u);
    return (uint16_t)(x >> 16);
}
float oracle_bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }

/* ------------------------------------------------------------------ */
/* mul_mat fp32: C[m,n] = bias[n] + sum_k A[m,k]*B[n,k], k ascending,  */
/* accumulator seeded with the bias.                                   */
/* src/backend/CPUKernels.cpp:763-771                                  */
/* ------------------------------------------------------------------ */
void oracle_mul_mat_f32(const float* a, const float* b, const float* bias, float* c,
                        int M, int K, int N) {
    for (int i = 0; i < M; i++) {
        for (int j = 0; j < N; j++) {
            float sum = bias ? bias[j] : 0.0f;
            for (int k = 0; k < K; k++) sum += a[(size_t)i * K + k] * b[(size_t)j * K + k];
            c[(size_t)j + (size_t)i * N] = sum;
        }
    }
}

/* mul_mat with 16-bit half operands, fp32 accumulate, bias added AFTER the dot.
 * src/backend/CPUKernels.cpp:392-396 (dot_half_row_soft), :655-668 */
void oracle_mul_mat_f16(const uint16_t* a, const uint16_t* b, const float* bias, float* c,
                        int M, int K, int N) {
    for (int i = 0; i < M; i++) {
        for (int j = 0; j < N; j++) {
            float acc = 0.f;
            for (int k = 0; k < K; k++)
                acc += oracle_f16_to_f32(a[(size_t)i * K + k]) * oracle_f16_to_f32(b[(size_t)j * K + k]);
            c[(size_t)j + (size_t)i * N] = bias ? (acc + bias[j]) : acc;
        }
    }
}

/* bf16 operands (new dtype): same loop as the half path, bias after the dot. */
void oracle_mul_mat_bf16(const uint16_t* a, const uint16_t* b, const float* bias, float* c,
                         int M, int K, int N) {
    for (int i = 0; i < M; i++) {
        for (int j = 0; j < N; j++) {
            float acc = 0.f;
            for (int k = 0; k < K; k++)
                acc += oracle_bf16_to_f32(a[(size_t)i * K + k]) * oracle_bf16_to_f32(b[(size_t)j * K + k]);
            c[(size_t)j + (size_t)i * N] = bias ? (acc + bias[j]) : acc;
        }
    }
}

/* ------------------------------------------------------------------ */
/* out_prod: dst[i0,i1,i2,i3] = sum_k s0[i0,k,i2/dps2,i3/dps3]*s1[i1,k,i2,i3]
 * dst zeroed first, k ascending, accumulated straight into dst.
 * src/backend/CPUKernels.cpp:787-887                                  */
/* ------------------------------------------------------------------ */
void oracle_out_prod(const float* s0, const float* s1, float* dst,
                     int64_t ne00, int64_t ne01, int64_t ne02, int64_t ne03,
                     int64_t ne10, int64_t ne11, int64_t ne12, int64_t ne13,
                     int64_t ne0, int64_t ne1, int64_t ne2, int64_t ne3) {
    (void)ne13;
    for (int64_t i = 0; i < ne0 * ne1 * ne2 * ne3; i++) dst[i] = 0.0f;
    const int64_t nr = ne1 * ne2 * ne3;
    const int64_t dps2 = ne2 / ne02, dps3 = ne3 / ne03;
    for (int64_t ir = 0; ir < nr; ir++) {
        const int64_t i3 = ir / (ne2 * ne1);
        const int64_t i2 = (ir - i3 * ne2 * ne1) / ne1;
        const int64_t i1 = ir - i3 * ne2 * ne1 - i2 * ne1;
        const int64_t i02 = i2 / dps2, i03 = i3 / dps3;
        float* d_row = dst + (i1 * ne0 + i2 * ne0 * ne1 + i3 * ne0 * ne1 * ne2);
        for (int64_t i01 = 0; i01 < ne01; i01++) {
            const float* a = s0 + (i01 * ne00 + i02 * ne00 * ne01 + i03 * ne00 * ne01 * ne02);
            const float* b = s1 + (i01 * ne10 + i2 * ne10 * ne11 + i3 * ne10 * ne11 * ne12);
            const float v = b[i1];
            for (int64_t i0 = 0; i0 < ne00; i0++) d_row[i0] += a[i0] * v;
        }
    }
}

/* ------------------------------------------------------------------ */
/* tri_mul: flat layout [D][I][K][B] with D outermost and B innermost.
 * outgoing: dst[d,i,j,b] = (1/L) sum_k left[d,i,k,b]*right[d,j,k,b]
 * incoming: dst[d,i,j,b] = (1/L) sum_k left[d,k,i,b]*right[d,k,j,b]
 * NaN -> 0, clamp to +-1e4.   src/backend/CPUKernels.cpp:907-970      */
/* ------------------------------------------------------------------ */
void oracle_tri_mul(const float* left, const float* right, float* dst,
                    int64_t D, int64_t I, int64_t J, int64_t K, int64_t B,
                    float L, int outgoing) {
    const float inv_L = 1.0f / L;
    const int64_t total = B * I * J * D;
    for (int64_t idx = 0; idx < total; idx++) {
        int64_t tmp = idx;
        int64_t b = tmp % B; tmp /= B;
        int64_t j = tmp % J; tmp /= J;
        int64_t i = tmp % I;
        int64_t d = tmp / I;
        float sum = 0.0f;
        if (outgoing) {
            for (int64_t k = 0; k < K; k++)
                sum += left[((d * I + i) * K + k) * B + b] * right[((d * J + j) * K + k) * B + b];
        } else {
            for (int64_t k = 0; k < K; k++)
                sum += left[((d * K + k) * I + i) * B + b] * right[((d * K + k) * J + j) * B + b];
        }
        float v = sum * inv_L;
        if (!(v == v) || v > 1e4f || v < -1e4f) v = (v != v) ? 0.0f : (v > 1e4f ? 1e4f : -1e4f);
        dst[idx] = v;
    }
}

/* ------------------------------------------------------------------ */
/* outer_prod_mean: flat [D][L][N][B];
 * dst[(d1*D+d2),i,j,b] = (1/N) sum_n left[d1,i,n,b]*right[d2,j,n,b]
 * src/backend/CPUKernels.cpp:982-1032                                 */
/* ------------------------------------------------------------------ */
void oracle_outer_prod_mean(const float* left, const float* right, float* dst,
                            int64_t D, int64_t L, int64_t N, int64_t B) {
    const float inv_N = 1.0f / (float)N;
    const int64_t total = D * D * L * L * B;
    for (int64_t idx = 0; idx < total; idx++) {
        int64_t tmp = idx;
        int64_t b = tmp % B; tmp /= B;
        int64_t j = tmp % L; tmp /= L;
        int64_t i = tmp % L; tmp /= L;
        int64_t d2 = tmp % D; tmp /= D;
        int64_t d1 = tmp;
        float sum = 0.0f;
        for (int64_t n = 0; n < N; n++)
            sum += left[((d1 * L + i) * N + n) * B + b] * right[((d2 * L + j) * N + n) * B + b];
        dst[idx] = sum * inv_N;
    }
}

/* ------------------------------------------------------------------ */
/* flash attention forward, blocked online softmax over key tiles of Bc.
 * Q/K/V/O [d,L,h,B] (d innermost), bias [Lk,Lq,h,B], LSE [L,h,B].
 * src/ops/FlashAttn.cpp:51-135.  `Lk` extends the reference (which has
 * L only, include/ppml/FlashAttn.h:26-36): pass Lk == L for the
 * reference's behaviour.                                              */
/* ------------------------------------------------------------------ */
int oracle_flash_attn_forward(int B, int H, int L, int Lk, int d, int causal, float scale,
                              float eps, int Bc,
                              const float* Q, const float* K, const float* V, const float* bias,
                              int64_t bias_batch_stride, float* O, float* LSE) {
    if (!Q || !K || !V || !O) return 0;
    if (B <= 0 || H <= 0 || L <= 0 || Lk <= 0 || d <= 0) return 0;
    if (Bc <= 0) Bc = 64;
    const float sc = (scale > 0.f) ? scale : 1.0f / sqrtf((float)d);
    float* acc = (float*)malloc(sizeof(float) * (size_t)d);
    float* s_tile = (float*)malloc(sizeof(float) * (size_t)Bc);
    for (int b = 0; b < B; ++b) {
        for (int hh = 0; hh < H; ++hh) {
            const float* Qb = Q + ((size_t)b * H + hh) * (size_t)L * d;
            const float* Kb = K + ((size_t)b * H + hh) * (size_t)Lk * d;
            const float* Vb = V + ((size_t)b * H + hh) * (size_t)Lk * d;
            float* Ob = O + ((size_t)b * H + hh) * (size_t)L * d;
            float* Lb = LSE ? LSE + ((size_t)b * H + hh) * (size_t)L : NULL;
            const float* Bb = bias ? bias + (size_t)b * (size_t)bias_batch_stride
                                            + (size_t)hh * (size_t)L * (size_t)Lk : NULL;
            for (int i = 0; i < L; ++i) {
                const float* q = Qb + (size_t)i * d;
                const int jmax = causal ? ((i + 1 < Lk) ? i + 1 : Lk) : Lk;
                float m = -INFINITY, l = 0.f;
                for (int dd = 0; dd < d; ++dd) acc[dd] = 0.f;
                for (int j0 = 0; j0 < jmax; j0 += Bc) {
                    const int j1 = (j0 + Bc < jmax) ? j0 + Bc : jmax;
                    const int nb = j1 - j0;
                    float m_tile = -INFINITY;
                    for (int j = j0; j < j1; ++j) {
                        const float* k = Kb + (size_t)j * d;
                        float s = 0.f;
                        for (int dd = 0; dd < d; ++dd) s += q[dd] * k[dd];
                        s *= sc;
                        if (Bb) s += Bb[(size_t)i * Lk + j];
                        s_tile[j - j0] = s;
                        if (s > m_tile) m_tile = s;
                    }
                    const float m_new = (m > m_tile) ? m : m_tile;
                    const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
                    float l_tile = 0.f;
                    for (int j = 0; j < nb; ++j) {
                        const float p = expf(s_tile[j] - m_new);
                        s_tile[j] = p;
                        l_tile += p;
                    }
                    for (int dd = 0; dd < d; ++dd) {
                        float pv = 0.f;
                        for (int j = 0; j < nb; ++j) pv += s_tile[j] * Vb[(size_t)(j0 + j) * d + dd];
                        acc[dd] = alpha * acc[dd] + pv;
                    }
                    l = alpha * l + l_tile;
                    m = m_new;
                }
                float* o = Ob + (size_t)i * d;
                if (l > 0.f) {
                    const float inv = 1.0f / (l + eps);
                    for (int dd = 0; dd < d; ++dd) o[dd] = acc[dd] * inv;
                    if (Lb) Lb[i] = m + logf(l + eps);
                } else {
                    for (int dd = 0; dd < d; ++dd) o[dd] = 0.f;
                    if (Lb) Lb[i] = -INFINITY;
                }
            }
        }
    }
    free(acc); free(s_tile);
    return 1;
}

/* ------------------------------------------------------------------ */
/* flash attention backward, row by row as the reference's CPU routine
 * (src/ops/FlashAttn.cpp:144-216; formulas include/ppml/FlashAttn.h:66-75):
 *   P_ij  = exp(S_ij - LSE_i)   (LSE holds the eps of the forward)
 *   D_i   = sum_d dO_id O_id ;  dP_ij = sum_d dO_id V_jd ;  dS_ij = P_ij (dP_ij - D_i)
 *   dQ_id = scale sum_j dS_ij K_jd ; dK_jd = scale sum_i dS_ij Q_id ; dV_jd = sum_i P_ij dO_id
 *   dbias_ij = dS_ij (masked positions and fully masked rows: 0)
 * Q/K/V/O/dO/dQ/dK/dV [d,L,h,B] (d innermost), bias read with a batch stride
 * (0: one [h,L,L] bias for every batch), dbias always [B,h,L,L], LSE [L,h,B].
 * Outputs are zeroed first; a null output is skipped.                  */
/* ------------------------------------------------------------------ */
int oracle_flash_attn_backward(int B, int H, int L, int d, int causal, float scale,
                               const float* Q, const float* K, const float* V, const float* bias,
                               int64_t bias_batch_stride, const float* O, const float* dO, const float* LSE,
                               float* dQ, float* dK, float* dV, float* dbias) {
    if (!Q || !K || !V || !O || !dO || !LSE) return 0;
    if (B <= 0 || H <= 0 || L <= 0 || d <= 0) return 0;
    if (!dQ && !dK && !dV && !dbias) return 0;
    const float sc = (scale > 0.f) ? scale : 1.0f / sqrtf((float)d);
    const size_t nq = (size_t)B * H * L * d, nb = (size_t)B * H * L * L;
    if (dQ) memset(dQ, 0, nq * sizeof(float));
    if (dK) memset(dK, 0, nq * sizeof(float));
    if (dV) memset(dV, 0, nq * sizeof(float));
    if (dbias) memset(dbias, 0, nb * sizeof(float));
    for (int b = 0; b < B; ++b) {
        for (int hh = 0; hh < H; ++hh) {
            const size_t base = ((size_t)b * H + hh) * (size_t)L * d;
            const float* Lb = LSE + ((size_t)b * H + hh) * (size_t)L;
            const float* Bb = bias ? bias + (size_t)b * (size_t)bias_batch_stride + (size_t)hh * L * L : NULL;
            float* dBb = dbias ? dbias + ((size_t)b * H + hh) * (size_t)L * L : NULL;
            for (int i = 0; i < L; ++i) {
                const float lse = Lb[i];
                if (!(lse > -INFINITY)) continue;
                const float* q = Q + base + (size_t)i * d;
                const float* o_row = O + base + (size_t)i * d;
                const float* do_row = dO + base + (size_t)i * d;
                float D = 0.f;
                for (int dd = 0; dd < d; ++dd) D += do_row[dd] * o_row[dd];
                const int jmax = causal ? (i + 1) : L;
                for (int j = 0; j < jmax; ++j) {
                    const float* k = K + base + (size_t)j * d;
                    const float* v = V + base + (size_t)j * d;
                    float s = 0.f;
                    for (int dd = 0; dd < d; ++dd) s += q[dd] * k[dd];
                    s *= sc;
                    if (Bb) s += Bb[(size_t)i * L + j];
                    const float p = expf(s - lse);
                    float dp = 0.f;
                    for (int dd = 0; dd < d; ++dd) dp += do_row[dd] * v[dd];
                    const float ds = p * (dp - D);
                    if (dBb) dBb[(size_t)i * L + j] = ds;
                    if (dQ) for (int dd = 0; dd < d; ++dd) dQ[base + (size_t)i * d + dd] += sc * ds * k[dd];
                    if (dK) for (int dd = 0; dd < d; ++dd) dK[base + (size_t)j * d + dd] += sc * ds * q[dd];
                    if (dV) for (int dd = 0; dd < d; ++dd) dV[base + (size_t)j * d + dd] += p * do_row[dd];
                }
            }
        }
    }
    return 1;
}

/* The legacy unfused attention path, the semantic ground truth for Lq != Lk:
 *   scores[j,i] = sum_d K[j,d]*Q[i,d]      (out_prod, src/modules/Attention.cpp:267)
 *   scores *= scale ; scores += bias       (:269-272)
 *   P = exp(s - max) * (1/(sum + 1e-9))    (kernel_softmax, src/backend/CPUKernels.cpp:1446-1467)
 *   O[i,d] = sum_j P[i,j]*V[j,d]           (second out_prod, :279-283)
 * Layout as in oracle_flash_attn_forward. */
void oracle_attention_legacy(int B, int H, int Lq, int Lk, int d, float scale,
                             const float* Q, const float* K, const float* V, const float* bias,
                             int64_t bias_batch_stride, float* O) {
    float* s = (float*)malloc(sizeof(float) * (size_t)Lk);
    for (int b = 0; b < B; ++b) for (int hh = 0; hh < H; ++hh) {
        const float* Qb = Q + ((size_t)b * H + hh) * (size_t)Lq * d;
        const float* Kb = K + ((size_t)b * H + hh) * (size_t)Lk * d;
        const float* Vb = V + ((size_t)b * H + hh) * (size_t)Lk * d;
        float* Ob = O + ((size_t)b * H + hh) * (size_t)Lq * d;
        const float* Bb = bias ? bias + (size_t)b * (size_t)bias_batch_stride
                                        + (size_t)hh * (size_t)Lq * (size_t)Lk : NULL;
        for (int i = 0; i < Lq; ++i) {
            for (int j = 0; j < Lk; ++j) {
                float acc = 0.f;
                for (int dd = 0; dd < d; ++dd) acc += Kb[(size_t)j * d + dd] * Qb[(size_t)i * d + dd];
                acc = acc * scale;
                if (Bb) acc = acc + Bb[(size_t)i * Lk + j];
                s[j] = acc;
            }
            float mx = s[0];
            for (int j = 1; j < Lk; ++j) if (s[j] > mx) mx = s[j];
            float sum = 0.f;
            for (int j = 0; j < Lk; ++j) sum += expf(s[j] - mx);
            const float inv = 1.0f / (sum + 1e-9f);
            for (int j = 0; j < Lk; ++j) s[j] = expf(s[j] - mx) * inv;
            for (int dd = 0; dd < d; ++dd) {
                float acc = 0.f;
                for (int j = 0; j < Lk; ++j) acc += s[j] * Vb[(size_t)j * d + dd];
                Ob[(size_t)i * d + dd] = acc;
            }
        }
    }
    free(s);
}

/* ------------------------------------------------------------------ */
/* Q8 block quantizers.  include/ppml/QuantBlocks.h:62-79 (Q8_0),
 * :81-111 (Q8_1), :128-135 (Q8_0R repack).
 * Q8_0 interleaved block = { fp16 d; int8 qs[32] }   (34 bytes)
 * Q8_1 interleaved block = { fp16 d; fp16 s; int8 qs[32] } (36 bytes)
 * Q8_0R = [nblocks*32 int8 qs][nblocks fp16 d]                        */
/* ------------------------------------------------------------------ */
int oracle_quantize_q8_0(const float* src, uint8_t* dst, int64_t n) {
    if (n % QK) return 0;
    const int64_t nb = n / QK;
    for (int64_t b = 0; b < nb; ++b) {
        const float* x = src + b * QK;
        float amax = 0.f;
        for (int i = 0; i < QK; ++i) amax = fmaxf(amax, fabsf(x[i]));
        const float d = amax / 127.0f;
        const float inv = (amax == 0.0f) ? 0.0f : 1.0f / d;
        uint16_t hd = oracle_f32_to_f16(d);
        uint8_t* blk = dst + b * 34;
        memcpy(blk, &hd, 2);
        for (int i = 0; i < QK; ++i) {
            float q = roundf(x[i] * inv);
            q = q > 127.0f ? 127.0f : (q < -127.0f ? -127.0f : q);
            ((int8_t*)blk)[2 + i] = (int8_t)q;
        }
    }
    return 1;
}

int oracle_quantize_q8_1(const float* src, uint8_t* dst, int64_t n) {
    if (n % QK) return 0;
    const int64_t nb = n / QK;
    for (int64_t b = 0; b < nb; ++b) {
        const float* x = src + b * QK;
        float amax = 0.f, vmax = 0.f;
        for (int i = 0; i < QK; ++i) {
            const float v = x[i];
            if (fabsf(v) > amax) { amax = fabsf(v); vmax = v; }
        }
        const float d = (amax == 0.0f) ? 0.0f : vmax / -128.0f;
        const float inv = (d == 0.0f) ? 0.0f : 1.0f / d;
        int32_t qsum = 0;
        uint8_t* blk = dst + b * 36;
        for (int i = 0; i < QK; ++i) {
            float q = roundf(x[i] * inv);
            q = q > 127.0f ? 127.0f : (q < -128.0f ? -128.0f : q);
            const int8_t qi = (int8_t)q;
            ((int8_t*)blk)[4 + i] = qi;
            qsum += qi;
        }
        uint16_t hd = oracle_f32_to_f16(d);
        uint16_t hs = oracle_f32_to_f16(d * (float)qsum);
        memcpy(blk, &hd, 2);
        memcpy(blk + 2, &hs, 2);
    }
    return 1;
}

void oracle_repack_q8_0(const uint8_t* src, int64_t nblocks, uint8_t* dst) {
    uint8_t* qs = dst;
    uint8_t* d = dst + nblocks * QK;
    for (int64_t b = 0; b < nblocks; ++b) {
        memcpy(qs + b * QK, src + b * 34 + 2, QK);
        memcpy(d + b * 2, src + b * 34, 2);
    }
}

void oracle_dequantize_q8_0(const uint8_t* src, float* dst, int64_t n) {
    const int64_t nb = n / QK;
    for (int64_t b = 0; b < nb; ++b) {
        uint16_t hd; memcpy(&hd, src + b * 34, 2);
        const float d = oracle_f16_to_f32(hd);
        for (int i = 0; i < QK; ++i) dst[b * QK + i] = d * (float)((const int8_t*)src)[b * 34 + 2 + i];
    }
}

void oracle_dequantize_q8_1(const uint8_t* src, float* dst, int64_t n) {
    const int64_t nb = n / QK;
    for (int64_t b = 0; b < nb; ++b) {
        uint16_t hd; memcpy(&hd, src + b * 36, 2);
        const float d = oracle_f16_to_f32(hd);
        for (int i = 0; i < QK; ++i) dst[b * QK + i] = d * (float)((const int8_t*)src)[b * 36 + 4 + i];
    }
}

/* ------------------------------------------------------------------ */
/* Q8 mul_mat (W8A8).  The reference has no CPU kernel for it
 * (include/ppml/QuantBlocks.h:56); this restates the CUDA kernel
 * mul_mat_vec_q8_kernel, src/cuda/MulMatQ8Kernel.cu:109-145, and its
 * host launcher :476-547:
 *   activations X[N][K] fp32 are quantized per 32-block to Q8_1,
 *   per block: sumi = sum_32 qw*qa (int32);
 *              acc += (float)sumi * (d_w * d_a)   in block order.
 * W: wtype 0 = Q8_0 interleaved, 1 = Q8_1 interleaved, 2 = Q8_0R planes;
 *    M rows (out features) of K.   c_trans 0: C[m*N+n]; 1: C[n*M+m].
 * bias (extension, may be NULL): added after the last block, bias[m].
 * sumi_out (may be NULL): int32 [N][M][K/32] block sums for exact checks.
 * returns 0 ok, 1 bad args, 2 K%32, 5 wtype                           */
/* ------------------------------------------------------------------ */
int oracle_mul_mat_q8(const void* W, const float* X, float* C, int M, int N, int K,
                      int wtype, int c_trans, const float* bias, int32_t* sumi_out) {
    if (!W || !X || !C || M <= 0 || N <= 0 || K <= 0) return 1;
    if (K % QK) return 2;
    if (wtype < 0 || wtype > 2) return 5;
    const int nblk = K / QK;
    uint8_t* qa = (uint8_t*)malloc((size_t)N * nblk * 36);
    oracle_quantize_q8_1(X, qa, (int64_t)N * K);
    const uint8_t* w = (const uint8_t*)W;
    const size_t nb_all = (size_t)M * nblk;
    for (int n = 0; n < N; ++n) {
        for (int m = 0; m < M; ++m) {
            float acc = 0.0f;
            for (int ib = 0; ib < nblk; ++ib) {
                const int8_t* qw; uint16_t hdw;
                const size_t blk = (size_t)m * nblk + ib;
                if (wtype == 2) { qw = (const int8_t*)(w + blk * QK); memcpy(&hdw, w + nb_all * QK + blk * 2, 2); }
                else if (wtype == 0) { qw = (const int8_t*)(w + blk * 34 + 2); memcpy(&hdw, w + blk * 34, 2); }
                else { qw = (const int8_t*)(w + blk * 36 + 4); memcpy(&hdw, w + blk * 36, 2); }
                const uint8_t* ab = qa + ((size_t)n * nblk + ib) * 36;
                uint16_t hda; memcpy(&hda, ab, 2);
                const int8_t* qx = (const int8_t*)(ab + 4);
                int32_t sumi = 0;
                for (int j = 0; j < QK; ++j) sumi += (int32_t)qw[j] * (int32_t)qx[j];
                if (sumi_out) sumi_out[((size_t)n * M + m) * nblk + ib] = sumi;
                acc += (float)sumi * (oracle_f16_to_f32(hdw) * oracle_f16_to_f32(hda));
            }
            if (bias) acc += bias[m];
            if (c_trans) C[(size_t)n * M + m] = acc; else C[(size_t)m * N + n] = acc;
        }
    }
    free(qa);
    return 0;
}
