// umma_gemm.cu -- host side of the tcgen05 contraction engine: eligibility checks, tensor maps,
// tile shape selection and the launch.
#include <cstdlib>
#include "kernels.h"
#include "tma_host.h"
#include "umma_gemm.cuh"

namespace ppml_b200 {

int num_sms() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

namespace {

template <MmaKind KIND, int BN, Epi EPI, bool CONVERT, bool MNMAJOR = false>
int launch_one(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmParams p, cudaStream_t st) {
    auto kern = umma_gemm_kernel<KIND, BN, EPI, CONVERT, MNMAJOR>;
    constexpr int smem = gemm_smem_bytes<BN>();
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
            cudaGetLastError();
            return ST_LAUNCH;
        }
        configured[dev] = true;
    }
    p.n_tiles = (p.N + BN - 1) / BN;
    p.m_tiles = (p.M + 127) / 128;
    const long long total = static_cast<long long>(p.m_tiles) * p.n_tiles * p.batch;
    if (total <= 0 || total > 0x7fffffffLL) return ST_BAD_ARGS;
    const int grid = static_cast<int>(total < num_sms() ? total : num_sms());
    // equal row ranges per CTA instead of whole tiles dealt round robin, when the tiles do not divide evenly
    static const int flat_env = [] { const char* e = std::getenv("PPML_B200_GEMM_FLAT"); return e ? (e[0] != '0' ? 1 : 0) : 1; }();
    // (one column tile only: with several, a partial row tile costs every one of them and the round robin balances better;
    // measured at M = 65536: 36.5 -> 35.0 us at 256 x 256 tf32, 31.9 -> 31.3 at 128 x 256, but 57 -> 63 at 256 x 512)
    // (and short contractions only: at K = 1024 the partial tile costs more tensor and L2 time than the balance gains,
    // 75 -> 80 us at 65536 x 1024 x 256)
    p.flat_rows = (flat_env && p.batch == 1 && !MNMAJOR && EPI != Epi::OPM_BLOCKED && p.n_tiles == 1 && p.k_steps <= 8 &&
                   p.m_tiles > grid && p.m_tiles % grid != 0) ? 1 : 0;
    kern<<<grid, CONVERT ? 320 : 192, smem, st>>>(tmA, tmB, p);
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_LAUNCH;
}

template <MmaKind KIND, Epi EPI, bool CONVERT>
int launch_bn(int BN, const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, cudaStream_t st) {
    switch (BN) {
        case 32: return launch_one<KIND, 32, EPI, CONVERT>(tmA, tmB, p, st);
        case 64: return launch_one<KIND, 64, EPI, CONVERT>(tmA, tmB, p, st);
        case 128: return launch_one<KIND, 128, EPI, CONVERT>(tmA, tmB, p, st);
        default: return launch_one<KIND, 256, EPI, CONVERT>(tmA, tmB, p, st);
    }
}

int launch_bn_mn(int BN, bool half, const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, cudaStream_t st) {
    if (half) {
        switch (BN) {
            case 32: case 64: return launch_one<MmaKind::F16, 64, Epi::ROW_MAJOR, false, true>(tmA, tmB, p, st);
            case 128: return launch_one<MmaKind::F16, 128, Epi::ROW_MAJOR, false, true>(tmA, tmB, p, st);
            default: return launch_one<MmaKind::F16, 256, Epi::ROW_MAJOR, false, true>(tmA, tmB, p, st);
        }
    }
    switch (BN) {
        case 32: return launch_one<MmaKind::TF32, 32, Epi::ROW_MAJOR, false, true>(tmA, tmB, p, st);
        case 64: return launch_one<MmaKind::TF32, 64, Epi::ROW_MAJOR, false, true>(tmA, tmB, p, st);
        case 128: return launch_one<MmaKind::TF32, 128, Epi::ROW_MAJOR, false, true>(tmA, tmB, p, st);
        default: return launch_one<MmaKind::TF32, 256, Epi::ROW_MAJOR, false, true>(tmA, tmB, p, st);
    }
}

int pick_bn(int N) {
    if (N <= 32) return 32;
    if (N <= 64) return 64;
    if (N <= 128) return 128;
    return 256;
}

}  // namespace

int launch_umma_gemm(const UmmaGemmArgs& a, cudaStream_t st) {
    if (!a.A || !a.B || !a.C || a.M <= 0 || a.N <= 0 || a.K <= 0 || a.batch <= 0) return ST_BAD_ARGS;
    const int es = (a.elem == 0) ? 4 : 2;
    // TMA: 16-byte aligned bases and strides; otherwise the CUDA-core kernel takes the call
    if ((reinterpret_cast<uintptr_t>(a.A) & 15u) || (reinterpret_cast<uintptr_t>(a.B) & 15u)) return ST_UNSUPPORTED_PATH;
    if ((a.lda * es) % 16 || (a.ldb * es) % 16 || (a.a_batch * es) % 16 || (a.b_batch * es) % 16) return ST_UNSUPPORTED_PATH;
    if (a.batch > 1 && (a.a_batch == 0 || a.b_batch == 0)) return ST_UNSUPPORTED_PATH;
    int* err = device_error_ptr();
    if (!err) return ST_LAUNCH;

    const int BN = pick_bn(a.N);
    const int bk = 128 / es;
    if (a.mn_major) {
        // A[b][k][m], B[b][k][n] with the row index contiguous: fp32 operands become tf32 in the TMA unit and use
        // the 32-byte-chunk swizzle, 16-bit operands the ordinary 128-byte swizzle
        if (a.opm_L > 0) return ST_UNSUPPORTED_PATH;
        CUtensorMap tmA, tmB;
        const bool half = a.elem != 0;
        const TmaType tt = !half ? TmaType::TF32 : (a.elem == 1 ? TmaType::F16 : TmaType::BF16);
        const uint32_t box = half ? 64 : 32;
        const uint64_t a_bs = (a.batch > 1) ? static_cast<uint64_t>(a.a_batch) * es : 0;
        const uint64_t b_bs = (a.batch > 1) ? static_cast<uint64_t>(a.b_batch) * es : 0;
        if (!make_tmap_3d(&tmA, tt, a.A, a.M, a.K, a.batch, static_cast<uint64_t>(a.lda) * es, a_bs, box, box, half ? 1 : 2))
            return ST_UNSUPPORTED_PATH;
        if (!make_tmap_3d(&tmB, tt, a.B, a.N, a.K, a.batch, static_cast<uint64_t>(a.ldb) * es, b_bs, box, box, half ? 1 : 2))
            return ST_UNSUPPORTED_PATH;
        GemmParams p{};
        p.M = a.M; p.N = a.N; p.K = a.K; p.batch = a.batch;
        p.k_steps = (a.K + bk - 1) / bk;
        p.ab_fmt = (a.elem == 2) ? 1 : 0;
        p.C = a.C; p.ldc = a.ldc; p.c_batch = a.c_batch;
        p.bias = a.bias; p.alpha = a.alpha; p.clamp = a.clamp;
        p.err = err;
        p.vec_ok = ((reinterpret_cast<uintptr_t>(a.C) & 15u) == 0) && (a.ldc % 4 == 0) && (a.c_batch % 4 == 0) && (a.N % 4 == 0);
        return launch_bn_mn(BN, half, tmA, tmB, p, st);
    }
    TmaType tt = (a.elem == 0) ? (a.tf32_mode == 1 ? TmaType::TF32 : TmaType::F32)
                               : (a.elem == 1 ? TmaType::F16 : TmaType::BF16);
    CUtensorMap tmA, tmB;
    const uint64_t a_bs = (a.batch > 1) ? static_cast<uint64_t>(a.a_batch) * es : 0;
    const uint64_t b_bs = (a.batch > 1) ? static_cast<uint64_t>(a.b_batch) * es : 0;
    if (!make_tmap_3d(&tmA, tt, a.A, a.K, a.M, a.batch, static_cast<uint64_t>(a.lda) * es, a_bs, bk, 128, true))
        return ST_UNSUPPORTED_PATH;
    if (!make_tmap_3d(&tmB, tt, a.B, a.K, a.N, a.batch, static_cast<uint64_t>(a.ldb) * es, b_bs, bk, BN, true))
        return ST_UNSUPPORTED_PATH;

    GemmParams p{};
    p.M = a.M; p.N = a.N; p.K = a.K; p.batch = a.batch;
    p.k_steps = (a.K + bk - 1) / bk;
    p.C = a.C; p.ldc = a.ldc; p.c_batch = a.c_batch;
    p.bias = a.bias; p.alpha = a.alpha; p.clamp = a.clamp;
    p.ln_stats = a.ln_stats; p.ln_u = a.ln_u; p.gate = a.gate; p.act = a.act;
    p.opm_D = a.opm_D; p.opm_L = a.opm_L;
    p.ab_fmt = (a.elem == 2) ? 1 : 0;
    p.err = err;
    const bool c_al = (reinterpret_cast<uintptr_t>(a.C) & 15u) == 0;
    if (a.opm_L > 0) p.vec_ok = c_al && (a.opm_L % 4 == 0);
    else p.vec_ok = c_al && (a.ldc % 4 == 0) && (a.c_batch % 4 == 0) && (a.N % 4 == 0);

    const bool opm = a.opm_L > 0;
    const bool fused = a.ln_stats != nullptr || a.gate != nullptr || a.act != 0;
    if (fused) {                                   // fp32 operands, row-major result only
        if (opm || a.elem != 0) return ST_UNSUPPORTED_PATH;
        return (a.tf32_mode == 0) ? launch_bn<MmaKind::TF32, Epi::ROW_MAJOR_FUSED, true>(BN, tmA, tmB, p, st)
                                  : launch_bn<MmaKind::TF32, Epi::ROW_MAJOR_FUSED, false>(BN, tmA, tmB, p, st);
    }
    if (a.elem == 0) {
        const bool conv = (a.tf32_mode == 0);
        if (opm) return conv ? launch_bn<MmaKind::TF32, Epi::OPM_BLOCKED, true>(BN, tmA, tmB, p, st)
                             : launch_bn<MmaKind::TF32, Epi::OPM_BLOCKED, false>(BN, tmA, tmB, p, st);
        return conv ? launch_bn<MmaKind::TF32, Epi::ROW_MAJOR, true>(BN, tmA, tmB, p, st)
                    : launch_bn<MmaKind::TF32, Epi::ROW_MAJOR, false>(BN, tmA, tmB, p, st);
    }
    if (opm) return launch_bn<MmaKind::F16, Epi::OPM_BLOCKED, false>(BN, tmA, tmB, p, st);
    return launch_bn<MmaKind::F16, Epi::ROW_MAJOR, false>(BN, tmA, tmB, p, st);
}

}  // namespace ppml_b200
