"""Generates tests/golden/*.npz by running the reference's own, unmodified CPU implementation
(compiled by oracle/Makefile into oracle/_ref/libppml_ref.so) on the seeded inputs of
tests/cases.py.  Run where the reference tree is mounted:

    make -C oracle ref && python tests/golden/make_golden.py

Only outputs (and the seeds/shapes that regenerate the inputs) are stored, so the files stay small.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import cases  # noqa: E402
from checkers import Ref  # noqa: E402

os.environ["PPML_CPU_F16C"] = "0"      # the scalar fp16 dot, the loop the restatement follows


HOT_LAUNCHERS = ("mul_mat_cuda", "mul_mat_mma_tf32_smem", "mul_mat_mma_f16", "mul_mat_cuda_f16", "mul_mat_q8_cuda",
                 "quantize_rows_q8_1_cuda", "dequantize_q8_", "flash_attn_forward_cuda", "flash_attn_backward_cuda", "out_prod_cuda",
                 "tri_mul_cuda", "outer_prod_mean_cuda", "mulmat_stats_cuda", "cutlass_hw_supported")


def reference_dir():
    """The reference checkout: $PPML_REFERENCE_DIR, else the directory `reference` beside this repository."""
    return os.environ.get("PPML_REFERENCE_DIR") or os.path.abspath(os.path.join(HERE, "..", "..", "..", "reference"))


def launcher_symbols(reference=None):
    """The mangled names the reference's dispatcher (src/backend/CUDAKernels.cpp) leaves undefined for the
    hot-path launchers: exactly what a drop-in library has to export."""
    import subprocess
    import tempfile
    reference = reference or reference_dir()
    with tempfile.TemporaryDirectory() as tmp:
        obj = os.path.join(tmp, "CUDAKernels.o")
        subprocess.check_call(["g++", "-std=c++17", "-O0", "-w", "-fPIC", f"-I{reference}/include",
                               "-I/usr/local/cuda/include", "-c", f"{reference}/src/backend/CUDAKernels.cpp", "-o", obj])
        names = subprocess.check_output(["nm", "-u", obj], text=True).split()
    want = sorted(n for n in names if n.startswith("_ZN4ppml") and any(h in n for h in HOT_LAUNCHERS)
                  and ("back" not in n or "flash_attn_backward_cuda" in n))
    with open(os.path.join(HERE, "reference_launcher_symbols.txt"), "w") as f:
        f.write("\n".join(want) + "\n")
    print("wrote", len(want), "launcher symbols")


def main():
    launcher_symbols()
    ref = Ref(n_threads=4)
    out = {}

    # OP_MUL_MAT, dev-forward shapes (M, K, N) incl. the SE3 radial shapes with K = 33
    for (M, K, N) in [(17, 9, 23), (408, 256, 256), (51, 128, 8), (255, 33, 32), (130, 64, 128)]:
        a, b, bi = cases.mul_mat_case(M, K, N, seed=1)
        out[f"mm_{M}_{K}_{N}"] = ref.mul_mat(a, b, None)
        out[f"mmb_{M}_{K}_{N}"] = ref.mul_mat(a, b, bi)
    a, b, bi = cases.mul_mat_case(40, 64, 48, seed=11)
    out["mm16_40_64_48"] = ref.mul_mat(a.astype(np.float16).view(np.uint16), b.astype(np.float16).view(np.uint16), bi, f16=True)

    # quantizers (bit patterns)
    w, x = cases.q8_case(24, 20, 128, seed=2)
    x[3, :32] = 0.0
    x[4, 0], x[4, 1] = 2.5, -2.5          # +a / -a tie: the first one decides the sign of d
    x[5, 0], x[5, 1] = -1.5, 1.5
    out["q80_w"] = ref.quantize_q8_0(w)
    out["q80r_w"] = ref.repack_q8_0(out["q80_w"])
    out["q81_x"] = ref.quantize_q8_1(x)
    out["deq80_w"] = ref.dequantize(out["q80_w"], 0)
    out["deq81_x"] = ref.dequantize(out["q81_x"], 1)

    # attention: fused CPU forward, its naive twin, and the unfused graph (ground truth for Lq != Lk)
    Q, K, V, bi = cases.attn_case(2, 3, 70, 32, seed=3)
    out["fa_O"], out["fa_LSE"] = ref.flash_attn(Q, K, V, bi, scale=1 / np.sqrt(32.0))
    out["fa_causal_O"], out["fa_causal_LSE"] = ref.flash_attn(Q, K, V, None, causal=True)
    out["fa_naive_O"], _ = ref.flash_attn(Q, K, V, bi, scale=1 / np.sqrt(32.0), naive=True)
    out["fa_legacy_O"] = ref.attention_legacy(Q, K, V, bi, 1 / np.sqrt(32.0))
    Q, K, V, bi = cases.attn_case(3, 2, 1, 8, Lk=40, seed=33)
    out["fa_legacy_q1_O"] = ref.attention_legacy(Q, K, V, bi, 1 / np.sqrt(32.0))

    # a row whose first key tile holds only -inf scores comes out as zeros in the reference (NaN, then `l > 0` fails)
    Q, K, V, bi = cases.attn_masked_first_tile_case(d=8, L=100, Lk=200)
    # the reference's config has one L: pad the queries to Lk rows and keep the first L (rows are independent)
    Qp = np.zeros((2, 2, 200, 8), np.float32); Qp[:, :, :100] = Q
    bp = np.zeros((2, 2, 200, 200), np.float32); bp[:, :, :100] = bi
    o, l_ = ref.flash_attn(Qp, K, V, bp, scale=1 / np.sqrt(32.0))
    out["fa_masked_O"], out["fa_masked_LSE"] = o[:, :, :100].copy(), l_[:, :, :100].copy()

    # attention backward (flash_attn_backward_cpu) on the forward's own O and LSE; rows 5 and 17 fully masked
    Q, K, V, bi, dO = cases.attn_backward_case(2, 3, 45, 32, seed=7, masked_rows=(5, 17))
    O, LSE = ref.flash_attn(Q, K, V, bi, scale=1 / np.sqrt(32.0))
    g = ref.flash_attn_backward(Q, K, V, O, dO, LSE, bi, scale=1 / np.sqrt(32.0))
    for n in ("dQ", "dK", "dV", "dbias"):
        out["fab_" + n] = g[n]
    g = ref.flash_attn_backward(Q, K, V, *ref.flash_attn(Q, K, V, None, causal=True)[:1], dO,
                                ref.flash_attn(Q, K, V, None, causal=True)[1], None, causal=True)
    for n in ("dQ", "dK", "dV", "dbias"):
        out["fab_causal_" + n] = g[n]

    # pair-track contractions
    l, r = cases.tri_case(6, 20, 24, 28, outgoing=True)
    out["tri_out"] = ref.tri_mul(l, r, 28.0, True)
    l, r = cases.tri_case(6, 20, 24, 28, outgoing=False)
    out["tri_in"] = ref.tri_mul(l, r, 28.0, False)
    l, r = cases.tri_case(3, 5, 6, 7, B=2, outgoing=True, seed=44)
    out["tri_out_b2"] = ref.tri_mul(l, r, 7.0, True, B=2)
    l = np.full((1, 2, 2, 1), 3e3, np.float32)
    out["tri_clamp"] = ref.tri_mul(l, l, 1.0, True)
    l, r = cases.opm_case(4, 12, 9)
    out["opm"] = ref.outer_prod_mean(l, r)
    s0, s1 = cases.out_prod_case(13, 11, 17, 3, 2)
    out["out_prod"] = ref.out_prod(s0, s1)
    s0, s1 = cases.out_prod_case(13, 11, 17, 4, 2, ne02=2, ne03=1)
    out["out_prod_bcast"] = ref.out_prod(s0, s1)

    np.savez_compressed(os.path.join(HERE, "reference_cpu.npz"), **out)
    print("wrote", len(out), "arrays,", os.path.getsize(os.path.join(HERE, "reference_cpu.npz")), "bytes")


if __name__ == "__main__":
    main()
