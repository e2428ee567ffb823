"""Seeded synthetic inputs shared by the golden-fixture generator and the parity tests.  The shapes
and value distributions are those of the benchmark configurations (dev-size forward shapes, the Q8
sweep, axial attention, pair-track contractions), scaled down where a CPU checker must finish in
seconds."""
import numpy as np


def rng(seed):
    return np.random.default_rng(seed)


def mul_mat_case(M, K, N, seed=1, bias=True):
    r = rng(seed)
    a = r.standard_normal((M, K)).astype(np.float32)
    b = (r.standard_normal((N, K)) * 0.02).astype(np.float32)      # N(0, 0.02) linear weights
    bi = (r.standard_normal(N) * 0.1).astype(np.float32) if bias else None
    return a, b, bi


def q8_case(M_out, N_tok, K, seed=2):
    r = rng(seed)
    w = (r.standard_normal((M_out, K)) * 0.02).astype(np.float32)
    x = r.standard_normal((N_tok, K)).astype(np.float32)
    return w, x


def attn_case(B, h, L, d, Lk=None, seed=3, bias=True, bias_bcast=False):
    r = rng(seed)
    Lk = L if Lk is None else Lk
    s = 1.0 / np.sqrt(32.0)
    Q = (r.standard_normal((B, h, L, d)) * s).astype(np.float32)
    K = (r.standard_normal((B, h, Lk, d)) * s).astype(np.float32)
    V = (r.standard_normal((B, h, Lk, d)) * s).astype(np.float32)
    bi = None
    if bias:
        shape = (h, L, Lk) if bias_bcast else (B, h, L, Lk)
        bi = r.standard_normal(shape).astype(np.float32)
    return Q, K, V, bi


def attn_backward_case(B, h, L, d, seed=7, bias=True, bias_bcast=False, masked_rows=()):
    """Inputs of the attention backward: the forward's operands, an upstream gradient dO, and optionally query rows
    whose bias is -inf everywhere (fully masked: LSE = -inf, all their gradients are 0)."""
    Q, K, V, bi = attn_case(B, h, L, d, seed=seed, bias=bias or bool(masked_rows), bias_bcast=bias_bcast)
    for r in masked_rows:
        bi[..., r, :] = -np.inf
    dO = rng(seed + 100).standard_normal((B, h, L, d)).astype(np.float32)
    return Q, K, V, bi, dO


def attn_masked_first_tile_case(d=8, L=100, Lk=200, seed=13):
    """Rows whose leading scores are -inf: row 3 has the reference's whole first key tile (64 keys) masked and later
    keys visible, row 4 has 63 of them masked, row 2 two whole tiles."""
    Q, K, V, bi = attn_case(2, 2, L, d, Lk=Lk, seed=seed)
    bi[:, :, 3, :64] = -np.inf
    bi[:, :, 4, :63] = -np.inf
    bi[:, :, 2, :130] = -np.inf
    return Q, K, V, bi


def tri_case(D, I, J, K, B=1, outgoing=True, seed=4):
    r = rng(seed)
    if outgoing:
        left = r.standard_normal((D, I, K, B)).astype(np.float32)
        right = r.standard_normal((D, J, K, B)).astype(np.float32)
    else:
        left = r.standard_normal((D, K, I, B)).astype(np.float32)
        right = r.standard_normal((D, K, J, B)).astype(np.float32)
    return left, right


def opm_case(D, L, N, B=1, seed=4):
    r = rng(seed)
    return (r.standard_normal((D, L, N, B)).astype(np.float32),
            r.standard_normal((D, L, N, B)).astype(np.float32))


def out_prod_case(ne00, ne10, K, ne2, ne3, ne02=None, ne03=None, seed=5):
    r = rng(seed)
    ne02 = ne2 if ne02 is None else ne02
    ne03 = ne3 if ne03 is None else ne03
    s0 = r.standard_normal((ne03, ne02, K, ne00)).astype(np.float32)
    s1 = r.standard_normal((ne3, ne2, K, ne10)).astype(np.float32)
    return s0, s1


def rel_err(got, ref):
    """max |got - ref| / max |ref| -- the normalised error every floating-point tolerance here uses."""
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))
