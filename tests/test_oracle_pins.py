"""Pins the CPU oracle to the reference's own known-answer tests and equivalence fixtures.

Each test restates one test of the reference (file:line given) against the oracle's
restatement of the same function.  The reference is Rust and cannot be executed on the
build or GPU machines, so these transcribed vectors are what anchors the oracle.
"""
import math

import numpy as np
import pytest

SEED_Q, SEED_K, SEED_V = 0xC0FFEE, 0xBADBEEF, 0xCAFE00


def _buffers(orc, shape, width):
    n = int(np.prod(shape))
    q = orc.fill_lcg(n, SEED_Q, width).reshape(shape)
    k = orc.fill_lcg(n, SEED_K, width).reshape(shape)
    v = orc.fill_lcg(n, SEED_V, width).reshape(shape)
    return q, k, v


def _close(a, b, atol, rtol=1e-4):
    a, b = np.asarray(a), np.asarray(b)
    both_nan = np.isnan(a) & np.isnan(b)
    ok = np.abs(a - b) <= atol + rtol * np.maximum(np.abs(a), np.abs(b))
    return bool(np.all(ok | both_nan))


def test_lcg_fixture_first_values(oracle):
    # cpu_forward.rs:769-780: s = seed*2654435761 (wrapping); s = s*1664525+1013904223.
    s = (0xC0FFEE * 2654435761) & 0xFFFFFFFF
    exp = []
    for _ in range(4):
        s = (s * 1664525 + 1013904223) & 0xFFFFFFFF
        exp.append((np.float32(s) / np.float32(0xFFFFFFFF) - np.float32(0.5)) * np.float32(3.0))
    got = oracle.fill_lcg(4, 0xC0FFEE, 3.0)
    assert np.array_equal(got, np.array(exp, dtype=np.float32))


# cpu_forward.rs:804-840, 917-929 (flash == naive, atol 1e-4 + 1e-4*max|.|)
@pytest.mark.parametrize("shape,br,bc", [((2, 4, 32, 16), 64, 64), ((1, 2, 70, 24), 64, 64),
                                         ((2, 4, 128, 64), 64, 64), ((4, 8, 96, 32), 64, 64)])
def test_flash_matches_naive_unit_shapes(oracle, shape, br, bc):
    q, k, v = _buffers(oracle, shape, 3.0)
    rc, o_flash = oracle.flash_forward_masked(q, k, v, br=br, bc=bc)
    rc2, o_naive = oracle.naive_forward_masked(q, k, v)
    assert rc == 0 and rc2 == 0
    assert _close(o_flash, o_naive, 1e-4)


def test_scaling_factor_is_one_over_sqrt_d(oracle):  # cpu_forward.rs:842-856
    q = np.array([1, 0, 0, 0], dtype=np.float32).reshape(1, 1, 1, 4)
    v = np.array([5, -2, 7, 1], dtype=np.float32).reshape(1, 1, 1, 4)
    rc, out = oracle.flash_forward_masked(q, q.copy(), v)
    assert rc == 0 and _close(out, v, 1e-6)


def test_empty_seq_is_no_op(oracle):  # cpu_forward.rs:860-869
    e = np.zeros((2, 4, 0, 16), dtype=np.float32)
    rc, out = oracle.flash_forward_masked(e, e, e)
    assert rc == 0 and out.size == 0


def test_zero_dim_returns_error(oracle):  # cpu_forward.rs:871-882
    e = np.zeros((1, 1, 4, 0), dtype=np.float32)
    rc, _ = oracle.flash_forward_masked(e, e, e)
    assert rc == oracle.ERR_ZERO_DIM


def test_nan_input_propagates(oracle):  # cpu_forward.rs:898-915
    shape = (1, 1, 4, 8)
    q = oracle.fill_lcg(32, 1, 3.0).reshape(shape)
    q[0, 0, 0, 0] = np.nan
    k = oracle.fill_lcg(32, 2, 3.0).reshape(shape)
    v = oracle.fill_lcg(32, 3, 3.0).reshape(shape)
    _, o_flash = oracle.flash_forward_masked(q, k, v, br=4, bc=4)
    _, o_naive = oracle.naive_forward_masked(q, k, v)
    assert np.array_equal(np.isnan(o_flash), np.isnan(o_naive))


def test_causal_flash_matches_causal_naive(oracle):  # cpu_forward.rs:933-941
    q, k, v = _buffers(oracle, (1, 2, 64, 32), 3.0)
    _, a = oracle.flash_forward_masked(q, k, v, oracle.MASK_CAUSAL)
    _, b = oracle.naive_forward_masked(q, k, v, oracle.MASK_CAUSAL)
    assert _close(a, b, 1e-4)


def test_padding_flash_matches_padding_naive(oracle):  # cpu_forward.rs:943-953
    q, k, v = _buffers(oracle, (1, 1, 8, 4), 3.0)
    keep = [1, 0, 1, 1, 0, 1, 0, 1]
    _, a = oracle.flash_forward_masked(q, k, v, oracle.MASK_PADDING, keep)
    _, b = oracle.naive_forward_masked(q, k, v, oracle.MASK_PADDING, keep)
    assert _close(a, b, 1e-4)


def test_causal_first_query_only_attends_to_self(oracle):  # cpu_forward.rs:955-980
    shape = (1, 1, 4, 8)
    q = np.ones(shape, dtype=np.float32)
    v = np.zeros(shape, dtype=np.float32)
    v[0, 0, 0] = 10.0 * np.arange(1, 9)
    v[0, 0, 1] = -99.0
    v[0, 0, 2] = 99.0
    _, out = oracle.flash_forward_masked(q, q.copy(), v, oracle.MASK_CAUSAL)
    assert _close(out[0, 0, 0], v[0, 0, 0], 1e-6)


def test_padding_mask_excludes_padded_positions_exactly(oracle):  # cpu_forward.rs:982-998
    shape = (1, 1, 4, 4)
    q = np.ones(shape, dtype=np.float32)
    v = np.zeros(shape, dtype=np.float32)
    v[0, 0, :, 0] = [10.0, 99.0, -99.0, 30.0]
    _, out = oracle.flash_forward_masked(q, q.copy(), v, oracle.MASK_PADDING, [1, 0, 0, 1])
    assert abs(out[0, 0, 0, 0] - 20.0) <= 1e-5 + 1e-4 * 20.0


def test_padding_mask_length_mismatch(oracle):  # cpu_forward.rs:1000-1014
    q, k, v = _buffers(oracle, (1, 1, 4, 4), 3.0)
    rc, _ = oracle.flash_forward_masked(q, k, v, oracle.MASK_PADDING, [1, 1, 1])
    assert rc == oracle.ERR_MASK_LEN


def test_flash_stable_for_large_magnitudes(oracle):  # cpu_forward.rs:1016-1037
    shape = (1, 1, 16, 8)
    i = np.arange(128, dtype=np.float32)
    q = (np.float32(1e3) + np.sin(i * np.float32(0.01))).astype(np.float32).reshape(shape)
    k = (np.float32(1e3) + np.cos(i * np.float32(0.013))).astype(np.float32).reshape(shape)
    v = np.sin(i * np.float32(0.07)).astype(np.float32).reshape(shape)
    _, a = oracle.flash_forward_masked(q, k, v)
    _, b = oracle.naive_forward_masked(q, k, v)
    assert _close(a, b, 1e-3) and np.all(np.isfinite(a))


# tests/equivalence.rs:34-125: 20 fixed shapes, LCG width 2.0, max-abs < 1e-4 and Frobenius < 1e-4*sqrt(n)
SHAPES_20 = [(1, 1, 1, 4), (1, 1, 2, 4), (1, 1, 16, 8), (1, 2, 32, 16), (2, 2, 32, 16), (1, 4, 64, 32),
             (2, 4, 128, 32), (1, 8, 64, 64), (1, 8, 128, 64), (2, 8, 128, 64), (4, 8, 128, 64),
             (1, 1, 63, 32), (1, 1, 64, 32), (1, 1, 65, 32), (1, 1, 127, 32), (1, 1, 128, 32),
             (1, 1, 129, 32), (1, 1, 32, 4), (1, 1, 32, 128), (1, 1, 96, 48)]


@pytest.mark.parametrize("shape", SHAPES_20)
def test_equivalence_20_shapes(oracle, shape):
    q, k, v = _buffers(oracle, shape, 2.0)
    _, a = oracle.flash_forward_masked(q, k, v)
    _, b = oracle.naive_forward_masked(q, k, v)
    d = np.abs(a - b)
    assert d.max() < 1e-4
    assert math.sqrt(float((d.astype(np.float64) ** 2).sum())) < 1e-4 * math.sqrt(a.size)
    assert np.all(np.isfinite(a))


def test_random_small_shapes_br16(oracle):
    # cpu_forward.rs:1045-1087: random B<3,H<4,N<40,D in [4,16), br=bc=16, tol 1e-3 (+ the saved
    # regression shape B1H1N1D4 from proptest-regressions/cpu_forward.txt).
    rng = np.random.default_rng(7)
    shapes = [(1, 1, 1, 4)] + [(int(rng.integers(1, 3)), int(rng.integers(1, 4)), int(rng.integers(1, 40)),
                                int(rng.integers(4, 16))) for _ in range(60)]
    for shape in shapes:
        n = int(np.prod(shape))
        i = np.arange(n, dtype=np.uint64)
        mk = lambda mul: (((i * np.uint64(mul) * np.uint64(2654435761)) & np.uint64(0xFFFFFFFF)).astype(np.float32)
                          / np.float32(0xFFFFFFFF) - np.float32(0.5)) * np.float32(2.0)
        q, k, v = (mk(m).astype(np.float32).reshape(shape) for m in (1, 13, 29))
        _, a = oracle.flash_forward_masked(q, k, v, br=16, bc=16)
        _, b = oracle.naive_forward_masked(q, k, v)
        assert _close(a, b, 1e-3, 1e-3), shape


# ---- online softmax (online_softmax.rs:153-307)

def _naive_ml(xs):
    xs = np.asarray(xs, dtype=np.float32)
    if xs.size == 0:
        return -math.inf, 0.0
    m = float(xs.max())
    return m, float(np.exp(xs - np.float32(m)).astype(np.float32).sum())


def _c(a, b, tol):
    if math.isinf(a) and math.isinf(b):
        return (a > 0) == (b > 0)
    return abs(a - b) <= tol * (1 + max(abs(a), abs(b)))


def test_online_single_tile_matches_naive(oracle):
    xs = [0.5, -1.0, 2.5, 0.1, -3.0, 4.0]
    m, l = oracle.online_softmax_full(xs)
    mn, ln = _naive_ml(xs)
    assert _c(m, mn, 1e-6) and _c(l, ln, 1e-6)


def test_online_four_tiles_combine(oracle):
    xs = np.sin(np.arange(32, dtype=np.float32) * np.float32(0.1)).astype(np.float32)
    st = (-math.inf, 0.0)
    for c in range(4):
        st = oracle.combine_tiles(st, oracle.online_softmax_full(xs[c * 8:(c + 1) * 8]))
    mn, ln = _naive_ml(xs)
    assert _c(st[0], mn, 1e-7) and _c(st[1], ln, 1e-6)


def test_online_associativity_commutativity(oracle):
    a, b, c, d = (1.5, 3.0), (0.7, 5.0), (2.1, 1.0), (-0.3, 7.0)
    ct = oracle.combine_tiles
    s1 = ct(ct(a, b), ct(c, d))
    s2 = ct(ct(ct(a, b), c), d)
    s3 = ct(a, ct(b, ct(c, d)))
    for s in (s2, s3):
        assert _c(s1[0], s[0], 1e-6) and _c(s1[1], s[1], 1e-6)
    ab, ba = ct(a, b), ct(b, a)
    assert _c(ab[0], ba[0], 1e-7) and _c(ab[1], ba[1], 1e-7)


def test_online_edge_cases(oracle):
    assert oracle.online_softmax_full([]) == (-math.inf, 0.0)
    m, l = oracle.online_softmax_full([-math.inf] * 4)
    assert m == -math.inf and (math.isnan(l) or l == 0.0)
    assert oracle.online_softmax_full([1.0, math.inf, -2.0, 0.0]) == (math.inf, 1.0)
    s = (1.5, 3.0)
    assert oracle.combine_tiles((-math.inf, 0.0), s) == s and oracle.combine_tiles(s, (-math.inf, 0.0)) == s
    assert oracle.online_softmax_full([2.5]) == (2.5, 1.0)
    m, l = oracle.online_softmax_full([1e30] * 4)
    assert m == np.float32(1e30) and l == 4.0


# ---- GQA (gqa.rs:272-389)

def test_gqa_equal_heads_range_check(oracle):
    n = 1 * 4 * 3 * 4
    q = ((np.arange(n) + 1) * 0.01).astype(np.float32)
    k = ((np.arange(n) + 1) * 0.02).astype(np.float32)
    v = ((np.arange(n) + 1) * 0.03).astype(np.float32)
    rc, out = oracle.gqa_forward_f32(q, k, v, 1, 4, 4, 3, 3, 4)
    assert rc == 0
    for h in range(4):
        vb = v[h * 12:(h + 1) * 12]
        ob = out[h * 12:(h + 1) * 12]
        assert ob.min() >= vb.min() - 1e-5 and ob.max() <= vb.max() + 1e-5


def test_gqa_4_to_1_finite_and_heads_differ(oracle):
    nq, nk = 8 * 4 * 8, 2 * 4 * 8
    q = np.sin(np.arange(nq, dtype=np.float32) * np.float32(0.001)).astype(np.float32)
    k = np.cos(np.arange(nk, dtype=np.float32) * np.float32(0.001)).astype(np.float32)
    v = np.tan((np.arange(nk, dtype=np.float32) + 1) * np.float32(0.0005)).astype(np.float32)
    rc, out = oracle.gqa_forward_f32(q, k, v, 1, 8, 2, 4, 4, 8)
    assert rc == 0 and np.all(np.isfinite(out))
    for kv_h in range(2):
        h0, h1 = kv_h * 4, kv_h * 4 + 3
        assert np.abs(out[h0 * 32:h0 * 32 + 8] - out[h1 * 32:h1 * 32 + 8]).sum() > 1e-6


def test_gqa_head_count_mismatch(oracle):
    z = np.zeros(20, dtype=np.float32)
    rc, _ = oracle.gqa_forward_f32(z, z[:8], z[:8], 1, 5, 2, 1, 1, 4)
    assert rc == oracle.ERR_HEADS


def test_gqa_decode_row_equals_naive_attention(oracle):
    # The decode row kernel (gqa.rs:216-270) against an independent numpy softmax.
    rng = np.random.default_rng(0)
    B, Hq, Hkv, L, D = 2, 8, 2, 37, 16
    q = rng.standard_normal((B, Hq, 1, D), dtype=np.float32)
    k = rng.standard_normal((B, Hkv, L, D), dtype=np.float32)
    v = rng.standard_normal((B, Hkv, L, D), dtype=np.float32)
    rc, out = oracle.gqa_forward_f32(q.ravel(), k.ravel(), v.ravel(), B, Hq, Hkv, 1, L, D)
    assert rc == 0
    out = out.reshape(B, Hq, D)
    for b in range(B):
        for h in range(Hq):
            s = (k[b, h // 4] @ q[b, h, 0]).astype(np.float64) / math.sqrt(D)
            w = np.exp(s - s.max())
            ref = (w / w.sum()) @ v[b, h // 4].astype(np.float64)
            assert np.abs(out[b, h] - ref).max() < 1e-5


# ---- the timed CPU arm: register-blocked tile GEMMs standing in for the `gemm` crate
@pytest.mark.parametrize("shape", SHAPES_20)
def test_micro_kernel_path_matches_loop_nests(oracle, shape):
    """The micro-kernel path of the timed baseline computes what the loop-nest oracle computes (1e-4, the
    reference's own flash-vs-naive gate), on the reference's 20-shape matrix; shapes whose dims the
    micro-kernels do not cover fall back to the loop nests and agree exactly."""
    q, k, v = _buffers(oracle, shape, 2.0)
    assert oracle.get_gemm_kernel() == 0
    _, a = oracle.flash_forward_masked(q, k, v)
    oracle.set_gemm_kernel(1)
    try:
        _, b = oracle.flash_forward_masked(q, k, v)
        _, c = oracle.flash_forward_masked(q, k, v, mask_kind=1)
    finally:
        oracle.set_gemm_kernel(0)
    _, c0 = oracle.flash_forward_masked(q, k, v, mask_kind=1)
    assert np.abs(a - b).max() < 1e-4 and np.abs(c - c0).max() < 1e-4
    _, n = oracle.naive_forward_masked(q, k, v)
    assert np.abs(b - n).max() < 1e-4


def test_micro_kernel_path_ragged_and_masked(oracle):
    """Sequence lengths that leave partial row and key tiles, causal + kv_len, LSE: both GEMM modes agree."""
    for (B, H, N, D) in ((1, 2, 200, 64), (2, 1, 129, 128), (1, 1, 70, 32)):
        q, k, v = (oracle.round_to_bf16(oracle.fill_normal((B, H, N, D), s)) for s in (5, 6, 7))
        lens = np.array([N - 3] * B, dtype=np.int32)
        _, a, la = oracle.flash_forward_ext(q, k, v, causal=True, kv_lens=lens)
        oracle.set_gemm_kernel(1)
        try:
            _, b, lb = oracle.flash_forward_ext(q, k, v, causal=True, kv_lens=lens)
        finally:
            oracle.set_gemm_kernel(0)
        assert np.array_equal(np.isnan(a), np.isnan(b))
        ok = ~np.isnan(a)
        assert np.abs(a[ok] - b[ok]).max() < 1e-4 and np.abs(la - lb).max() < 1e-4
    if oracle.micro_isa() != "none":
        assert oracle.tile_gemm_gflops(64, 200) > 0.0 and oracle.fma_peak_gflops() > 0.0
