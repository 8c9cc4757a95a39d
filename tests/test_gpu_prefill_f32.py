"""GPU parity of the f32 CUDA-core forward and of the host mirrors of the reference API
(flash_forward, flash_forward_masked, gqa_forward_f32) at the reference's own 1e-4 gate."""
import numpy as np
import pytest

from tests import util
from tests.test_oracle_pins import SHAPES_20, SEED_Q, SEED_K, SEED_V

pytestmark = pytest.mark.gpu


def _lcg(orc, shape, width):
    n = int(np.prod(shape))
    return tuple(orc.fill_lcg(n, s, width).reshape(shape) for s in (SEED_Q, SEED_K, SEED_V))


@pytest.mark.parametrize("shape", SHAPES_20)
def test_flash_forward_host_matches_naive_20_shapes(oracle, shape):
    """tests/equivalence.rs:34-125 with the GPU in place of the CPU tiled path."""
    import rustorch_b200 as rt
    q, k, v = _lcg(oracle, shape, 2.0)
    out = np.zeros_like(q)
    rt.flash_forward(rt.AttentionShape.new(*shape), q, k, v, out)
    _, ref = oracle.naive_forward_masked(q, k, v)
    d = np.abs(out - ref)
    assert d.max() < 1e-4 and np.sqrt((d.astype(np.float64) ** 2).sum()) < 1e-4 * np.sqrt(out.size)
    assert np.all(np.isfinite(out))


def test_masked_host_entry_kats(oracle):
    import rustorch_b200 as rt
    # causal_first_query_only_attends_to_self (cpu_forward.rs:955-980)
    shape = rt.AttentionShape.new(1, 1, 4, 8)
    q = np.ones((1, 1, 4, 8), dtype=np.float32)
    v = np.zeros_like(q)
    v[0, 0, 0] = 10.0 * np.arange(1, 9)
    v[0, 0, 1], v[0, 0, 2] = -99.0, 99.0
    out = np.zeros_like(q)
    rt.flash_forward_masked(shape, q, q.copy(), v, rt.Mask.causal(), out)
    assert np.abs(out[0, 0, 0] - v[0, 0, 0]).max() <= 1e-5
    # padding_mask_excludes_padded_positions_exactly (cpu_forward.rs:982-998)
    shape = rt.AttentionShape.new(1, 1, 4, 4)
    q = np.ones((1, 1, 4, 4), dtype=np.float32)
    v = np.zeros_like(q)
    v[0, 0, :, 0] = [10.0, 99.0, -99.0, 30.0]
    out = np.zeros_like(q)
    rt.flash_forward_masked(shape, q, q.copy(), v, rt.Mask.padding([True, False, False, True]), out)
    assert abs(out[0, 0, 0, 0] - 20.0) < 1e-4
    # scaling_factor_is_one_over_sqrt_d (cpu_forward.rs:842-856)
    shape = rt.AttentionShape.new(1, 1, 1, 4)
    q = np.array([1, 0, 0, 0], dtype=np.float32)
    v = np.array([5, -2, 7, 1], dtype=np.float32)
    out = np.zeros(4, dtype=np.float32)
    rt.flash_forward(shape, q, q.copy(), v, out)
    assert np.abs(out - v).max() < 1e-6


def test_host_entry_errors(oracle):
    import rustorch_b200 as rt
    z = lambda n: np.zeros(n, dtype=np.float32)
    with pytest.raises(rt.ZeroDim):
        rt.flash_forward(rt.AttentionShape.new(1, 1, 4, 0), z(0), z(0), z(0), z(0))
    with pytest.raises(rt.BufferShapeMismatch) as e:
        rt.flash_forward(rt.AttentionShape.new(1, 1, 4, 8), z(32), z(16), z(32), z(32))
    assert e.value.which == "k" and e.value.expected == 32 and e.value.got == 16
    with pytest.raises(rt.OutputShapeMismatch):
        rt.flash_forward(rt.AttentionShape.new(1, 1, 4, 8), z(32), z(32), z(32), z(31))
    with pytest.raises(rt.PaddingLengthMismatch) as e:
        rt.flash_forward_masked(rt.AttentionShape.new(1, 1, 4, 4), z(16), z(16), z(16), rt.Mask.padding([True] * 3),
                                z(16))
    assert e.value.expected == 4 and e.value.got == 3
    e0 = z(0)
    rt.flash_forward(rt.AttentionShape.new(2, 4, 0, 16), e0, e0, e0, e0)  # empty seq is a no-op


def test_nan_propagation_and_large_magnitudes(oracle):
    import rustorch_b200 as rt
    shape = (1, 1, 4, 8)
    q = oracle.fill_lcg(32, 1, 3.0).reshape(shape)
    q[0, 0, 0, 0] = np.nan
    k = oracle.fill_lcg(32, 2, 3.0).reshape(shape)
    v = oracle.fill_lcg(32, 3, 3.0).reshape(shape)
    out = np.zeros_like(q)
    rt.flash_forward(rt.AttentionShape.new(*shape), q, k, v, out)
    _, ref = oracle.naive_forward_masked(q, k, v)
    assert np.array_equal(np.isnan(out), np.isnan(ref))
    shape = (1, 1, 16, 8)
    i = np.arange(128, dtype=np.float32)
    q = (np.float32(1e3) + np.sin(i * np.float32(0.01))).astype(np.float32).reshape(shape)
    k = (np.float32(1e3) + np.cos(i * np.float32(0.013))).astype(np.float32).reshape(shape)
    v = np.sin(i * np.float32(0.07)).astype(np.float32).reshape(shape)
    out = np.zeros_like(q)
    rt.flash_forward(rt.AttentionShape.new(*shape), q, k, v, out)
    _, ref = oracle.naive_forward_masked(q, k, v)
    assert np.all(np.isfinite(out)) and np.all(np.abs(out - ref) <= 1e-3 + 1e-4 * np.abs(ref))


@pytest.mark.parametrize("causal,use_keep,use_lens", [(True, False, False), (False, True, False), (True, True, True),
                                                      (False, False, True)])
def test_device_f32_masks_and_lse(oracle, causal, use_keep, use_lens):
    import torch
    import rustorch_b200 as rt
    B, H, N, D = 2, 3, 150, 40
    q, k, v = (oracle.fill_normal((B, H, N, D), s) for s in (1, 2, 3))
    rng = np.random.default_rng(5)
    keep = (rng.random((B, N)) > 0.3).astype(np.uint8) if use_keep else None
    if keep is not None:
        keep[:, :70] = 0 if not causal else keep[:, :70]  # a fully masked leading stretch (first tile and more)
        keep[0, 100] = 1
    lens = np.array([150, 77], dtype=np.int32) if use_lens else None
    out, lse = rt.prefill_f32(util.to_cuda(q), util.to_cuda(k), util.to_cuda(v), causal=causal,
                              kv_lens=util.to_cuda(lens) if use_lens else None,
                              key_keep=util.to_cuda(keep) if use_keep else None)
    torch.cuda.synchronize()
    _, ref, ref_lse = oracle.naive_forward_ext(q, k, v, causal=causal, keep=keep, kv_lens=lens)
    got = util.to_np(out)
    assert np.array_equal(np.isnan(got), np.isnan(ref))
    ok = ~np.isnan(ref)
    assert np.abs(got[ok] - ref[ok]).max() < 1e-4
    util.check_lse(util.to_np(lse), ref_lse)
    # the oracle's tiled path with the leading-masked-tile fix gives the same numbers
    _, ref2, _ = oracle.flash_forward_ext(q, k, v, causal=causal, keep=keep, kv_lens=lens)
    assert np.array_equal(np.isnan(ref2), np.isnan(ref)) and np.abs(ref2[ok] - ref[ok]).max() < 1e-4


@pytest.mark.parametrize("batch,n_heads,n_kv,seq_q,seq_kv,hd", [(1, 4, 4, 3, 3, 4), (1, 8, 2, 4, 4, 8),
                                                                (2, 8, 2, 1, 37, 16), (1, 8, 4, 5, 19, 64),
                                                                (2, 4, 1, 96, 96, 32)])
def test_gqa_forward_f32_host(oracle, batch, n_heads, n_kv, seq_q, seq_kv, hd):
    import rustorch_b200 as rt
    rng = np.random.default_rng(1)
    q = rng.standard_normal(batch * n_heads * seq_q * hd).astype(np.float32)
    k = rng.standard_normal(batch * n_kv * seq_kv * hd).astype(np.float32)
    v = rng.standard_normal(batch * n_kv * seq_kv * hd).astype(np.float32)
    out = np.zeros_like(q)
    rt.gqa_forward_f32(q, k, v, out, batch, n_heads, n_kv, seq_q, seq_kv, hd)
    rc, ref = oracle.gqa_forward_f32(q, k, v, batch, n_heads, n_kv, seq_q, seq_kv, hd)
    assert rc == 0 and np.abs(out - ref).max() < 1e-4


def test_gqa_forward_f32_errors():
    import rustorch_b200 as rt
    z = lambda n: np.zeros(n, dtype=np.float32)
    with pytest.raises(rt.HeadCountMismatch):
        rt.gqa_forward_f32(z(20), z(8), z(8), z(20), 1, 5, 2, 1, 1, 4)
    with pytest.raises(rt.WrongInputLen) as e:
        rt.gqa_forward_f32(z(7), z(8), z(8), z(16), 1, 4, 2, 1, 1, 4)
    assert e.value.which == "q" and e.value.expected == 16


def test_random_shapes_property_replay_on_gpu(oracle):
    """The reference's randomised property test (cpu_forward.rs:1045-1087: B < 3, H < 4, N < 40, D in [4, 16),
    flash == naive at 1e-3) and its saved regression case B1 H1 N1 D4 (proptest-regressions/cpu_forward.txt:7),
    replayed with the GPU f32 kernel in place of the CPU tiled path: 200 seeded cases, all three mask kinds."""
    import rustorch_b200 as rt
    rng = np.random.default_rng(0x51A5)
    shapes = [(1, 1, 1, 4)] + [(int(rng.integers(1, 3)), int(rng.integers(1, 4)), int(rng.integers(1, 40)),
                                int(rng.integers(4, 16))) for _ in range(199)]
    for i, shape in enumerate(shapes):
        n = int(np.prod(shape))
        q, k, v = (oracle.fill_lcg(n, 1000 + 3 * i + j, 2.0).reshape(shape) for j in range(3))
        kind = i % 3
        keep = None
        if kind == 2:
            keep = rng.integers(0, 2, shape[2]).astype(bool)
            keep[int(rng.integers(0, shape[2]))] = True  # at least one visible key: no NaN rows
        mask = (rt.Mask.none(), rt.Mask.causal(), rt.Mask.padding(keep) if keep is not None else None)[kind]
        out = np.zeros_like(q)
        rt.flash_forward_masked(rt.AttentionShape.new(*shape), q, k, v, mask, out)
        _, ref = oracle.naive_forward_masked(q, k, v, mask_kind=kind, keep=keep)
        assert np.abs(out - ref).max() < 1e-3, (shape, kind)
        assert np.all(np.isfinite(out))


@pytest.mark.parametrize("precision,kind", [("f32", 1), ("bf16", 1), ("f32", 2)])
def test_flash_forward_host_entry_on_a_chunked_shape(oracle, precision, kind):
    """A call large enough (50 MB of upload) to be cut into (batch element, head range) chunks with a halving
    tail and pipelined over three streams: causal in both precisions and a padding mask in f32, three heads
    (first, one at a chunk boundary, last) against the oracle."""
    import rustorch_b200 as rt
    shape = (2, 16, 1024, 128)
    n = int(np.prod(shape))
    q, k, v = (oracle.fill_normal(shape, 700 + j).astype(np.float32) for j in range(3))
    keep = None
    if kind == 2:
        keep = (np.random.default_rng(9).random(shape[2]) > 0.3)
        keep[5] = True
    mask = rt.Mask.causal() if kind == 1 else rt.Mask.padding(keep)
    out = np.zeros(shape, dtype=np.float32)
    rt.flash_forward_masked(rt.AttentionShape.new(*shape), q.reshape(-1), k.reshape(-1), v.reshape(-1), mask,
                            out.reshape(-1), precision=precision)
    for b, h in ((0, 0), (1, 8), (1, 15)):
        qs, ks, vs = (t[b:b + 1, h:h + 1] for t in (q, k, v))
        if precision == "bf16":  # the entry rounds its inputs to bf16; the oracle gets the same rounded inputs
            qs, ks, vs = (oracle.round_to_bf16(t) for t in (qs, ks, vs))
        _, ref, _ = oracle.flash_forward_ext(qs, ks, vs, causal=(kind == 1), keep=keep.astype(np.uint8) if keep is not None else None)
        got = out[b:b + 1, h:h + 1]
        if precision == "f32":
            assert np.abs(got - ref).max() < 1e-4, (b, h)
        else:
            util.check_output(got, ref, label=f"chunked host entry b{b} h{h}")
