"""The oracle's extensions beyond the reference API (LSE, combined masks, per-batch lengths, cache decode,
partial merge, bf16 rounding, counter-based inputs), checked against independent numpy math."""
import math

import numpy as np
import pytest


def _np_attention(q, k, v, masked):
    """float64 softmax attention for one (b,h); masked[i,j] True = excluded. Returns (out, lse)."""
    d = q.shape[-1]
    s = (q.astype(np.float64) @ k.astype(np.float64).T) / math.sqrt(d)
    s[masked] = -np.inf
    m = s.max(axis=1, keepdims=True)
    with np.errstate(invalid="ignore"):
        p = np.exp(s - np.where(np.isinf(m), 0.0, m))
    p[masked] = 0.0
    l = p.sum(axis=1, keepdims=True)
    with np.errstate(invalid="ignore", divide="ignore"):
        out = np.where(l > 0, (p @ v.astype(np.float64)) / l, np.nan)
        lse = np.where(l[:, 0] > 0, m[:, 0] + np.log(l[:, 0]), -np.inf)
    return out, lse


@pytest.mark.parametrize("causal,use_keep,use_lens", [(False, False, False), (True, False, False), (False, True, False),
                                                      (True, True, False), (True, False, True), (True, True, True)])
def test_ext_forward_masks_and_lse(oracle, causal, use_keep, use_lens):
    B, H, N, D = 2, 2, 150, 24
    q, k, v = (oracle.fill_normal((B, H, N, D), s) for s in (1, 2, 3))
    rng = np.random.default_rng(0)
    keep = (rng.random((B, N)) > 0.35).astype(np.uint8) if use_keep else None
    if keep is not None:
        keep[:, :70] = 0  # the first 64-key tile (and more) is fully masked
        keep[:, 75] = 1
    lens = np.array([150, 61], dtype=np.int32) if use_lens else None
    rc, out, lse = oracle.flash_forward_ext(q, k, v, causal=causal, keep=keep, kv_lens=lens)
    rc2, out_n, lse_n = oracle.naive_forward_ext(q, k, v, causal=causal, keep=keep, kv_lens=lens)
    assert rc == 0 and rc2 == 0
    for b in range(B):
        masked = np.zeros((N, N), dtype=bool)
        if causal:
            masked |= np.triu(np.ones((N, N), dtype=bool), 1)
        if keep is not None:
            masked |= (keep[b] == 0)[None, :]
        if lens is not None:
            masked |= (np.arange(N) >= lens[b])[None, :]
        for h in range(H):
            ref, ref_lse = _np_attention(q[b, h], k[b, h], v[b, h], masked)
            for got, got_lse in ((out[b, h], lse[b, h]), (out_n[b, h], lse_n[b, h])):
                assert np.array_equal(np.isnan(got), np.isnan(ref))
                ok = ~np.isnan(ref)
                assert not ok.any() or np.abs(got[ok] - ref[ok]).max() < 2e-5
                assert np.array_equal(np.isneginf(got_lse), np.isneginf(ref_lse))
                fin = np.isfinite(ref_lse)
                assert not fin.any() or np.abs(got_lse[fin] - ref_lse[fin]).max() < 2e-5


def test_leading_masked_tile_quirk_is_reproduced_and_fixable(oracle):
    """The reference's tiled path turns a row NaN when its first visited tile is fully masked
    (cpu_forward.rs:380: exp(-inf - -inf)); its naive path does not.  The flag selects which."""
    q, k, v = (oracle.fill_normal((1, 1, 130, 8), s) for s in (4, 5, 6))
    keep = np.ones(130, dtype=np.uint8)
    keep[:64] = 0
    rc, ref_like = oracle.flash_forward_masked(q, k, v, oracle.MASK_PADDING, keep)
    assert rc == 0 and np.isnan(ref_like).all()
    _, naive = oracle.naive_forward_masked(q, k, v, oracle.MASK_PADDING, keep)
    assert np.isfinite(naive).all()
    _, fixed, _ = oracle.flash_forward_ext(q, k, v, keep=keep, fix_leading_masked_tile=True)
    assert np.abs(fixed - naive).max() < 1e-5
    _, unfixed, _ = oracle.flash_forward_ext(q, k, v, keep=keep, fix_leading_masked_tile=False)
    assert np.isnan(unfixed).all()


def test_decode_cache_equals_reference_call_on_trimmed_cache(oracle):
    """Per sequence, the cache decode equals gqa_forward_f32(batch=1, seq_q=1, seq_kv=len) on the trimmed
    cache — the call LlamaModel::decode_step makes (model.rs:638-668)."""
    B, Hq, Hkv, D, S = 3, 8, 2, 16, 64
    q = oracle.fill_normal((B, Hq, D), 1)
    kc, vc = oracle.fill_normal((B, Hkv, S, D), 2), oracle.fill_normal((B, Hkv, S, D), 3)
    lens = np.array([64, 1, 37], dtype=np.int32)
    rc, out, lse = oracle.gqa_decode_cache(q, kc, vc, lens)
    assert rc == 0
    for b in range(B):
        L = int(lens[b])
        rc, ref = oracle.gqa_forward_f32(q[b].ravel(), np.ascontiguousarray(kc[b, :, :L]).ravel(),
                                         np.ascontiguousarray(vc[b, :, :L]).ravel(), 1, Hq, Hkv, 1, L, D)
        assert rc == 0 and np.array_equal(ref.reshape(Hq, D), out[b])
        for h in range(Hq):
            _, ref_lse = _np_attention(q[b, h][None], kc[b, h // 4, :L], vc[b, h // 4, :L], np.zeros((1, L), bool))
            assert abs(lse[b, h] - ref_lse[0]) < 1e-5
    rc, out0, lse0 = oracle.gqa_decode_cache(q, kc, vc, np.zeros(B, np.int32))
    assert np.all(out0 == 0) and np.isneginf(lse0).all()


def test_partial_merge_laws(oracle):
    """combine_tiles laws lifted to (O, LSE) partials: split == unsplit, EMPTY identity, order independence."""
    B, Hq, Hkv, D, S = 1, 8, 2, 32, 512
    q = oracle.fill_normal((B, Hq, D), 7)
    kc, vc = oracle.fill_normal((B, Hkv, S, D), 8), oracle.fill_normal((B, Hkv, S, D), 9)
    lens = np.array([400], dtype=np.int32)
    _, full, full_lse = oracle.gqa_decode_cache(q, kc, vc, lens)
    cuts = [0, 100, 101, 300, 512]
    po, pl = [], []
    for lo, hi in zip(cuts[:-1], cuts[1:]):
        _, o, l = oracle.gqa_decode_cache(q, kc, vc, lens, lo, hi)
        po.append(o.reshape(Hq, D))
        pl.append(l.reshape(Hq))
    po, pl = np.stack(po), np.stack(pl)
    mo, ml = oracle.merge_partials(po, pl)
    assert np.abs(mo - full[0]).max() < 1e-5 and np.abs(ml - full_lse[0]).max() < 1e-5
    perm = [3, 0, 2, 1]
    mo2, ml2 = oracle.merge_partials(po[perm], pl[perm])
    assert np.abs(mo2 - mo).max() < 1e-6 and np.abs(ml2 - ml).max() < 1e-6
    # an empty partial (a rank that holds no visible key) is the identity element
    eo = np.concatenate([po, np.full((1, Hq, D), 123.0, np.float32)])
    el = np.concatenate([pl, np.full((1, Hq), -np.inf, np.float32)])
    mo3, ml3 = oracle.merge_partials(eo, el)
    assert np.array_equal(mo3, mo) and np.array_equal(ml3, ml)
    # nested merge (associativity): ((0,1),(2,3))
    a_o, a_l = oracle.merge_partials(po[:2], pl[:2])
    b_o, b_l = oracle.merge_partials(po[2:], pl[2:])
    mo4, ml4 = oracle.merge_partials(np.stack([a_o, b_o]), np.stack([a_l, b_l]))
    assert np.abs(mo4 - mo).max() < 1e-6 and np.abs(ml4 - ml).max() < 1e-6
    zo, zl = oracle.merge_partials(eo[-1:], el[-1:])
    assert np.all(zo == 0) and np.isneginf(zl).all()


def test_kv_cache_append_indexing(oracle):
    """kv_cache.rs:285-360: offsets, running length, overflow."""
    B, Hkv, S, D = 2, 2, 8, 4
    kc, vc = np.zeros((B, Hkv, S, D), np.float32), np.zeros((B, Hkv, S, D), np.float32)
    k1 = np.arange(B * Hkv * 3 * D, dtype=np.float32).reshape(B, Hkv, 3, D)
    n = oracle.kv_cache_append(kc, vc, k1, -k1, 0)
    assert n == 3 and np.array_equal(kc[:, :, :3], k1) and np.array_equal(vc[:, :, :3], -k1) and not kc[:, :, 3:].any()
    k2 = np.full((B, Hkv, 5, D), 7.0, np.float32)
    assert oracle.kv_cache_append(kc, vc, k2, k2, n) == 8 and np.all(kc[:, :, 3:] == 7.0)
    assert oracle.kv_cache_append(kc, vc, k2[:, :, :1], k2[:, :, :1], 8) == -1


def test_bf16_rounding_is_nearest_even(oracle):
    import torch
    x = np.concatenate([oracle.fill_normal(4096, 11) * 3.0,
                        np.array([1.00390625, 1.01171875, 0.0, -0.0, 65504.0, 1e-40, np.inf], np.float32)])
    ref = torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.array_equal(oracle.round_to_bf16(x), ref)
    assert np.array_equal(oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(x)), ref)
    assert oracle.round_to_bf16(np.array([1.00390625], np.float32))[0] == 1.0       # tie -> even
    assert oracle.round_to_bf16(np.array([1.01171875], np.float32))[0] == 1.015625  # tie -> even (up)


def test_counter_based_inputs(oracle):
    a = oracle.fill_normal(1 << 16, 42)
    assert np.array_equal(a, oracle.fill_normal(1 << 16, 42))
    assert np.array_equal(a[1000:3000], oracle.fill_normal(2000, 42, first_index=1000))  # any shard stands alone
    assert abs(a.mean()) < 0.02 and abs(a.std() - 1.0) < 0.02 and not np.array_equal(a, oracle.fill_normal(1 << 16, 43))
    lens = oracle.fill_uniform_int(4096, 0x5EED, 1024, 8192)
    assert lens.min() >= 1024 and lens.max() <= 8192 and abs(lens.mean() - 4608) < 150


def test_rope_restatement(oracle):
    """rope.rs:162-205 (half-split) and :96-150 (adjacent): position 0 is the identity, a rotation keeps
    pair norms, and the two layouts are the same rotation under the (k, k+D/2) <-> (2k, 2k+1) relabelling."""
    x = oracle.fill_normal((2, 3, 16), 5)
    assert np.array_equal(oracle.rope_token(x, [0, 0]), x)
    pos = np.array([7, 123], dtype=np.int32)
    a = oracle.rope_token(x, pos, 10000.0, 0)
    b = oracle.rope_token(x, pos, 10000.0, 1)
    assert np.allclose(np.hypot(a[..., :8], a[..., 8:]), np.hypot(x[..., :8], x[..., 8:]), atol=1e-5)
    perm = np.concatenate([np.arange(0, 16, 2), np.arange(1, 16, 2)])  # adjacent layout -> half-split layout
    assert np.allclose(oracle.rope_token(x[..., perm], pos, 10000.0, 0), b[..., perm], atol=1e-6)
    # known value: D = 2, pos = 1, theta_0 = 1 -> rotation by 1 radian
    v = oracle.rope_token(np.array([[[1.0, 0.0]]], dtype=np.float32), [1])
    assert np.allclose(v[0, 0], [math.cos(1.0), math.sin(1.0)], atol=1e-6)
