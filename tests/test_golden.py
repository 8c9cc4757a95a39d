"""Committed golden fixtures (tests/golden/, produced by make_golden.py from the oracle) and the reference's
own known-answer vectors (reference_kats.json): the oracle must reproduce them on CPU, the CUDA kernels on GPU."""
import json
import os

import numpy as np
import pytest

from tests import util

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _load(name, orc):
    z = np.load(os.path.join(GOLD, name + ".npz"))
    d = {k: z[k] for k in z.files}
    for k in ("q", "k", "v"):
        d[k] = orc.bf16_bits_to_f32(d[k])
    return d


def _same(a, b, tol=1e-6):
    return np.array_equal(np.isnan(a), np.isnan(b)) and np.array_equal(np.isneginf(a), np.isneginf(b)) and \
        np.nanmax(np.abs(np.where(np.isfinite(a) & np.isfinite(b), a - b, 0.0)), initial=0.0) <= tol


# ------------------------------------------------------------------ CPU: the oracle against the fixtures
def test_oracle_reproduces_golden_prefill(oracle):
    g = _load("prefill_causal_d64", oracle)
    _, out, lse = oracle.flash_forward_ext(g["q"], g["k"], g["v"], causal=True)
    assert _same(out, g["out"]) and _same(lse, g["lse"])
    g = _load("prefill_varlen_d128", oracle)
    _, out, lse = oracle.flash_forward_ext(g["q"], g["k"], g["v"], causal=True, kv_lens=g["kv_lens"])
    assert _same(out, g["out"]) and _same(lse, g["lse"])
    _, out, lse = oracle.naive_forward_ext(g["q"], g["k"], g["v"], causal=True, kv_lens=g["kv_lens"])
    assert _same(out, g["out"], 2e-5) and _same(lse, g["lse"], 2e-5)  # tiled == naive on the fixture too
    g = _load("prefill_keep_d64", oracle)
    _, out, lse = oracle.flash_forward_ext(g["q"], g["k"], g["v"], keep=g["keep"])
    assert _same(out, g["out"]) and _same(lse, g["lse"])
    g = _load("prefill_chunk_gqa_d64", oracle)
    _, out, lse = oracle.attention_general(g["q"], g["k"], g["v"], causal=True, kv_lens=g["kv_lens"],
                                           q_offsets=g["q_offsets"])
    assert _same(out, g["out"]) and _same(lse, g["lse"])


def test_oracle_reproduces_golden_decode(oracle):
    g = _load("decode_gqa_d128", oracle)
    _, out, lse = oracle.gqa_decode_cache(g["q"], g["k"], g["v"], g["kv_lens"])
    assert _same(out, g["out"]) and _same(lse, g["lse"])
    B, Hq, D = out.shape
    mo, ml = oracle.merge_partials(g["part_o"].reshape(2, B * Hq, D), g["part_lse"].reshape(2, B * Hq))
    assert _same(mo.reshape(B, Hq, D), g["out"], 1e-5) and _same(ml.reshape(B, Hq), g["lse"], 1e-5)


def test_oracle_reproduces_golden_backward(oracle):
    g = _load("backward_causal_d64", oracle)
    do_ = oracle.bf16_bits_to_f32(g["d_out"])
    rc, dq, dk, dv, lse = oracle.flash_backward(g["q"], g["k"], g["v"], do_, causal=True, with_lse=True)
    assert rc == 0
    assert _same(dq, g["dq"]) and _same(dk, g["dk"]) and _same(dv, g["dv"]) and _same(lse, g["lse"], 1e-5)


def test_reference_kats_on_the_oracle(oracle):
    kats = json.load(open(os.path.join(GOLD, "reference_kats.json")))
    for name in ("scaling_factor_is_one_over_sqrt_d", "causal_first_query_only_attends_to_self",
                 "padding_mask_excludes_padded_positions_exactly"):
        c = kats[name]
        q, k, v = (np.array(c[x], dtype=np.float32).reshape(c["shape"]) for x in ("q", "k", "v"))
        kind = {"none": oracle.MASK_NONE, "causal": oracle.MASK_CAUSAL, "padding": oracle.MASK_PADDING}[c["mask"]]
        rc, out = oracle.flash_forward_masked(q, k, v, kind, c.get("keep"))
        assert rc == 0
        _check_kat(c, out)
    f = kats["online_softmax_fixtures"]
    m, l = oracle.online_softmax_full(f["huge"])
    assert [m, l] == [np.float32(f["huge_expect"][0]), f["huge_expect"][1]]


def _check_kat(c, out):
    if "expect_out" in c:
        assert np.abs(out.ravel() - np.array(c["expect_out"], dtype=np.float32)).max() <= c["atol"] * 10
    if "expect_row0" in c:
        assert np.abs(out[0, 0, 0] - np.array(c["expect_row0"], dtype=np.float32)).max() <= c["atol"] * 10
    if "expect_out00" in c:
        assert abs(out[0, 0, 0, 0] - c["expect_out00"]) <= c["atol"] * 30


# ------------------------------------------------------------------ GPU: the kernels against the fixtures
@pytest.mark.gpu
@pytest.mark.parametrize("name,kw", [("prefill_causal_d64", dict(causal=True)), ("prefill_varlen_d128", dict(causal=True)),
                                     ("prefill_keep_d64", dict()), ("prefill_chunk_gqa_d64", dict(causal=True))])
def test_gpu_prefill_matches_golden(oracle, name, kw):
    import torch
    import rustorch_b200 as rt
    g = _load(name, oracle)
    args = dict(kw)
    if "kv_lens" in g:
        args["kv_lens"] = util.to_cuda(g["kv_lens"])
    if "q_offsets" in g:
        args["q_offsets"] = util.to_cuda(g["q_offsets"])
    if "keep" in g:
        args["key_keep"] = util.to_cuda(g["keep"])
    out, lse = rt.prefill_bf16(util.to_cuda_bf16(g["q"]), util.to_cuda_bf16(g["k"]), util.to_cuda_bf16(g["v"]), **args)
    torch.cuda.synchronize()
    util.check_output(util.to_np(out), g["out"], label=name)
    util.check_lse(util.to_np(lse), g["lse"], label=name)
    # the f32 CUDA-core kernel on the same fixture, at its own 1e-4 gate
    o32, l32 = rt.prefill_f32(util.to_cuda(g["q"]), util.to_cuda(g["k"]), util.to_cuda(g["v"]), **args)
    got = util.to_np(o32)
    ok = ~np.isnan(g["out"])
    assert np.array_equal(np.isnan(got), ~ok) and np.abs(got[ok] - g["out"][ok]).max() < 1e-4
    util.check_lse(util.to_np(l32), g["lse"], label=name + " f32")


@pytest.mark.gpu
def test_gpu_decode_matches_golden(oracle):
    import torch
    import rustorch_b200 as rt
    g = _load("decode_gqa_d128", oracle)
    dq, dk, dv, dl = util.to_cuda_bf16(g["q"]), util.to_cuda_bf16(g["k"]), util.to_cuda_bf16(g["v"]), util.to_cuda(g["kv_lens"])
    out, lse = rt.gqa_decode(dq, dk, dv, kv_lens=dl)
    util.check_output(util.to_np(out), g["out"], label="decode golden")
    util.check_lse(util.to_np(lse), g["lse"])
    recs = torch.stack([rt.gqa_decode_record(dq, dk, dv, kv_lens=dl, kv_begin=0, kv_end=64),
                        rt.gqa_decode_record(dq, dk, dv, kv_lens=dl, kv_begin=64, kv_end=-1)])
    B, Hq, D = g["out"].shape
    util.check_output(util.to_np(recs[:, :, :D]).reshape(2, B, Hq, D), g["part_o"], bf16_out=False, label="shard partials")
    util.check_lse(util.to_np(recs[:, :, D]).reshape(2, B, Hq), g["part_lse"])
    merged, mlse = rt.merge_records(recs, out_dtype=torch.float32)
    util.check_output(util.to_np(merged).reshape(B, Hq, D), g["out"], bf16_out=False)
    util.check_lse(util.to_np(mlse).reshape(B, Hq), g["lse"])


@pytest.mark.gpu
def test_gpu_reference_kats_through_the_host_mirror():
    import rustorch_b200 as rt
    kats = json.load(open(os.path.join(GOLD, "reference_kats.json")))
    for name in ("scaling_factor_is_one_over_sqrt_d", "causal_first_query_only_attends_to_self",
                 "padding_mask_excludes_padded_positions_exactly"):
        c = kats[name]
        q, k, v = (np.array(c[x], dtype=np.float32).reshape(c["shape"]) for x in ("q", "k", "v"))
        mask = {"none": rt.Mask.none(), "causal": rt.Mask.causal(),
                "padding": rt.Mask.padding(c.get("keep", []))}[c["mask"]]
        out = np.zeros_like(q)
        rt.flash_forward_masked(rt.AttentionShape.new(*c["shape"]), q, k, v, mask, out)
        _check_kat(c, out)


@pytest.mark.gpu
def test_gpu_backward_matches_golden(oracle):
    """Both CUDA backward kernels against the committed gradients: f32 at 2e-4, bf16 tensor cores at 2e-2 of the
    largest entry."""
    import torch
    import rustorch_b200 as rt
    g = _load("backward_causal_d64", oracle)
    do_ = oracle.bf16_bits_to_f32(g["d_out"])
    q, k, v, d = (torch.from_numpy(x).cuda() for x in (g["q"], g["k"], g["v"], do_))
    out, lse = rt.prefill_f32(q, k, v, causal=True)
    got = rt.backward_f32(q, k, v, out, d, lse, causal=True)
    qh, kh, vh, dh = (x.to(torch.bfloat16) for x in (q, k, v, d))
    outh, lseh = rt.prefill_bf16(qh, kh, vh, causal=True)
    goth = rt.backward_bf16(qh, kh, vh, outh, dh, lseh, causal=True)
    torch.cuda.synchronize()
    assert np.abs(lse.cpu().numpy() - g["lse"]).max() < 1e-4
    for name, a, b in zip(("dq", "dk", "dv"), got, goth):
        ref = g[name]
        scale = max(1.0, float(np.abs(ref).max()))
        assert np.abs(a.cpu().numpy() - ref).max() <= 2e-4 * scale, name
        assert np.abs(b.cpu().numpy() - ref).max() <= 2e-2 * scale, name


# ---- outputs of the reference's own CUDA decode kernel (see tests/golden/make_ref_decode_golden.py)
def _ref_decode_fixture():
    import importlib.util
    path = os.path.join(GOLD, "decode_ref_kernel.npz")
    if not os.path.exists(path):
        pytest.skip("decode_ref_kernel.npz not generated yet (needs one GPU run of make_ref_decode_golden.py)")
    spec = importlib.util.spec_from_file_location("make_ref_decode_golden",
                                                  os.path.join(GOLD, "make_ref_decode_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return np.load(path), mod


def _bf16_bits_to_f32(bits):
    return (bits.astype(np.uint32) << 16).view(np.float32)


def test_oracle_decode_matches_reference_kernel_outputs(oracle):
    """The oracle's decode_attn_row restatement against what the reference's CUDA kernel itself returned
    (bf16 outputs, fast-math exp): max-abs 1e-2 (+ half a bf16 ulp where |o| >= 4), relative L2 5e-3."""
    data, mod = _ref_decode_fixture()
    for i, case in enumerate(data["cases"].tolist()):
        q, k, v = mod.inputs(oracle, case)
        rc, out, _ = oracle.gqa_decode_cache(q[None], k[None], v[None], np.array([case[4]], dtype=np.int32))
        assert rc == 0
        util.check_output(_bf16_bits_to_f32(data[f"out_{i}"]), out[0], label=f"reference kernel case {case}")


@pytest.mark.gpu
def test_dropin_decode_matches_reference_kernel_outputs(oracle):
    import torch
    import rustorch_b200 as rt
    data, mod = _ref_decode_fixture()
    for i, case in enumerate(data["cases"].tolist()):
        Hq, Hkv, D, S, L, _ = case
        q, k, v = mod.inputs(oracle, case)
        dq, dk, dv = (util.to_cuda_bf16(x) for x in (q, k, v))
        out = torch.empty((Hq, D), dtype=torch.bfloat16, device="cuda")
        rt.LlmKernels().gqa_decode_online_bf16(torch.cuda.current_stream(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                               out.data_ptr(), Hq, Hkv, L, D, S)
        torch.cuda.synchronize()
        util.check_output(util.to_np(out), _bf16_bits_to_f32(data[f"out_{i}"]), label=f"drop-in vs reference {case}")
