"""Shared helpers of the parity tests: seeded inputs, device transfer, error metrics.

Tolerances (from the target statement of this path): output max-abs <= 1e-2, relative L2 <= 5e-3,
LSE abs <= 1e-3, with bf16-rounded inputs upcast to f32 for the oracle.  One refinement: a bf16
OUTPUT cannot be closer than half an ulp to the true value, and for |o| >= 4 half an ulp is
0.0156 > 1e-2, so the max-abs budget is widened by that half ulp for such elements only.
"""
import numpy as np

SEED_Q, SEED_K, SEED_V, SEED_LEN = 0xC0FFEE, 0xBADBEEF, 0xCAFE00, 0x5EED
TOL_MAX_ABS, TOL_REL_L2, TOL_LSE = 1e-2, 5e-3, 1e-3


def normal_bf16(orc, shape, seed):
    """N(0,1) from the counter-based generator, rounded to bf16 (RNE), stored as f32."""
    return orc.round_to_bf16(orc.fill_normal(shape, seed))


def to_cuda_bf16(x):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).cuda().to(torch.bfloat16).contiguous()


def to_cuda(x):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def to_np(t):
    import torch
    return t.detach().to(torch.float32).cpu().numpy()


def bf16_half_ulp(ref):
    a = np.abs(ref).astype(np.float64)
    e = np.floor(np.log2(np.maximum(a, 1e-30)))
    return np.where(a >= 4.0, 2.0 ** (e - 8), 0.0)


def check_output(got, ref, bf16_out=True, label=""):
    """NaN patterns must match; finite entries within the tolerances. Returns (max_abs, rel_l2)."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, f"{label}: shape {got.shape} vs {ref.shape}"
    nan_g, nan_r = np.isnan(got), np.isnan(ref)
    assert np.array_equal(nan_g, nan_r), f"{label}: NaN pattern differs ({nan_g.sum()} vs {nan_r.sum()})"
    ok = ~nan_r
    if not ok.any():
        return 0.0, 0.0
    d = np.abs(got[ok] - ref[ok])
    budget = TOL_MAX_ABS + (bf16_half_ulp(ref[ok]) if bf16_out else 0.0)
    worst = int(np.argmax(d - budget))
    assert np.all(d <= budget), f"{label}: max-abs {d[worst]:.5f} (ref {ref[ok][worst]:.4f}) over budget"
    rel = float(np.sqrt((d ** 2).sum()) / max(np.sqrt((ref[ok] ** 2).sum()), 1e-30))
    assert rel <= TOL_REL_L2, f"{label}: relative L2 {rel:.3e} > {TOL_REL_L2}"
    return float(d.max()), rel


def check_lse(got, ref, label=""):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    inf_r = np.isneginf(ref)
    assert np.array_equal(np.isneginf(got), inf_r), f"{label}: -inf LSE pattern differs"
    nan_r = np.isnan(ref)
    assert np.array_equal(np.isnan(got), nan_r), f"{label}: NaN LSE pattern differs"
    ok = ~(inf_r | nan_r)
    if ok.any():
        d = np.abs(got[ok] - ref[ok]).max()
        assert d <= TOL_LSE, f"{label}: LSE error {d:.2e} > {TOL_LSE}"
        return float(d)
    return 0.0
