"""GPU parity of the f32 flash-attention backward against the oracle's restatement of
flash_backward (crates/rustorch-attention/src/cpu_backward.rs:46-185)."""
import numpy as np
import pytest

from tests import util

pytestmark = pytest.mark.gpu

# f32 arithmetic on both sides; the tiled kernel sums in a different order than the reference's
# j-major loops, so the gate is the reference's forward equivalence gate scaled to gradient size.
TOL = 2e-4


def _det(orc, shape, seed, width=2.0):
    return orc.fill_lcg(int(np.prod(shape)), seed, width).reshape(shape)


def _gpu_backward(q, k, v, do_, causal):
    import torch
    import rustorch_b200 as rt
    dq_, dk_, dv_, ddo = (util.to_cuda(x) for x in (q, k, v, do_))
    out, lse = rt.prefill_f32(dq_, dk_, dv_, causal=causal)
    gq, gk, gv = rt.backward_f32(dq_, dk_, dv_, out, ddo, lse, causal=causal)
    torch.cuda.synchronize()
    return util.to_np(gq), util.to_np(gk), util.to_np(gv)


def _check(got, ref, label):
    d = np.abs(got.astype(np.float64) - ref)
    scale = max(1.0, float(np.abs(ref).max()))
    assert d.max() <= TOL * scale, f"{label}: max abs {d.max():.3e} (ref magnitude {scale:.3f})"


@pytest.mark.parametrize("shape", [(1, 1, 4, 4), (1, 2, 33, 16), (2, 3, 64, 64), (1, 2, 130, 128), (1, 1, 100, 256),
                                   (2, 2, 257, 40)])
@pytest.mark.parametrize("causal", [False, True])
def test_backward_f32_matches_oracle(oracle, shape, causal):
    q, k, v, do_ = (_det(oracle, shape, s) for s in (1, 2, 3, 4))
    rc, rq, rk, rv = oracle.flash_backward(q, k, v, do_, causal=causal)
    assert rc == 0
    gq, gk, gv = _gpu_backward(q, k, v, do_, causal)
    _check(gq, rq, f"dq {shape} causal={causal}")
    _check(gk, rk, f"dk {shape} causal={causal}")
    _check(gv, rv, f"dv {shape} causal={causal}")


def test_backward_host_entry_reference_kats(oracle):
    """cpu_backward.rs:230-299 through the host mirror of flash_backward."""
    import rustorch_b200 as rt
    shape = rt.AttentionShape.new(1, 1, 4, 4)
    dims = (1, 1, 4, 4)
    q, k, v, do_ = (_det(oracle, dims, s) for s in (1, 2, 3, 4))
    dq, dk, dv = (np.zeros(dims, dtype=np.float32) for _ in range(3))
    rt.flash_backward(shape, q, k, v, do_, dq, dk, dv)
    rc, rq, rk, rv = oracle.flash_backward(q, k, v, do_)
    assert np.abs(dq - rq).max() < 1e-5 and np.abs(dk - rk).max() < 1e-5 and np.abs(dv - rv).max() < 1e-5
    # backward_dq_matches_finite_difference: indices 0, 5, 10, eps 1e-3, gate 5e-3
    for idx in (0, 5, 10):
        flat = q.reshape(-1)
        s = flat[idx]
        flat[idx] = s + np.float32(1e-3)
        _, op = oracle.naive_forward_masked(q, k, v)
        flat[idx] = s - np.float32(1e-3)
        _, om = oracle.naive_forward_masked(q, k, v)
        flat[idx] = s
        fd = float(np.sum(do_ * (op - om) / 2e-3))
        assert abs(dq.reshape(-1)[idx] - fd) < 5e-3
    # backward_zero_grad_yields_zero_outputs
    shape3 = rt.AttentionShape.new(1, 1, 3, 4)
    q, k, v = (_det(oracle, (1, 1, 3, 4), s) for s in (1, 2, 3))
    dq, dk, dv = (np.ones((1, 1, 3, 4), dtype=np.float32) for _ in range(3))
    rt.flash_backward(shape3, q, k, v, np.zeros((1, 1, 3, 4), dtype=np.float32), dq, dk, dv)
    assert not dq.any() and not dk.any() and not dv.any()
    # backward_empty_seq_is_no_op
    e = np.zeros((0,), dtype=np.float32)
    rt.flash_backward(rt.AttentionShape.new(1, 1, 0, 4), e, e, e, e, e.copy(), e.copy(), e.copy())
    # backward_shape_mismatch_returns_error
    with pytest.raises(rt.BufferShapeMismatch) as err:
        z = np.zeros(16, dtype=np.float32)
        rt.flash_backward(shape, np.zeros(10, dtype=np.float32), z, z, z, z.copy(), z.copy(), z.copy())
    assert err.value.which == "q" and err.value.expected == 16 and err.value.got == 10
    with pytest.raises(rt.OutputShapeMismatch):
        rt.flash_backward(shape, z, z, z, z, np.zeros(8, dtype=np.float32), z.copy(), z.copy())


def test_backward_linearity_and_full_size_property(oracle):
    """Size-independent properties at a size the O(N^2)-memory oracle cannot reach: the gradients are
    linear in dO, and sum_j dV_j = sum_i dO_i (every probability row sums to 1)."""
    import torch
    import rustorch_b200 as rt
    B, H, N, D = 1, 4, 2048, 64
    g = torch.Generator(device="cuda").manual_seed(5)
    q, k, v, d1, d2 = (torch.randn((B, H, N, D), device="cuda", generator=g) for _ in range(5))
    out, lse = rt.prefill_f32(q, k, v, causal=True)
    a = rt.backward_f32(q, k, v, out, d1, lse, causal=True)
    b = rt.backward_f32(q, k, v, out, d2, lse, causal=True)
    c = rt.backward_f32(q, k, v, out, d1 + 2 * d2, lse, causal=True)
    torch.cuda.synchronize()
    for x, y, z in zip(a, b, c):
        assert (x + 2 * y - z).abs().max().item() < 2e-4 * max(1.0, z.abs().max().item())
    assert (a[2].sum(dim=2) - d1.sum(dim=2)).abs().max().item() < 1e-2


def _rel_l2(got, ref):
    return float(np.sqrt(((got.astype(np.float64) - ref) ** 2).sum()) / max(1e-30, np.sqrt((ref.astype(np.float64) ** 2).sum())))


@pytest.mark.parametrize("shape", [(1, 2, 64, 64), (2, 2, 200, 64), (1, 3, 257, 128), (2, 1, 512, 128), (1, 1, 1, 64)])
@pytest.mark.parametrize("causal", [False, True])
def test_backward_bf16_tensor_core_matches_oracle(oracle, shape, causal):
    """bf16 operands, P and dS rounded to bf16 inside the kernel (as the forward rounds P), delta from the bf16
    forward output: gradients within 2e-2 of the largest reference entry and 1e-2 in relative L2."""
    import torch
    import rustorch_b200 as rt
    q, k, v, do_ = (util.normal_bf16(oracle, shape, s) for s in (util.SEED_Q, util.SEED_K, util.SEED_V, 0xD0))
    rc, rq, rk, rv = oracle.flash_backward(q, k, v, do_, causal=causal)
    assert rc == 0
    dq_, dk_, dv_, ddo = (util.to_cuda_bf16(x) for x in (q, k, v, do_))
    out, lse = rt.prefill_bf16(dq_, dk_, dv_, causal=causal)
    gq, gk, gv = rt.backward_bf16(dq_, dk_, dv_, out, ddo, lse, causal=causal)
    torch.cuda.synchronize()
    for name, got, ref in (("dq", gq, rq), ("dk", gk, rk), ("dv", gv, rv)):
        got = util.to_np(got)
        assert np.all(np.isfinite(got)), name
        lim = 2e-2 * max(1.0, float(np.abs(ref).max()))
        assert np.abs(got - ref).max() <= lim, f"{name} {shape} causal={causal}: {np.abs(got - ref).max():.3e} > {lim:.3e}"
        if shape[2] > 1:
            assert _rel_l2(got, ref) <= 1e-2, f"{name} {shape} causal={causal}: rel L2 {_rel_l2(got, ref):.3e}"


def test_backward_bf16_agrees_with_f32_kernel_at_size(oracle):
    """At a size beyond the O(N^2)-memory oracle the two CUDA backward kernels (f32 CUDA cores, bf16 tensor
    cores) are compared with each other on the same bf16-representable inputs."""
    import torch
    import rustorch_b200 as rt
    B, H, N, D = 1, 2, 1536, 128
    g = torch.Generator(device="cuda").manual_seed(9)
    q, k, v, do_ = (torch.randn((B, H, N, D), device="cuda", generator=g).to(torch.bfloat16) for _ in range(4))
    out, lse = rt.prefill_bf16(q, k, v, causal=True)
    a = rt.backward_bf16(q, k, v, out, do_, lse, causal=True)
    of, lf = rt.prefill_f32(q.float(), k.float(), v.float(), causal=True)
    b = rt.backward_f32(q.float(), k.float(), v.float(), of, do_.float(), lf, causal=True)
    torch.cuda.synchronize()
    for x, y in zip(a, b):
        rel = ((x - y).double().norm() / y.double().norm()).item()
        assert rel < 1e-2, rel
