"""Pins the oracle's restatement of flash_backward to the reference's own tests
(crates/rustorch-attention/src/cpu_backward.rs:187-300) and checks the causal extension."""
import numpy as np
import pytest


def _det(orc, shape, seed):
    """deterministic(n, seed) of cpu_backward.rs:190-198 = the LCG fixture with width 2."""
    return orc.fill_lcg(int(np.prod(shape)), seed, 2.0).reshape(shape)


def _finite_diff(orc, which, q, k, v, do_, idx, eps, causal=False):
    """finite_diff_grad of cpu_backward.rs:202-228 (central difference of dO . naive_forward)."""
    arrs = {"q": q, "k": k, "v": v}
    flat = arrs[which].reshape(-1)
    saved = flat[idx]
    kind = 1 if causal else 0
    flat[idx] = saved + np.float32(eps)
    _, o_plus = orc.naive_forward_masked(q, k, v, mask_kind=kind)
    flat[idx] = saved - np.float32(eps)
    _, o_minus = orc.naive_forward_masked(q, k, v, mask_kind=kind)
    flat[idx] = saved
    return float(np.sum(do_.astype(np.float64) * (o_plus.astype(np.float64) - o_minus) / (2 * eps)))


def test_backward_dq_matches_finite_difference(oracle):  # cpu_backward.rs:230-250
    shape = (1, 1, 4, 4)
    q, k, v, do_ = (_det(oracle, shape, s) for s in (1, 2, 3, 4))
    rc, dq, dk, dv = oracle.flash_backward(q, k, v, do_)
    assert rc == 0
    for idx in (0, 5, 10):
        assert abs(dq.reshape(-1)[idx] - _finite_diff(oracle, "q", q, k, v, do_, idx, 1e-3)) < 5e-3
    # the reference spot-checks dQ only; dK and dV obey the same identity
    for idx in (0, 5, 10, 15):
        assert abs(dk.reshape(-1)[idx] - _finite_diff(oracle, "k", q, k, v, do_, idx, 1e-3)) < 5e-3
        assert abs(dv.reshape(-1)[idx] - _finite_diff(oracle, "v", q, k, v, do_, idx, 1e-3)) < 5e-3


def test_backward_empty_seq_is_no_op(oracle):  # cpu_backward.rs:252-260
    e = np.zeros((1, 1, 0, 4), dtype=np.float32)
    rc, dq, dk, dv = oracle.flash_backward(e, e, e, e)
    assert rc == 0 and dq.size == 0


def test_backward_zero_grad_yields_zero_outputs(oracle):  # cpu_backward.rs:280-299
    shape = (1, 1, 3, 4)
    q, k, v = (_det(oracle, shape, s) for s in (1, 2, 3))
    rc, dq, dk, dv = oracle.flash_backward(q, k, v, np.zeros(shape, dtype=np.float32))
    assert rc == 0
    assert not dq.any() and not dk.any() and not dv.any()


@pytest.mark.parametrize("causal", [False, True])
def test_backward_finite_difference_larger_shape(oracle, causal):
    """Same identity on a multi-head shape, for the unmasked case and for the causal extension."""
    shape = (2, 2, 9, 8)
    q, k, v, do_ = (_det(oracle, shape, s) for s in (11, 12, 13, 14))
    rc, dq, dk, dv = oracle.flash_backward(q, k, v, do_, causal=causal)
    assert rc == 0
    rng = np.random.default_rng(0)
    for idx in rng.integers(0, q.size, size=6):
        for which, g in (("q", dq), ("k", dk), ("v", dv)):
            fd = _finite_diff(oracle, which, q, k, v, do_, int(idx), 1e-2, causal=causal)
            assert abs(g.reshape(-1)[idx] - fd) < 5e-3, (which, idx)


def test_backward_lse_matches_forward_lse(oracle):
    shape = (1, 2, 17, 8)
    q, k, v, do_ = (_det(oracle, shape, s) for s in (21, 22, 23, 24))
    rc, _, _, _, lse = oracle.flash_backward(q, k, v, do_, causal=True, with_lse=True)
    _, _, ref_lse = oracle.naive_forward_ext(q, k, v, causal=True)
    assert rc == 0 and np.abs(lse - ref_lse).max() < 1e-5


def test_causal_backward_ignores_future_keys(oracle):
    """With a causal mask the gradient w.r.t. key/value row j only collects queries i >= j: the last
    key row sees one query, the first query row sees one key (so dQ_0 = 0: softmax of one entry)."""
    shape = (1, 1, 6, 4)
    q, k, v, do_ = (_det(oracle, shape, s) for s in (31, 32, 33, 34))
    rc, dq, dk, dv = oracle.flash_backward(q, k, v, do_, causal=True)
    assert rc == 0
    assert np.abs(dq[0, 0, 0]).max() < 1e-7
    # dV_last = P[last,last] * dO_last
    _, _, lse = oracle.naive_forward_ext(q, k, v, causal=True)
    s_ll = float(q[0, 0, 5] @ k[0, 0, 5]) / 2.0
    p_ll = np.exp(s_ll - lse[0, 0, 5])
    assert np.abs(dv[0, 0, 5] - p_ll * do_[0, 0, 5]).max() < 1e-6
