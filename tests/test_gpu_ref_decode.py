"""Decode parity pinned to the reference itself: the reference's own CUDA C kernels
(crates/rustorch-cuda/src/llm_kernels.rs:106-145, 345-458), compiled unchanged into a test-only
library by oracle/build_ref.py, run next to the CPU oracle and the library's drop-in entry points
on the batch-1 call shapes of the reference model (crates/rustorch-llm/src/cuda_backend.rs:946-987)
and of its decode microbenchmark (crates/rustorch-llm/examples/kernel_microbench.rs:1070-1072).

Three-way check per case:
  reference kernel  vs  oracle (decode_attn_row restatement)   -> the oracle's decode is the reference's
  rt_gqa_decode_online_bf16  vs  reference kernel              -> the drop-in returns what the reference returns
  rt_gqa_decode_online_bf16  vs  oracle                        -> the usual parity gate
All three at output max-abs <= 1e-2 (+ half a bf16 ulp where |o| >= 4) and relative L2 <= 5e-3.
"""
import numpy as np
import pytest

from tests import util

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref_cuda():
    from oracle import ref_cuda as rc
    if not rc.available():
        pytest.skip("oracle/_ref/libref_llm_kernels.so not built (needs the reference checkout at build time)")
    return rc


def _case(orc, Hq, Hkv, D, S):
    q = util.normal_bf16(orc, (1, Hq, D), util.SEED_Q)
    k = util.normal_bf16(orc, (1, Hkv, S, D), util.SEED_K)
    v = util.normal_bf16(orc, (1, Hkv, S, D), util.SEED_V)
    return q, k, v


@pytest.mark.parametrize("Hq,Hkv,D", [(32, 8, 128), (16, 2, 256), (8, 8, 64)])
@pytest.mark.parametrize("kv_len", [1, 63, 1000, 8192])
def test_reference_kernel_oracle_and_dropin_agree(oracle, ref_cuda, Hq, Hkv, D, kv_len):
    import torch
    import rustorch_b200 as rt
    S = 8192
    q, k, v = _case(oracle, Hq, Hkv, D, S)
    dq, dk, dv = util.to_cuda_bf16(q[0]), util.to_cuda_bf16(k[0]), util.to_cuda_bf16(v[0])

    ref_out = ref_cuda.gqa_decode_online_bf16(dq, dk, dv, kv_len)

    ours = torch.empty((Hq, D), dtype=torch.bfloat16, device="cuda")
    rt.LlmKernels().gqa_decode_online_bf16(torch.cuda.current_stream(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                           ours.data_ptr(), Hq, Hkv, kv_len, D, S)
    torch.cuda.synchronize()

    rc, orc_out, _ = oracle.gqa_decode_cache(q, k, v, np.array([kv_len], dtype=np.int32))
    assert rc == 0
    label = f"Hq{Hq} Hkv{Hkv} D{D} kv{kv_len}"
    util.check_output(util.to_np(ref_out), orc_out[0], label=f"reference kernel vs oracle, {label}")
    util.check_output(util.to_np(ours), util.to_np(ref_out), label=f"drop-in vs reference kernel, {label}")
    util.check_output(util.to_np(ours), orc_out[0], label=f"drop-in vs oracle, {label}")


def test_reference_kv_append_is_bit_identical(oracle, ref_cuda):
    import torch
    import rustorch_b200 as rt
    Hkv, D, S = 8, 128, 256
    _, k, v = _case(oracle, 8, Hkv, D, S)
    k_new = util.to_cuda_bf16(util.normal_bf16(oracle, (Hkv, D), 31))
    v_new = util.to_cuda_bf16(util.normal_bf16(oracle, (Hkv, D), 32))
    rk, rv = util.to_cuda_bf16(k[0]), util.to_cuda_bf16(v[0])
    ok, ov = rk.clone(), rv.clone()
    kern = rt.LlmKernels()
    for pos in (0, 100, S - 1):
        ref_cuda.kv_append_bf16(rk, rv, k_new, v_new, pos)
        kern.kv_append_bf16(torch.cuda.current_stream(), ok.data_ptr(), ov.data_ptr(), k_new.data_ptr(),
                            v_new.data_ptr(), pos, Hkv, D, S)
    torch.cuda.synchronize()
    assert torch.equal(rk, ok) and torch.equal(rv, ov)


def test_reference_rope_matches_adjacent_style(oracle, ref_cuda):
    """The reference kernel named rope_half_split_bf16 rotates adjacent pairs (2p, 2p+1); the fused
    rope + append entry reproduces it with style "adjacent" (one bf16 ulp: fast-math sincos there)."""
    import torch
    import rustorch_b200 as rt
    Hq, Hkv, D, S = 8, 2, 128, 512
    inv_freq = rt.rope_inv_freq(D, 10000.0)
    for pos in (0, 7, 300):
        q = util.normal_bf16(oracle, (1, Hq, D), 41 + pos)
        k_new = util.normal_bf16(oracle, (1, Hkv, D), 42 + pos)
        v_new = util.normal_bf16(oracle, (1, Hkv, D), 43 + pos)
        rq, rk = util.to_cuda_bf16(q[0]), util.to_cuda_bf16(k_new[0])
        ref_cuda.rope_half_split_bf16(rq, inv_freq, pos)
        ref_cuda.rope_half_split_bf16(rk, inv_freq, pos)
        oq = util.to_cuda_bf16(q)
        kc = torch.zeros((1, Hkv, S, D), dtype=torch.bfloat16, device="cuda")
        vc = torch.zeros_like(kc)
        rt.rope_kv_append(oq, util.to_cuda_bf16(k_new), util.to_cuda_bf16(v_new), kc, vc, inv_freq, pos=pos,
                          style="adjacent")
        torch.cuda.synchronize()
        tol = 2.0 ** -7 * max(np.abs(q).max(), np.abs(k_new).max())
        assert np.abs(util.to_np(oq[0]) - util.to_np(rq)).max() <= tol
        assert np.abs(util.to_np(kc[0, :, pos]) - util.to_np(rk)).max() <= tol
