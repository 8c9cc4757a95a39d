"""The allocation-free decode entry (rt_gqa_decode_online_bf16_static) against the ordinary one.

Some callers of the decode cannot give it scratch memory: a binding that keeps the reference's
ten-argument gqa_decode_online_bf16 signature has no parameter for it, and a serving runtime that
handed all device memory to its own pools may not call cudaMalloc in its decode loop.  For them the
library carries its own 8 MiB scratch array.  This test calls that entry through the C ABI twice in a
row (the second problem is shorter, so slots written by the first call stay behind in the shared
array) and requires bit-identical output to the entry that takes a caller workspace.

Collected last on purpose (file name), so a run that stops at the first failure has already run
every other test.  It passes alone in a fresh process and after the rest of the suite.
"""
import pytest

pytestmark = pytest.mark.gpu


def test_static_scratch_decode_matches_workspace_decode_twice():
    import torch
    import rustorch_b200 as rt
    from rustorch_b200 import _lib

    Hq, Hkv, D, S = 32, 8, 128, 8192
    g = torch.Generator(device="cuda").manual_seed(99)
    kc = torch.randn((Hkv, S, D), device="cuda", generator=g).to(torch.bfloat16)
    vc = torch.randn((Hkv, S, D), device="cuda", generator=g).to(torch.bfloat16)
    kern = rt.LlmKernels()
    stream = torch.cuda.current_stream()
    # One call up front: module load and the per-device symbol lookup happen on the first call, and they may
    # take device memory of their own.  What is checked below is the steady state of a decode loop.
    warm_q = torch.zeros((Hq, D), dtype=torch.bfloat16, device="cuda")
    warm_o = torch.empty_like(warm_q)
    rt.gqa_decode_online_bf16_static(stream, warm_q.data_ptr(), kc.data_ptr(), vc.data_ptr(), warm_o.data_ptr(), Hq,
                                     Hkv, 256, D, S)
    torch.cuda.synchronize()
    for kv_len in (8000, 700):  # 63 chunks of 128 tokens, then 6: the second call must ignore the first call's leftovers
        q = torch.randn((Hq, D), device="cuda", generator=g).to(torch.bfloat16)
        ref = torch.empty((Hq, D), dtype=torch.bfloat16, device="cuda")
        got = torch.full((Hq, D), float("nan"), dtype=torch.bfloat16, device="cuda")
        kern.gqa_decode_online_bf16(stream, q.data_ptr(), kc.data_ptr(), vc.data_ptr(), ref.data_ptr(), Hq, Hkv,
                                    kv_len, D, S)
        torch.cuda.synchronize()
        # Free device memory as the driver reports it (cudaMemGetInfo): unlike torch's own counter this also
        # sees a cudaMalloc made inside the library.  No torch allocation happens between the two readings.
        free_before, _ = torch.cuda.mem_get_info()
        torch_before = torch.cuda.memory_allocated()
        rt.gqa_decode_online_bf16_static(stream, q.data_ptr(), kc.data_ptr(), vc.data_ptr(), got.data_ptr(), Hq, Hkv,
                                         kv_len, D, S)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after >= free_before, f"the call took {free_before - free_after} bytes of device memory"
        assert torch.cuda.memory_allocated() == torch_before
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, ref), f"kv_len={kv_len}: max diff {(got.float() - ref.float()).abs().max().item()}"
        # and it is the right answer, not merely the same one
        kk = kc[:, :kv_len].float().repeat_interleave(Hq // Hkv, dim=0)
        vv = vc[:, :kv_len].float().repeat_interleave(Hq // Hkv, dim=0)
        s = torch.einsum("hd,hld->hl", q.float(), kk) / (D ** 0.5)
        exact = torch.einsum("hl,hld->hd", torch.softmax(s, dim=-1), vv)
        assert (got.float() - exact).abs().max().item() <= 1e-2
    assert _lib.device_status() == 0


def test_static_scratch_decode_rejects_oversized_problems():
    import torch
    import rustorch_b200 as rt
    from rustorch_b200 import _lib

    t = torch.zeros((8, 64, 128), dtype=torch.bfloat16, device="cuda")
    q = torch.zeros((32, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.CudaError) as e:  # 1024 chunks x 32 heads x 129 floats = 16.9 MB > 8 MiB
        rt.gqa_decode_online_bf16_static(torch.cuda.current_stream(), q.data_ptr(), t.data_ptr(), t.data_ptr(),
                                         q.data_ptr(), 32, 8, 10, 128, 1 << 20)
    assert e.value.code == _lib.RT_ERR_STATIC_SCRATCH and "8388608" in str(e.value)
