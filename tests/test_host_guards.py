"""The decode-side Python wrappers refuse tensors the kernels would misread, before any launch.

The kernels take raw device pointers: a CPU tensor would give them a host address, an int64 length
vector or a non-contiguous cache would be read as dense int32 / bf16 data.  None of these may reach
the C ABI.  The CPU tests need no GPU because the guard trips on the first argument it looks at.
"""
import pytest
import torch

import rustorch_b200 as rt
from rustorch_b200 import gqa


def test_cpu_tensors_are_rejected_without_a_launch():
    q = torch.zeros((1, 4, 64), dtype=torch.bfloat16)
    kc = torch.zeros((1, 2, 16, 64), dtype=torch.bfloat16)
    with pytest.raises(TypeError, match="CUDA"):
        rt.gqa_decode(q, kc, kc, kv_len=3)
    with pytest.raises(TypeError, match="CUDA"):
        rt.gqa_decode_record(q, kc, kc, kv_len=3)
    with pytest.raises(TypeError, match="CUDA"):
        rt.kv_append(kc, kc, q[:, :2], q[:, :2], pos=0)
    with pytest.raises(TypeError, match="CUDA"):
        rt.rope_kv_append(q, q[:, :2], q[:, :2], kc, kc, torch.zeros(32), pos=0)
    with pytest.raises(TypeError, match="CUDA"):
        rt.merge_records(torch.zeros((2, 4, 65)))


def test_guard_checks_dtype_contiguity_shape():
    lens = torch.tensor([1, 2])  # int64, CPU: what torch.tensor(list_of_lengths) gives
    with pytest.raises(TypeError, match="CUDA"):
        gqa._guard("kv_lens", lens, torch.int32)
    with pytest.raises(TypeError, match="torch.Tensor"):
        gqa._guard("kv_lens", [1, 2], torch.int32)


@pytest.mark.gpu
def test_cuda_q_with_bad_companions_is_rejected():
    q = torch.zeros((2, 4, 64), dtype=torch.bfloat16, device="cuda")
    kc = torch.zeros((2, 2, 16, 64), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(TypeError, match="kv_lens"):
        rt.gqa_decode(q, kc, kc, kv_lens=torch.tensor([3, 4], dtype=torch.int32))  # CPU lengths
    with pytest.raises(TypeError, match="kv_lens"):
        rt.gqa_decode(q, kc, kc, kv_lens=torch.tensor([3, 4], device="cuda"))       # int64 lengths
    with pytest.raises(TypeError, match="k_cache"):
        rt.gqa_decode(q, kc.half(), kc.half(), kv_len=3)                            # fp16 cache
    with pytest.raises(TypeError, match="contiguous"):
        rt.gqa_decode(q, kc.transpose(1, 2), kc.transpose(1, 2), kv_len=3)          # permuted cache
    with pytest.raises(TypeError, match="v_cache"):
        rt.gqa_decode(q, kc, kc[:, :, :8].contiguous(), kv_len=3)                   # K / V shapes differ
    with pytest.raises(TypeError, match="positions"):
        rt.kv_append(kc, kc.clone(), q[:, :2].contiguous(), q[:, :2].contiguous(),
                     positions=torch.tensor([0, 1], dtype=torch.int32))
    out, _ = rt.gqa_decode(q, kc, kc, kv_lens=torch.tensor([3, 4], dtype=torch.int32, device="cuda"))
    torch.cuda.synchronize()
    assert out.shape == (2, 4, 64)
