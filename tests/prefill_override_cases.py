"""Prefill cases that run under launch overrides (RT_ATTN_PREFILL_SCHED, RT_ATTN_PREFILL_TILES).

The library reads those variables once per process, so tests/test_gpu_prefill_tc.py runs this file in a
child pytest process per override (it is not collected by the default `pytest tests` pattern).  Every case is
checked against the CPU oracle; the parent passes the override in the environment.
"""
import numpy as np
import pytest

from tests import util
from tests.test_gpu_prefill_tc import _qkv, _run_tc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", ["odd_blocks_causal", "gqa_chunk_offsets", "varlen", "no_mask"])
def test_schedule_cases(oracle, case):
    """Both launch schedules of the kernel (one CTA per SM walking a paired list of 256-row blocks, or one CTA per
    block) on shapes that stress the list: an odd number of blocks per head (the middle block has no partner),
    grouped KV heads with per-batch causal offsets, per-batch lengths, and no mask at all."""
    import os
    sched = os.environ.get("RT_ATTN_PREFILL_SCHED", "default")
    if case == "odd_blocks_causal":
        B, Hq, Hkv, Nq, Nkv, D = 40, 8, 8, 1280, 1280, 128    # 320 heads x 5 blocks: more slots than SMs
        kw, okw = dict(causal=True), dict(causal=True)
    elif case == "gqa_chunk_offsets":
        B, Hq, Hkv, Nq, Nkv, D = 3, 8, 2, 700, 2048, 64
        lens = np.array([2048, 700, 1500], dtype=np.int32)
        offs = (lens - Nq).astype(np.int32)
        kw = dict(causal=True, kv_lens=util.to_cuda(lens), q_offsets=util.to_cuda(offs))
        okw = dict(causal=True, kv_lens=lens, q_offsets=offs)
    elif case == "varlen":
        B, Hq, Hkv, Nq, Nkv, D = 6, 4, 4, 900, 900, 64
        lens = np.array([900, 1, 257, 640, 0, 333], dtype=np.int32)
        kw, okw = dict(causal=True, kv_lens=util.to_cuda(lens)), dict(causal=True, kv_lens=lens)
    else:
        B, Hq, Hkv, Nq, Nkv, D = 2, 5, 5, 777, 777, 128
        kw, okw = dict(), dict()
    if case == "odd_blocks_causal":   # the oracle is O(N^2) per head: check 6 of the 320 heads
        q = util.normal_bf16(oracle, (B, Hq, Nq, D), util.SEED_Q)
        k = util.normal_bf16(oracle, (B, Hkv, Nkv, D), util.SEED_K)
        v = util.normal_bf16(oracle, (B, Hkv, Nkv, D), util.SEED_V)
        out, lse = _run_tc(q, k, v, **kw)
        for b, h in ((0, 0), (0, 7), (17, 3), (39, 0), (39, 7), (20, 5)):
            _, ref, ref_lse = oracle.attention_general(q[b:b + 1, h:h + 1], k[b:b + 1, h:h + 1], v[b:b + 1, h:h + 1], **okw)
            util.check_output(out[b:b + 1, h:h + 1], ref, label=f"{case} {sched} b{b} h{h}")
            util.check_lse(lse[b:b + 1, h:h + 1], ref_lse)
        return
    q = util.normal_bf16(oracle, (B, Hq, Nq, D), util.SEED_Q)
    k = util.normal_bf16(oracle, (B, Hkv, Nkv, D), util.SEED_K)
    v = util.normal_bf16(oracle, (B, Hkv, Nkv, D), util.SEED_V)
    out, lse = _run_tc(q, k, v, **kw)
    _, ref, ref_lse = oracle.attention_general(q, k, v, **okw)
    util.check_output(out, ref, label=f"{case} {sched}")
    util.check_lse(lse, ref_lse)


@pytest.mark.parametrize("D,N,causal", [(64, 2048, True), (128, 300, False), (128, 129, True)])
def test_item_size_cases(oracle, D, N, causal):
    """Small launches hand each CTA one 128-row Q tile instead of two (more CTAs for the same rows); both item
    sizes give the same numbers."""
    import os
    tiles = os.environ.get("RT_ATTN_PREFILL_TILES", "default")
    q, k, v = _qkv(oracle, (1, 3, N, D))
    out, lse = _run_tc(q, k, v, causal=causal)
    _, ref, ref_lse = oracle.flash_forward_ext(q, k, v, causal=causal)
    util.check_output(out, ref, label=f"tiles={tiles} N{N} D{D}")
    util.check_lse(lse, ref_lse)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("causal", [False, True])
def test_key_split_edges(oracle, D, causal):
    """Per-sequence lengths around the 64- and 128-key boundaries: with 128-row items the two tiles of a CTA take
    the even and the odd 64-key steps, so these lengths give a tile no step, one step more than the other, or
    the same number; length 0 rows are NaN with LSE -inf."""
    lens = np.array([0, 1, 63, 64, 65, 127, 128, 129, 191, 192, 193, 255, 256], dtype=np.int32)
    B, H, N = len(lens), 1, 256
    q, k, v = _qkv(oracle, (B, H, N, D))
    out, lse = _run_tc(q, k, v, causal=causal, kv_lens=util.to_cuda(lens))
    _, ref, ref_lse = oracle.flash_forward_ext(q, k, v, causal=causal, kv_lens=lens)
    util.check_output(out, ref, label=f"key split edges D{D} causal={causal}")
    util.check_lse(lse, ref_lse)
