"""Two-GPU test of the split-KV decode exchange (skipped where fewer than two GPUs are visible): every rank
decodes its KV shard, the ranks exchange the packed (O | LSE) records over peer memory
(rt_splitkv_push_record + rt_attn_merge_records_after) and over NCCL, and both must give every rank the
result of a single-GPU decode over the whole range."""
import os
import socket

import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, tmpdir):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"   # plain peer stores and ring collectives only
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import rustorch_b200 as rt
        from rustorch_b200 import _lib, sharding
        Hq, Hkv, D, T = 32, 8, 128, 4096 * world
        g = torch.Generator(device="cuda").manual_seed(7)   # the same data on every rank
        q = torch.randn((1, Hq, D), device="cuda", generator=g).to(torch.bfloat16)
        k = torch.randn((1, Hkv, T, D), device="cuda", generator=g).to(torch.bfloat16)
        v = torch.randn((1, Hkv, T, D), device="cuda", generator=g).to(torch.bfloat16)
        lo, hi = sharding.kv_shard(T, world, rank, align=16)
        full, full_lse = rt.gqa_decode(q, k, v, kv_len=T, out_dtype=torch.float32)
        ex = sharding.PeerRecordExchange.create(Hq, D)
        for step in range(3):   # three epochs: both slot sets are reused
            rec = rt.gqa_decode_record(q, k, v, kv_len=T, kv_begin=lo, kv_end=hi)
            want, want_lse = rt.merge_records(sharding.all_gather_partials(rec), out_dtype=torch.float32)
            rt.gqa_decode_record(q, k, v, kv_len=T, kv_begin=lo, kv_end=hi, record=ex.next_epoch())
            ex.push()
            got, got_lse = ex.merge(out_dtype=torch.float32)
            torch.cuda.synchronize()
            assert _lib.device_status() == 0
            assert torch.equal(got, want) and torch.equal(got_lse, want_lse)
            # the same with the record delivered from inside the decode kernel
            ex.decode_push(q, k, v, kv_len=T, kv_begin=lo, kv_end=hi)
            got2, got2_lse = ex.merge(out_dtype=torch.float32)
            torch.cuda.synchronize()
            assert _lib.device_status() == 0
            # (that launch merges its chunks in the decode kernel: the same partials in another summation order)
            assert (got2 - want).abs().max().item() < 1e-5 and (got2_lse - want_lse).abs().max().item() < 1e-5
            # and with the whole tail in one kernel: chunk merge, row delivery, per-row wait, cross-rank merge
            got3, got3_lse = ex.decode_exchange(q, k, v, kv_len=T, kv_begin=lo, kv_end=hi, out_dtype=torch.float32)
            torch.cuda.synchronize()
            assert _lib.device_status() == 0
            assert (got3 - want).abs().max().item() < 1e-5 and (got3_lse - want_lse).abs().max().item() < 1e-5
            # and the same tail with the flag inside every 8-byte word (no fence, no flag store)
            got4, got4_lse = ex.decode_exchange(q, k, v, kv_len=T, kv_begin=lo, kv_end=hi, out_dtype=torch.float32, ll=True)
            torch.cuda.synchronize()
            assert _lib.device_status() == 0
            assert (got4 - want).abs().max().item() < 1e-5 and (got4_lse - want_lse).abs().max().item() < 1e-5
            assert (got - full.reshape(Hq, D)).abs().max().item() < 1e-3
            assert (got_lse - full_lse.reshape(Hq)).abs().max().item() < 1e-4
        dist.barrier()
        open(os.path.join(tmpdir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_split_kv_exchange_over_two_gpus(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(2))
