"""World-size-2 (gloo, CPU) test of the multi-GPU host logic: KV-range sharding, record packing, the
all-gather and the merge order.  The per-shard partials and the merge come from the oracle here (the
CUDA kernels need a GPU); on GPUs the same plumbing carries the kernels' partials."""
import os
import socket

import numpy as np
import pytest


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, kv_len, tmpdir):
    import torch
    import torch.distributed as dist
    from oracle import oracle as orc
    from rustorch_b200 import sharding

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, Hq, Hkv, D, S = 1, 8, 2, 32, 256
        q = orc.fill_normal((B, Hq, D), 1)          # every rank holds the full q
        kc = orc.fill_normal((B, Hkv, S, D), 2)
        vc = orc.fill_normal((B, Hkv, S, D), 3)
        lens = np.array([kv_len], dtype=np.int32)
        lo, hi = sharding.kv_shard(kv_len, world, rank, align=16)
        _, o, lse = orc.gqa_decode_cache(q, kc, vc, lens, lo, hi)
        rec = sharding.pack_partial(torch.from_numpy(o.reshape(Hq, D)), torch.from_numpy(lse.reshape(Hq)))
        allrec = sharding.all_gather_partials(rec)
        assert allrec.shape == (world, Hq, D + 1)
        po, pl = sharding.unpack_partials(allrec)
        merged, mlse = orc.merge_partials(po.numpy(), pl.numpy())
        _, full, full_lse = orc.gqa_decode_cache(q, kc, vc, lens)
        assert np.abs(merged - full[0]).max() < 1e-5 and np.abs(mlse - full_lse[0]).max() < 1e-5
        # every rank ends with the same merged result
        t = torch.from_numpy(merged.copy())
        ref = t.clone()
        dist.broadcast(ref, src=0)
        assert torch.equal(ref, t)
        open(os.path.join(tmpdir, f"ok{rank}"), "w").write(f"{lo},{hi}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("kv_len", [200, 16])  # 16: rank 1 holds an empty shard (identity partial)
def test_split_kv_over_two_gloo_ranks(tmp_path, kv_len):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_worker, args=(2, port, kv_len, str(tmp_path)), nprocs=2, join=True)
    ranges = [tuple(map(int, open(tmp_path / f"ok{r}").read().split(","))) for r in range(2)]
    assert ranges[0][0] == 0 and ranges[0][1] == ranges[1][0] and ranges[1][1] == kv_len


def test_shard_units_cover_exactly_once():
    from rustorch_b200 import sharding
    for n in (0, 1, 7, 128, 129):
        for world in (1, 2, 3, 8):
            spans = [sharding.shard_units(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_units(4, 2, 2)


def test_kv_shard_alignment_and_config5_sizes():
    from rustorch_b200 import sharding
    spans = [sharding.kv_shard(1_048_576, 8, r, align=16) for r in range(8)]
    assert all(e - b == 131_072 for b, e in spans)  # the long-context workload: 131072 positions per GPU
    spans = [sharding.kv_shard(1000, 3, r, align=64) for r in range(3)]
    assert spans[0][0] == 0 and spans[-1][1] == 1000 and all(b % 64 == 0 for b, _ in spans)


def test_balance_sequences_lpt():
    from rustorch_b200 import sharding
    rng = np.random.default_rng(0)
    lens = rng.integers(1024, 8193, 64)
    parts = sharding.balance_sequences(lens.tolist(), 8)
    assert sorted(i for p in parts for i in p) == list(range(64))
    loads = [int(lens[p].sum()) for p in parts]
    assert max(loads) <= 1.05 * (lens.sum() / 8)  # decode work (sum of lengths) balanced within 5 %
    assert sharding.balance_sequences([5.0], 4) == [[0], [], [], []]
