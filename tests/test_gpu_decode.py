"""GPU parity of the split-KV GQA decode and the (O, LSE) merge against the CPU oracle."""
import numpy as np
import pytest

from tests import util

pytestmark = pytest.mark.gpu


def _problem(orc, B, Hq, Hkv, D, max_seq, lens):
    q = util.normal_bf16(orc, (B, Hq, D), util.SEED_Q)
    k = util.normal_bf16(orc, (B, Hkv, max_seq, D), util.SEED_K)
    v = util.normal_bf16(orc, (B, Hkv, max_seq, D), util.SEED_V)
    return q, k, v, np.asarray(lens, dtype=np.int32)


def _run(q, k, v, lens, **kw):
    import torch
    import rustorch_b200 as rt
    out, lse = rt.gqa_decode(util.to_cuda_bf16(q), util.to_cuda_bf16(k), util.to_cuda_bf16(v),
                             kv_lens=util.to_cuda(lens), **kw)
    torch.cuda.synchronize()
    return util.to_np(out), util.to_np(lse)


@pytest.mark.parametrize("D,Hq,Hkv", [(128, 8, 2), (128, 4, 4), (128, 4, 2), (128, 16, 2), (64, 8, 2), (64, 8, 8),
                                       (64, 8, 4), (64, 8, 1), (256, 8, 2), (256, 2, 2)])
def test_decode_small_matches_oracle(oracle, D, Hq, Hkv):
    q, k, v, lens = _problem(oracle, 3, Hq, Hkv, D, 1024, [1, 63, 1000])
    out, lse = _run(q, k, v, lens)
    rc, ref, ref_lse = oracle.gqa_decode_cache(q, k, v, lens)
    assert rc == 0
    util.check_output(out, ref, label=f"decode D{D} Hq{Hq} Hkv{Hkv}")
    util.check_lse(lse, ref_lse)


def test_decode_ragged_lengths_and_f32_out(oracle):
    import torch
    B, Hq, Hkv, D, S = 8, 32, 8, 128, 2048
    lens = oracle.fill_uniform_int(B, util.SEED_LEN, 1, S)
    lens[0], lens[1], lens[2] = S, 1, 513
    q, k, v, lens = _problem(oracle, B, Hq, Hkv, D, S, lens)
    out, lse = _run(q, k, v, lens, out_dtype=torch.float32)
    _, ref, ref_lse = oracle.gqa_decode_cache(q, k, v, lens)
    util.check_output(out, ref, bf16_out=False, label="ragged f32")
    util.check_lse(lse, ref_lse)


def test_decode_empty_sequence_gives_zeros(oracle):
    q, k, v, lens = _problem(oracle, 2, 8, 2, 128, 1024, [0, 700])
    out, lse = _run(q, k, v, lens)
    assert np.all(out[0] == 0) and np.all(np.isneginf(lse[0]))
    _, ref, ref_lse = oracle.gqa_decode_cache(q, k, v, lens)
    util.check_output(out, ref)
    util.check_lse(lse, ref_lse)


def test_kv_range_partials_merge_to_full(oracle):
    """Split the KV range in 4 shards (as 4 GPUs would), merge the (O, LSE) partials, compare with
    the un-split result and the oracle.  One shard is empty for the short sequence (identity)."""
    import torch
    import rustorch_b200 as rt
    B, Hq, Hkv, D, S = 2, 32, 8, 128, 4096
    q, k, v, lens = _problem(oracle, B, Hq, Hkv, D, S, [4096, 1500])
    dq, dk, dv, dl = util.to_cuda_bf16(q), util.to_cuda_bf16(k), util.to_cuda_bf16(v), util.to_cuda(lens)
    parts_o, parts_l = [], []
    for r in range(4):
        o, l = rt.gqa_decode(dq, dk, dv, kv_lens=dl, kv_begin=r * 1024, kv_end=(r + 1) * 1024,
                             out_dtype=torch.float32)
        parts_o.append(o.reshape(B * Hq, D))
        parts_l.append(l.reshape(B * Hq))
    merged, mlse = rt.merge_partials(torch.stack(parts_o), torch.stack(parts_l), out_dtype=torch.float32)
    torch.cuda.synchronize()
    _, ref, ref_lse = oracle.gqa_decode_cache(q, k, v, lens)
    util.check_output(util.to_np(merged).reshape(B, Hq, D), ref, bf16_out=False, label="merged shards")
    util.check_lse(util.to_np(mlse).reshape(B, Hq), ref_lse)
    # the oracle's own partials + merge agree too (checks the merge algebra end to end)
    po = np.stack([oracle.gqa_decode_cache(q, k, v, lens, r * 1024, (r + 1) * 1024)[1].reshape(B * Hq, D)
                   for r in range(4)])
    pl = np.stack([oracle.gqa_decode_cache(q, k, v, lens, r * 1024, (r + 1) * 1024)[2].reshape(B * Hq)
                   for r in range(4)])
    mo, ml = oracle.merge_partials(po, pl)
    assert np.abs(mo.reshape(B, Hq, D) - ref).max() < 1e-5
    assert np.isneginf(pl[2:, Hq:]).all()  # shards 2,3 of the short sequence are empty


def test_reference_signature_gqa_decode_online_bf16(oracle):
    """LlmKernels::gqa_decode_online_bf16(stream,q,k,v,out,n_heads,n_kv,kv_len,head_dim,max_seq) drop-in."""
    import torch
    import rustorch_b200 as rt
    Hq, Hkv, D, S, L = 32, 8, 128, 2048, 1337
    q, k, v, _ = _problem(oracle, 1, Hq, Hkv, D, S, [L])
    dq, dk, dv = util.to_cuda_bf16(q[0]), util.to_cuda_bf16(k[0]), util.to_cuda_bf16(v[0])
    out = torch.empty((Hq, D), dtype=torch.bfloat16, device="cuda")
    kern = rt.LlmKernels()
    kern.gqa_decode_online_bf16(torch.cuda.current_stream(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                out.data_ptr(), Hq, Hkv, L, D, S)
    torch.cuda.synchronize()
    _, ref, _ = oracle.gqa_decode_cache(q, k, v, [L])
    util.check_output(util.to_np(out), ref[0], label="LlmKernels drop-in")
    # and through the reference's CPU-side API shape: gqa_forward_f32(batch=1, seq_q=1, seq_kv=L) on the trimmed cache
    rc, ref2 = oracle.gqa_forward_f32(q[0].ravel(), np.ascontiguousarray(k[0, :, :L]).ravel(),
                                      np.ascontiguousarray(v[0, :, :L]).ravel(), 1, Hq, Hkv, 1, L, D)
    assert rc == 0 and np.abs(ref2.reshape(Hq, D) - ref[0]).max() < 1e-6


def test_kv_append_then_decode(oracle):
    import torch
    import rustorch_b200 as rt
    B, Hq, Hkv, D, S = 2, 8, 2, 128, 256
    q, k, v, lens = _problem(oracle, B, Hq, Hkv, D, S, [10, 200])
    k_new = util.normal_bf16(oracle, (B, Hkv, D), 11)
    v_new = util.normal_bf16(oracle, (B, Hkv, D), 12)
    dk, dv = util.to_cuda_bf16(k), util.to_cuda_bf16(v)
    rt.kv_append(dk, dv, util.to_cuda_bf16(k_new), util.to_cuda_bf16(v_new), positions=util.to_cuda(lens))
    for b in range(B):
        k[b, :, lens[b]] = k_new[b]
        v[b, :, lens[b]] = v_new[b]
    torch.cuda.synchronize()
    assert np.array_equal(util.to_np(dk), k) and np.array_equal(util.to_np(dv), v)
    out, _ = rt.gqa_decode(util.to_cuda_bf16(q), dk, dv, kv_lens=util.to_cuda(lens + 1))
    _, ref, _ = oracle.gqa_decode_cache(q, k, v, lens + 1)
    util.check_output(util.to_np(out), ref)


def test_decode_validation_errors():
    import torch
    import rustorch_b200 as rt
    from rustorch_b200 import _lib
    q = torch.zeros((1, 5, 128), dtype=torch.bfloat16, device="cuda")
    kc = torch.zeros((1, 2, 64, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(rt.HeadCountMismatch):
        rt.gqa_decode(q, kc, kc, kv_len=3)
    q = torch.zeros((1, 4, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.CudaError) as e:
        rt.gqa_decode(q, kc, kc, kv_len=65)  # kv_len > max_seq
    assert e.value.code == _lib.RT_ERR_BAD_LENGTH
    big = torch.zeros((1, 2, 4096, 128), dtype=torch.bfloat16, device="cuda")
    tiny_ws = torch.empty(16, dtype=torch.uint8, device="cuda")
    with pytest.raises(_lib.CudaError) as e:
        rt.gqa_decode(q, big, big, kv_len=100, workspace=tiny_ws)
    assert e.value.code == _lib.RT_ERR_WORKSPACE
    q96 = torch.zeros((1, 4, 96), dtype=torch.bfloat16, device="cuda")
    k96 = torch.zeros((1, 2, 64, 96), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.Unsupported):
        rt.gqa_decode(q96, k96, k96, kv_len=3)


def test_decode_cfg4_shape_slice(oracle):
    """The batched-decode workload's geometry (Hq=32, Hkv=8, D=128, max_seq 8192, lens ~ U[1024,8192]) on 8 of its
    64 sequences, full check against the oracle; plus split-invariance at the full batch."""
    import torch
    import rustorch_b200 as rt
    B, Hq, Hkv, D, S = 8, 32, 8, 128, 8192
    lens = oracle.fill_uniform_int(B, util.SEED_LEN, 1024, 8192)
    q, k, v, lens = _problem(oracle, B, Hq, Hkv, D, S, lens)
    out, lse = _run(q, k, v, lens)
    _, ref, ref_lse = oracle.gqa_decode_cache(q, k, v, lens)
    util.check_output(out, ref, label="cfg4 slice")
    util.check_lse(lse, ref_lse)


def test_decode_cfg4_full_size_split_invariance():
    """The full batched-decode workload (B=64): the result must not depend on how the KV range is sharded."""
    import torch
    import rustorch_b200 as rt
    B, Hq, Hkv, D, S = 64, 32, 8, 128, 8192
    g = torch.Generator(device="cuda").manual_seed(4)
    q = torch.randn((B, Hq, D), device="cuda", generator=g).to(torch.bfloat16)
    kc = torch.randn((B, Hkv, S, D), device="cuda", generator=g).to(torch.bfloat16)
    vc = torch.randn((B, Hkv, S, D), device="cuda", generator=g).to(torch.bfloat16)
    lens = torch.randint(1024, 8193, (B,), device="cuda", generator=g, dtype=torch.int32)
    full, lse = rt.gqa_decode(q, kc, vc, kv_lens=lens, out_dtype=torch.float32)
    po, pl = [], []
    for lo, hi in ((0, 3000), (3000, 3001), (3001, 8192)):
        o, l = rt.gqa_decode(q, kc, vc, kv_lens=lens, kv_begin=lo, kv_end=hi, out_dtype=torch.float32)
        po.append(o.reshape(B * Hq, D))
        pl.append(l.reshape(B * Hq))
    merged, mlse = rt.merge_partials(torch.stack(po), torch.stack(pl), out_dtype=torch.float32)
    torch.cuda.synchronize()
    # P is rounded to bf16 relative to a running maximum that depends on the chunking, so two shardings
    # agree to ~2^-9 / sqrt(len) per element, not bit for bit; the row sums (LSE) stay in f32.
    assert (merged.reshape(B, Hq, D) - full).abs().max().item() < 1e-3
    assert (mlse.reshape(B, Hq) - lse).abs().max().item() < 1e-4
    # independent check on a few rows with plain torch math in f32
    for b in (0, 17, 63):
        L = int(lens[b])
        kk = kc[b, :, :L].float().repeat_interleave(4, dim=0)
        vv = vc[b, :, :L].float().repeat_interleave(4, dim=0)
        s = torch.einsum("hd,hld->hl", q[b].float(), kk) / (D ** 0.5)
        ref = torch.einsum("hl,hld->hd", torch.softmax(s, dim=-1), vv)
        assert (ref - full[b]).abs().max().item() < 2e-3


def test_packed_records_equal_separate_partials(oracle):
    """rt_gqa_decode_record_bf16 + rt_attn_merge_records (the split-KV exchange format, one [rows, D+1]
    record per shard) against the separate (O, LSE) outputs and against the oracle."""
    import torch
    import rustorch_b200 as rt
    B, Hq, Hkv, D, S = 2, 32, 8, 128, 4096
    q, k, v, lens = _problem(oracle, B, Hq, Hkv, D, S, [4096, 900])
    dq, dk, dv, dl = util.to_cuda_bf16(q), util.to_cuda_bf16(k), util.to_cuda_bf16(v), util.to_cuda(lens)
    recs = []
    for r in range(4):
        rec = rt.gqa_decode_record(dq, dk, dv, kv_lens=dl, kv_begin=r * 1024, kv_end=(r + 1) * 1024)
        o, l = rt.gqa_decode(dq, dk, dv, kv_lens=dl, kv_begin=r * 1024, kv_end=(r + 1) * 1024,
                             out_dtype=torch.float32)
        assert rec.shape == (B * Hq, D + 1)
        assert torch.equal(rec[:, :D], o.reshape(B * Hq, D)) and torch.equal(rec[:, D], l.reshape(B * Hq))
        recs.append(rec)
    allrec = torch.stack(recs)
    merged, mlse = rt.merge_records(allrec, out_dtype=torch.float32)
    m2, l2 = rt.merge_partials(allrec[:, :, :D].contiguous(), allrec[:, :, D].contiguous(), out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert torch.equal(merged, m2) and torch.equal(mlse, l2)
    _, ref, ref_lse = oracle.gqa_decode_cache(q, k, v, lens)
    util.check_output(util.to_np(merged).reshape(B, Hq, D), ref, bf16_out=False, label="records")
    util.check_lse(util.to_np(mlse).reshape(B, Hq), ref_lse)
    # a single-chunk launch (short cache) writes the record directly from the decode kernel
    q1, k1, v1, l1 = _problem(oracle, 1, 8, 2, 64, 128, [100])
    rec = rt.gqa_decode_record(util.to_cuda_bf16(q1), util.to_cuda_bf16(k1), util.to_cuda_bf16(v1),
                               kv_lens=util.to_cuda(l1))
    _, r1, rl1 = oracle.gqa_decode_cache(q1, k1, v1, l1)
    util.check_output(util.to_np(rec[:, :64]).reshape(1, 8, 64), r1, bf16_out=False)
    util.check_lse(util.to_np(rec[:, 64]).reshape(1, 8), rl1)


@pytest.mark.parametrize("style,code", [("half_split", 0), ("adjacent", 1)])
def test_rope_kv_append_then_decode(oracle, style, code):
    """The fused step before the decode: rotate q and the new K row, append K and V at each sequence's position."""
    import torch
    import rustorch_b200 as rt
    B, Hq, Hkv, D, S = 3, 8, 2, 128, 512
    q, kc, vc, lens = _problem(oracle, B, Hq, Hkv, D, S, [17, 300, 511])
    k_new = util.normal_bf16(oracle, (B, Hkv, D), 21)
    v_new = util.normal_bf16(oracle, (B, Hkv, D), 22)
    dq, dk, dv = util.to_cuda_bf16(q), util.to_cuda_bf16(kc), util.to_cuda_bf16(vc)
    inv_freq = rt.rope_inv_freq(D, 10000.0)
    rt.rope_kv_append(dq, util.to_cuda_bf16(k_new), util.to_cuda_bf16(v_new), dk, dv, inv_freq,
                      positions=util.to_cuda(lens), style=style)
    torch.cuda.synchronize()
    q_ref = oracle.rope_token(q, lens, 10000.0, code)
    k_ref = oracle.rope_token(k_new, lens, 10000.0, code)
    # bf16 storage: equal to the rounded oracle value up to one bf16 ulp (sincosf vs libm in the last bit)
    assert np.abs(util.to_np(dq) - q_ref).max() <= 2.0 ** -7 * np.abs(q_ref).max()
    got_k, got_v = util.to_np(dk), util.to_np(dv)
    for b in range(B):
        assert np.abs(got_k[b, :, lens[b]] - k_ref[b]).max() <= 2.0 ** -7 * np.abs(k_ref).max()
        assert np.array_equal(got_v[b, :, lens[b]], v_new[b])
        kc[b, :, lens[b]] = got_k[b, :, lens[b]]
        vc[b, :, lens[b]] = v_new[b]
    assert np.array_equal(got_k, kc) and np.array_equal(got_v, vc)  # nothing else in the caches moved
    # rotation preserves the norm of every pair, hence of the row
    assert np.allclose(np.linalg.norm(util.to_np(dq), axis=-1), np.linalg.norm(q, axis=-1), rtol=1e-2)
    out, _ = rt.gqa_decode(dq, dk, dv, kv_lens=util.to_cuda(lens + 1))
    _, ref, _ = oracle.gqa_decode_cache(util.to_np(dq), kc, vc, lens + 1)
    util.check_output(util.to_np(out), ref, label="rope + append + decode")


def test_peer_exchange_push_and_merge_on_one_device(oracle):
    """The split-KV exchange over peer stores (rt_splitkv_push_record + rt_attn_merge_records_after), with the
    "peers" being buffers of one device: every emulated rank decodes its KV shard into its own slot, pushes it
    to all ranks, and every rank's merge equals the merge of the gathered records, twice in a row (the two
    slot sets alternate)."""
    import torch
    import rustorch_b200 as rt
    from rustorch_b200 import _lib, sharding
    B, Hq, Hkv, D, S, world = 1, 32, 8, 128, 3000, 3
    q, k, v, lens = _problem(oracle, B, Hq, Hkv, D, S, [2900])
    dk, dv, dl = util.to_cuda_bf16(k), util.to_cuda_bf16(v), util.to_cuda(lens)
    ranks = sharding.PeerRecordExchange.local_pair(world, B * Hq, D)
    for step in range(2):
        qs = util.normal_bf16(oracle, (B, Hq, D), 77 + step)
        dq = util.to_cuda_bf16(qs)
        recs = []
        for r, ex in enumerate(ranks):
            b0, b1 = sharding.kv_shard(2900, world, r, align=16)
            recs.append(rt.gqa_decode_record(dq, dk, dv, kv_lens=dl, kv_begin=b0, kv_end=b1, record=ex.next_epoch()))
        for ex in ranks:
            ex.push()
        want, want_lse = rt.merge_records(torch.stack([r.clone() for r in recs]), out_dtype=torch.float32)
        for ex in ranks:
            got, got_lse = ex.merge(out_dtype=torch.float32)
            assert torch.equal(got, want) and torch.equal(got_lse, want_lse)
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
        _, ref, ref_lse = oracle.gqa_decode_cache(qs, k, v, lens)
        util.check_output(util.to_np(want).reshape(B, Hq, D), ref, bf16_out=False, label=f"exchange step {step}")
        util.check_lse(util.to_np(want_lse).reshape(B, Hq), ref_lse)


def test_peer_exchange_wait_runs_out_and_reports(oracle):
    """A record that never arrives: the merge's bounded wait (here ~10 ms) expires, the kernel leaves the outputs
    alone, the status word reports code 401, and the context stays usable."""
    import torch
    import rustorch_b200 as rt
    from rustorch_b200 import _lib, sharding
    ranks = sharding.PeerRecordExchange.local_pair(2, 32, 128)
    ranks[0].next_epoch().fill_(1.0)
    ranks[0].push()              # rank 1 never pushes: flag 1 on rank 0 stays 0
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    out, lse = ranks[0].merge(out_dtype=torch.float32, wait_clocks=20_000_000)
    torch.cuda.synchronize()
    assert _lib.device_status() == 401
    assert _lib.device_status() == 0  # reading clears it
    # the device still works
    o, l = rt.merge_records(torch.ones((2, 32, 129), dtype=torch.float32, device="cuda"), out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert torch.allclose(o, torch.ones_like(o))


@pytest.mark.parametrize("kv_total,S", [(2900, 3000), (40000, 40960), (100, 128)])
def test_peer_exchange_fused_decode_push_on_one_device(oracle, kv_total, S):
    """rt_gqa_decode_record_push_bf16: the merge kernel of each emulated rank delivers its record to all ranks
    itself (many chunks), or the copy kernel does (a single chunk); either way every rank's merge equals the merge
    of the gathered records."""
    import torch
    import rustorch_b200 as rt
    from rustorch_b200 import _lib, sharding
    B, Hq, Hkv, D, world = 1, 32, 8, 128, 3
    g = torch.Generator(device="cuda").manual_seed(11)
    k = torch.randn((B, Hkv, S, D), device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn((B, Hkv, S, D), device="cuda", generator=g).to(torch.bfloat16)
    ranks = sharding.PeerRecordExchange.local_pair(world, B * Hq, D)
    for step in range(3):
        q = torch.randn((B, Hq, D), device="cuda", generator=g).to(torch.bfloat16)
        recs = []
        for r, ex in enumerate(ranks):
            b0, b1 = sharding.kv_shard(kv_total, world, r, align=16)
            plain = rt.gqa_decode_record(q, k, v, kv_len=kv_total, kv_begin=b0, kv_end=b1)
            got = ex.decode_push(q, k, v, kv_len=kv_total, kv_begin=b0, kv_end=b1)
            # the pushing launch merges its chunks inside the decode kernel, the plain one in the merge kernel:
            # the same partials summed in another order
            assert (got - plain).abs().max().item() < 1e-5
            recs.append(got.clone())
        want, want_lse = rt.merge_records(torch.stack(recs), out_dtype=torch.float32)
        for ex in ranks:
            out, lse = ex.merge(out_dtype=torch.float32)
            assert torch.equal(out, want) and torch.equal(lse, want_lse)
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
        assert all(int(ex._done.item()) == 0 for ex in ranks)
    full, full_lse = rt.gqa_decode(q, k, v, kv_len=kv_total, out_dtype=torch.float32)
    assert (want - full.reshape(B * Hq, D)).abs().max().item() < 1e-3


def test_decode_long_context_shard_at_full_size(oracle):
    """One GPU's share of the long-context split-KV workload at its real size: B=1, Hq=32, Hkv=8, D=128,
    131072 cached positions (0.5 GiB of K and V on the device, 147 chunks into the chunk-merge kernel),
    against the oracle's decode_attn_row restatement, through rt_gqa_decode_record_bf16 +
    rt_attn_merge_records; then the same range cut into 8 shards by 8 emulated ranks on this device
    (peer exchange with the peers being local buffers), every rank's merge against the oracle."""
    import torch
    import rustorch_b200 as rt
    from rustorch_b200 import _lib, sharding
    B, Hq, Hkv, D, T = 1, 32, 8, 128, 131072
    q, k, v, lens = _problem(oracle, B, Hq, Hkv, D, T, [T])
    rc, ref, ref_lse = oracle.gqa_decode_cache(q, k, v, lens)
    assert rc == 0
    dq, dk, dv = util.to_cuda_bf16(q), util.to_cuda_bf16(k), util.to_cuda_bf16(v)

    rec = rt.gqa_decode_record(dq, dk, dv, kv_len=T)
    out, lse = rt.merge_records(rec.unsqueeze(0), out_dtype=torch.float32)
    out16, _ = rt.gqa_decode(dq, dk, dv, kv_len=T)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    util.check_output(util.to_np(out).reshape(B, Hq, D), ref, bf16_out=False, label="131072-position shard, f32 record")
    util.check_lse(util.to_np(lse).reshape(B, Hq), ref_lse)
    util.check_output(util.to_np(out16), ref, label="131072-position shard, bf16 out")

    world = 8
    ranks = sharding.PeerRecordExchange.local_pair(world, B * Hq, D)
    for r, ex in enumerate(ranks):
        b0, b1 = sharding.kv_shard(T, world, r, align=16)
        rt.gqa_decode_record(dq, dk, dv, kv_len=T, kv_begin=b0, kv_end=b1, record=ex.next_epoch())
    for ex in ranks:
        ex.push()
    for ex in ranks:
        got, got_lse = ex.merge(out_dtype=torch.float32)
        torch.cuda.synchronize()
        util.check_output(util.to_np(got).reshape(B, Hq, D), ref, bf16_out=False, label="8 emulated shards")
        util.check_lse(util.to_np(got_lse).reshape(B, Hq), ref_lse)
    assert _lib.device_status() == 0


@pytest.mark.parametrize("ll", [False, True])
@pytest.mark.parametrize("kv_total,S", [(2900, 3000), (40000, 40960), (100, 128)])
def test_row_exchange_on_one_device(oracle, kv_total, S, ll):
    """rt_gqa_decode_exchange_bf16 with the ranks emulated on one device: every rank's exchange kernel merges its
    chunk partials row by row and delivers the rows (wait = 0), then rt_attn_merge_records_after_rows waits per
    row and merges.  Every rank must end with the merge of the ranks' records (many chunks, few chunks, and a
    single chunk whose record comes straight from the decode kernel), three epochs so both slot sets are used
    and one is used again.  ll: the same through rt_gqa_decode_exchange_ll_bf16 / rt_attn_merge_ll_rows, where
    every element travels as an 8-byte {value, epoch} word and the reader spins on the words."""
    import torch
    import rustorch_b200 as rt
    from rustorch_b200 import _lib, sharding
    B, Hq, Hkv, D, world = 1, 32, 8, 128, 3
    g = torch.Generator(device="cuda").manual_seed(12)
    k = torch.randn((B, Hkv, S, D), device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn((B, Hkv, S, D), device="cuda", generator=g).to(torch.bfloat16)
    ranks = sharding.PeerRecordExchange.local_pair(world, B * Hq, D)
    for step in range(3):
        q = torch.randn((B, Hq, D), device="cuda", generator=g).to(torch.bfloat16)
        recs = []
        for r, ex in enumerate(ranks):
            b0, b1 = sharding.kv_shard(kv_total, world, r, align=16)
            recs.append(rt.gqa_decode_record(q, k, v, kv_len=kv_total, kv_begin=b0, kv_end=b1))
            ex.decode_exchange(q, k, v, kv_len=kv_total, kv_begin=b0, kv_end=b1, wait=False, ll=ll)
        want, want_lse = rt.merge_records(torch.stack(recs), out_dtype=torch.float32)
        for ex in ranks:
            out, lse = ex.merge_rows(out_dtype=torch.float32, ll=ll)
            assert (out - want).abs().max().item() < 1e-5 and (lse - want_lse).abs().max().item() < 1e-5
            par = ex.epoch & 1
            if ll:  # every word carries the epoch in its upper half and the record's bits in the lower
                words = ex.ll_words[par]
                assert bool(((words >> 32) == ex.epoch).all())
                vals = (words & 0xFFFFFFFF).to(torch.int32).view(torch.float32)
                assert (vals - torch.stack(recs)).abs().max().item() < 1e-5
            else:   # the slots hold exactly the records the ranks produced
                assert (ex.records[par] - torch.stack(recs)).abs().max().item() < 1e-5
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
    full, full_lse = rt.gqa_decode(q, k, v, kv_len=kv_total, out_dtype=torch.float32)
    assert (want - full.reshape(B * Hq, D)).abs().max().item() < 1e-3
    if kv_total == 2900:  # and against the oracle
        _, ref, ref_lse = oracle.gqa_decode_cache(util.to_np(q), util.to_np(k), util.to_np(v), np.array([kv_total], dtype=np.int32))
        util.check_output(util.to_np(want).reshape(B, Hq, D), ref, bf16_out=False, label="row exchange")
        util.check_lse(util.to_np(want_lse).reshape(B, Hq), ref_lse)


@pytest.mark.parametrize("ll", [False, True])
def test_row_exchange_wait_runs_out_and_reports(ll):
    """A row that never arrives: the per-row wait (here ~10 ms) expires, nothing is written, status 401."""
    import torch
    from rustorch_b200 import _lib, sharding
    ranks = sharding.PeerRecordExchange.local_pair(2, 32, 128)
    for ex in ranks:
        ex.epoch = 1  # nobody delivered anything for epoch 1
    out, lse = ranks[0].merge_rows(out_dtype=torch.float32, wait_clocks=20_000_000, ll=ll)
    torch.cuda.synchronize()
    assert _lib.device_status() == 401
    assert _lib.device_status() == 0
