"""Host-side partitioning of the attention path across the GPUs of one box.

The reference has no multi-device attention (its NCCL layer is a single-rank stub,
crates/rustorch-cuda/src/nccl.rs:116-143).  The path shards in two ways:

* prefill and batched decode: (batch, head) units / sequences are independent — the unit the
  reference's rayon loop parallelises over (crates/rustorch-attention/src/cpu_forward.rs:219-226).
  Each rank takes a contiguous slab (`shard_units`) or a length-balanced set of sequences
  (`balance_sequences`); no collective is needed.
* long-context decode: the KV range is split contiguously (`kv_shard`); every rank produces a
  normalised partial (O f32 [rows, D], LSE [rows]), the ranks exchange one packed record each
  (`pack_partial` + `all_gather_partials`) and merge locally with the combine_tiles algebra
  (crates/rustorch-attention/src/online_softmax.rs:105-131).

Everything here is plain torch / torch.distributed plumbing and runs on CPU (gloo) as well as on
GPUs (nccl); the arithmetic lives in the CUDA library.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple


def shard_units(n_units: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced [begin, end) slice of `n_units` independent units for `rank`."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} for world size {world}")
    base, extra = divmod(max(n_units, 0), world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def kv_shard(kv_len: int, world: int, rank: int, align: int = 1) -> Tuple[int, int]:
    """Contiguous KV range [begin, end) of `rank`; shard boundaries are multiples of `align`."""
    blocks = (max(kv_len, 0) + align - 1) // align
    b0, b1 = shard_units(blocks, world, rank)
    return min(b0 * align, kv_len), min(b1 * align, kv_len)


def balance_sequences(costs: Sequence[float], world: int) -> List[List[int]]:
    """Longest-processing-time assignment of sequences to ranks; returns the indices of each rank.

    `costs[i]` is the work of sequence i (sum of lengths for decode, length squared for causal
    prefill).  Greedy LPT keeps the heaviest rank within 4/3 of the optimum.
    """
    loads = [0.0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for i in sorted(range(len(costs)), key=lambda j: (-costs[j], j)):
        r = min(range(world), key=lambda x: (loads[x], x))
        out[r].append(i)
        loads[r] += float(costs[i])
    return [sorted(ix) for ix in out]


def pack_partial(o, lse):
    """(O [rows, D] f32, LSE [rows] f32) -> one contiguous record [rows, D + 1]."""
    import torch
    return torch.cat([o, lse.unsqueeze(-1)], dim=-1).contiguous()


def unpack_partials(records):
    """[R, rows, D + 1] -> (O [R, rows, D], LSE [R, rows]), both contiguous."""
    return records[..., :-1].contiguous(), records[..., -1].contiguous()


def all_gather_partials(record, group=None):
    """All-gather one packed record per rank -> [world, rows, D + 1] (rank order = KV order)."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    out = torch.empty((world,) + tuple(record.shape), dtype=record.dtype, device=record.device)
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(out, record.contiguous(), group=group)
    else:  # gloo has no flat-tensor all-gather
        dist.all_gather(list(out.unbind(0)), record.contiguous(), group=group)
    return out


class PeerRecordExchange:
    """Split-KV exchange over peer memory instead of an NCCL all-gather.

    Every rank holds two sets of `world` record slots ([rows, D+1] f32 each) and `world` flags that
    its peers can write.  One exchange = `rt_splitkv_push_record` (this rank's record goes to its
    slot on every peer with plain NVLink stores, then the peer's flag is set to the epoch) followed
    by `rt_attn_merge_records_after` (bounded wait for all flags, then the usual merge).  The two
    slot sets alternate, so a fast rank cannot overwrite what a slow peer still merges.

    `slots[r]` / `flags[r]` are (tensor, peer base pointers) pairs: with `torch.distributed`
    they come from symmetric memory (`create`); `local_pair` builds the same structure from ordinary
    tensors of ONE device so that the kernels can be exercised without a second GPU.
    """

    def __init__(self, rank: int, world: int, rows: int, dim: int, records, flags, record_ptrs, flag_ptrs):
        self.rank, self.world, self.rows, self.dim = rank, world, rows, dim
        self.records = records          # local f32 [2, world, rows, dim + 1]
        self.flags = flags              # local int32 [2, world]
        self.record_ptrs = list(record_ptrs)  # base address of every rank's `records`
        self.flag_ptrs = list(flag_ptrs)      # base address of every rank's `flags`
        self.epoch = 0
        self._done = None  # device int32, zero between calls (used by decode_push)
        self.row_flags = None      # local int32 [2, world, rows]: one flag per (rank, row), for decode_exchange
        self.row_flag_ptrs = None  # base address of every rank's `row_flags'
        self.ll_words = None       # local int64 [2, world, rows, dim + 1]: {f32 bits, epoch} words, for decode_exchange(ll=True)
        self.ll_word_ptrs = None   # base address of every rank's `ll_words`
        if (rows * (dim + 1)) % 4:
            raise ValueError("rows * (dim + 1) must be a multiple of 4 (16-byte copies)")

    @classmethod
    def create(cls, rows: int, dim: int, group=None, device=None):
        """Collective: allocates the slots in symmetric memory and exchanges the peer mappings."""
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        group = group if group is not None else dist.group.WORLD
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        records = symm.empty((2, world, rows, dim + 1), dtype=torch.float32, device=device)
        flags = symm.empty((2, world), dtype=torch.int32, device=device)
        flags.zero_()
        h_rec = symm.rendezvous(records, group.group_name)
        h_flag = symm.rendezvous(flags, group.group_name)
        torch.cuda.synchronize()
        dist.barrier(group)  # every rank's flags are zero before anyone pushes
        row_flags = symm.empty((2, world, rows), dtype=torch.int32, device=device)
        row_flags.zero_()
        h_rows = symm.rendezvous(row_flags, group.group_name)
        torch.cuda.synchronize()
        dist.barrier(group)
        ll_words = symm.empty((2, world, rows, dim + 1), dtype=torch.int64, device=device)
        ll_words.zero_()
        h_ll = symm.rendezvous(ll_words, group.group_name)
        torch.cuda.synchronize()
        dist.barrier(group)
        ex = cls(rank, world, rows, dim, records, flags, h_rec.buffer_ptrs, h_flag.buffer_ptrs)
        ex.row_flags, ex.row_flag_ptrs = row_flags, list(h_rows.buffer_ptrs)
        ex.ll_words, ex.ll_word_ptrs = ll_words, list(h_ll.buffer_ptrs)
        ex._handles = (h_rec, h_flag, h_rows, h_ll)  # keep the mappings alive
        return ex

    @classmethod
    def local_pair(cls, world: int, rows: int, dim: int, device="cuda"):
        """`world` exchange objects whose "peers" are buffers of one device (tests, single GPU)."""
        import torch
        recs = [torch.zeros((2, world, rows, dim + 1), dtype=torch.float32, device=device) for _ in range(world)]
        flgs = [torch.zeros((2, world), dtype=torch.int32, device=device) for _ in range(world)]
        rowf = [torch.zeros((2, world, rows), dtype=torch.int32, device=device) for _ in range(world)]
        out = [cls(r, world, rows, dim, recs[r], flgs[r], [t.data_ptr() for t in recs], [t.data_ptr() for t in flgs])
               for r in range(world)]
        llw = [torch.zeros((2, world, rows, dim + 1), dtype=torch.int64, device=device) for _ in range(world)]
        for r, ex in enumerate(out):
            ex.row_flags, ex.row_flag_ptrs = rowf[r], [t.data_ptr() for t in rowf]
            ex.ll_words, ex.ll_word_ptrs = llw[r], [t.data_ptr() for t in llw]
        return out

    def next_epoch(self):
        """Advances the epoch; returns the slot (a [rows, D+1] view of local memory) that this rank's
        decode kernel should write its record into for this exchange."""
        self.epoch += 1
        return self.records[self.epoch & 1, self.rank]

    def _peer_ptrs(self):
        import ctypes
        par = self.epoch & 1
        rec_bytes = self.rows * (self.dim + 1) * 4
        slot_off = (par * self.world + self.rank) * rec_bytes
        flag_off = (par * self.world + self.rank) * 4
        slots = (ctypes.c_void_p * self.world)(*[p + slot_off for p in self.record_ptrs])
        flags = (ctypes.c_void_p * self.world)(*[p + flag_off for p in self.flag_ptrs])
        return slots, flags

    def decode_push(self, q, k_cache, v_cache, kv_lens=None, kv_len=None, kv_begin: int = 0, kv_end: int = -1,
                    scale=None, workspace=None):
        """Advances the epoch, decodes this rank's KV shard into its slot and delivers the record to every peer
        from inside the merge kernel (``rt_gqa_decode_record_push_bf16``).  Follow with ``merge()``."""
        import torch
        from . import _lib
        from .gqa import _guard_decode_args, _stream_ptr, decode_workspace_bytes
        B, Hq, Hkv, D, max_seq = _guard_decode_args(q, k_cache, v_cache, kv_lens, workspace)
        if self._done is None:
            self._done = torch.zeros(1, dtype=torch.int32, device=self.records.device)
        need = decode_workspace_bytes(B, Hq, Hkv, D, max_seq)
        if workspace is None and need:
            workspace = getattr(self, "_ws", None)
            if workspace is None or workspace.numel() < need:
                workspace = self._ws = torch.empty(need, dtype=torch.uint8, device=q.device)
        record = self.next_epoch()
        slots, flags = self._peer_ptrs()
        rc = _lib.lib().rt_gqa_decode_record_push_bf16(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), record.data_ptr(), slots, flags, self.world,
            self.epoch, self._done.data_ptr(), B, Hq, Hkv, D, max_seq,
            kv_lens.data_ptr() if kv_lens is not None else None, 0 if kv_len is None else int(kv_len), kv_begin, kv_end,
            -1.0 if scale is None else float(scale), workspace.data_ptr() if workspace is not None else None,
            workspace.numel() if workspace is not None else 0, _stream_ptr())
        _lib.check(rc, "rt_gqa_decode_record_push_bf16")
        return record

    def decode_exchange(self, q, k_cache, v_cache, kv_lens=None, kv_len=None, kv_begin: int = 0, kv_end: int = -1,
                        scale=None, workspace=None, out_dtype=None, wait: bool = True, wait_clocks: int = 0,
                        ll: bool = False):
        """One exchange in two launches (``rt_gqa_decode_exchange_bf16``): the decode kernel over this rank's KV
        shard, then ONE kernel that merges its chunk partials row by row, delivers each row to every rank, waits
        for the same row from every rank and merges them.  Returns (out [rows, D], lse [rows]).  With
        ``wait=False`` the second kernel stops after the delivery and ``merge_rows()`` finishes the step (for
        several ranks emulated on one GPU, where no kernel may wait for a later launch of the same GPU).
        ``ll=True`` sends every element as an 8-byte {value, epoch} word (``rt_gqa_decode_exchange_ll_bf16``): no
        fence and no flag store between data and flag, the reader spins on the words; ``merge_rows(ll=True)``
        is its second half."""
        import ctypes
        import torch
        from . import _lib
        from .gqa import _guard_decode_args, _stream_ptr, decode_workspace_bytes
        B, Hq, Hkv, D, max_seq = _guard_decode_args(q, k_cache, v_cache, kv_lens, workspace)
        need = decode_workspace_bytes(B, Hq, Hkv, D, max_seq)
        if workspace is None and need:
            workspace = getattr(self, "_ws", None)
            if workspace is None or workspace.numel() < need:
                workspace = self._ws = torch.empty(need, dtype=torch.uint8, device=q.device)
        self.epoch += 1
        par = self.epoch & 1
        rec_bytes = self.rows * (self.dim + 1) * 4
        slot_off = (par * self.world + self.rank) * rec_bytes
        flag_off = (par * self.world + self.rank) * self.rows * 4
        slots = (ctypes.c_void_p * self.world)(*[p + slot_off for p in self.record_ptrs])
        flags = (ctypes.c_void_p * self.world)(*[p + flag_off for p in self.row_flag_ptrs])
        out_dtype = out_dtype or torch.bfloat16
        out = torch.empty((self.rows, self.dim), dtype=out_dtype, device=q.device)
        lse = torch.empty((self.rows,), dtype=torch.float32, device=q.device)
        if ll:
            word_off = (par * self.world + self.rank) * self.rows * (self.dim + 1) * 8
            words = (ctypes.c_void_p * self.world)(*[p + word_off for p in self.ll_word_ptrs])
            rc = _lib.lib().rt_gqa_decode_exchange_ll_bf16(
                q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                out.data_ptr() if out_dtype == torch.bfloat16 else None,
                out.data_ptr() if out_dtype == torch.float32 else None, lse.data_ptr(), words,
                self.ll_words[par].data_ptr(), self.records[par, self.rank].data_ptr(), self.world, self.rank, self.epoch,
                wait_clocks, 1 if wait else 0, B, Hq, Hkv, D, max_seq,
                kv_lens.data_ptr() if kv_lens is not None else None, 0 if kv_len is None else int(kv_len), kv_begin,
                kv_end, -1.0 if scale is None else float(scale), workspace.data_ptr() if workspace is not None else None,
                workspace.numel() if workspace is not None else 0, _stream_ptr())
            _lib.check(rc, "rt_gqa_decode_exchange_ll_bf16")
            return out, lse
        rc = _lib.lib().rt_gqa_decode_exchange_bf16(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
            out.data_ptr() if out_dtype == torch.bfloat16 else None, out.data_ptr() if out_dtype == torch.float32 else None,
            lse.data_ptr(), slots, flags, self.records[par].data_ptr(), self.row_flags[par].data_ptr(), self.world,
            self.rank, self.epoch, wait_clocks, 1 if wait else 0, B, Hq, Hkv, D, max_seq,
            kv_lens.data_ptr() if kv_lens is not None else None, 0 if kv_len is None else int(kv_len), kv_begin, kv_end,
            -1.0 if scale is None else float(scale), workspace.data_ptr() if workspace is not None else None,
            workspace.numel() if workspace is not None else 0, _stream_ptr())
        _lib.check(rc, "rt_gqa_decode_exchange_bf16")
        return out, lse

    def merge_rows(self, out_dtype=None, wait_clocks: int = 0, ll: bool = False):
        """Second half of ``decode_exchange(wait=False)``: waits per row for every rank's row, then merges."""
        import torch
        from . import _lib
        from .gqa import _stream_ptr
        par = self.epoch & 1
        out_dtype = out_dtype or torch.bfloat16
        out = torch.empty((self.rows, self.dim), dtype=out_dtype, device=self.records.device)
        lse = torch.empty((self.rows,), dtype=torch.float32, device=self.records.device)
        if ll:
            rc = _lib.lib().rt_attn_merge_ll_rows(
                self.ll_words[par].data_ptr(), self.epoch, wait_clocks, self.world, self.rows, self.dim,
                out.data_ptr() if out_dtype == torch.bfloat16 else None,
                out.data_ptr() if out_dtype == torch.float32 else None, lse.data_ptr(), _stream_ptr())
            _lib.check(rc, "rt_attn_merge_ll_rows")
            return out, lse
        rc = _lib.lib().rt_attn_merge_records_after_rows(
            self.records[par].data_ptr(), self.row_flags[par].data_ptr(), self.epoch, wait_clocks, self.world, self.rows,
            self.dim, out.data_ptr() if out_dtype == torch.bfloat16 else None,
            out.data_ptr() if out_dtype == torch.float32 else None, lse.data_ptr(), _stream_ptr())
        _lib.check(rc, "rt_attn_merge_records_after_rows")
        return out, lse

    def push(self):
        import ctypes
        from . import _lib
        from .gqa import _stream_ptr
        par = self.epoch & 1
        rec_bytes = self.rows * (self.dim + 1) * 4
        slot_off = (par * self.world + self.rank) * rec_bytes
        flag_off = (par * self.world + self.rank) * 4
        slots = (ctypes.c_void_p * self.world)(*[p + slot_off for p in self.record_ptrs])
        flags = (ctypes.c_void_p * self.world)(*[p + flag_off for p in self.flag_ptrs])
        rc = _lib.lib().rt_splitkv_push_record(self.records[par, self.rank].data_ptr(), slots, flags, self.world,
                                               self.rows, self.dim, self.epoch, _stream_ptr())
        _lib.check(rc, "rt_splitkv_push_record")

    def merge(self, out_dtype=None, wait_clocks: int = 0):
        import torch
        from . import _lib
        from .gqa import _stream_ptr
        par = self.epoch & 1
        out_dtype = out_dtype or torch.bfloat16
        out = torch.empty((self.rows, self.dim), dtype=out_dtype, device=self.records.device)
        lse = torch.empty((self.rows,), dtype=torch.float32, device=self.records.device)
        rc = _lib.lib().rt_attn_merge_records_after(self.records[par].data_ptr(), self.flags[par].data_ptr(), self.epoch,
                                                    wait_clocks, self.world, self.rows, self.dim,
                                                    out.data_ptr() if out_dtype == torch.bfloat16 else None,
                                                    out.data_ptr() if out_dtype == torch.float32 else None,
                                                    lse.data_ptr(), _stream_ptr())
        _lib.check(rc, "rt_attn_merge_records_after")
        return out, lse
