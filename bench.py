#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py --gpus N --steps K --warmup W            (N>1: launched under torch.distributed.run)
    python bench.py --impl reference --gpus N --steps K --warmup W

Headline workload (one "step" = one pass of the hot path over one batch of synthetic input):
causal prefill, bf16, B=4 H=32 N=4096 D=128 per GPU, Q,K,V ~ N(0,1) from a seed, scale 1/sqrt(128),
output bf16 + f32 LSE.  `value` is attention TFLOP/s with inputs resident in HBM, counting only the
unmasked (query,key) pairs: FLOPs = 4*D*B*H*N(N+1)/2.  `e2e` is the same metric through the C-ABI
host entry (pinned host buffers, H2D and D2H inside the timed region).  The same JSON line carries
the HBM-bound half of the metric under "decode" (batched GQA decode, B=64 Hq=32 Hkv=8 D=128, cache of
8192 positions, lengths ~ U[1024,8192]: KV-read GB/s = 4096 B * sum(len) / time) and, on N>1 GPUs,
"decode_splitkv" (KV range sharded over the ranks, (O,LSE) partials all-gathered with NCCL and merged).

Multi-GPU: (b,h) units are independent, so every rank runs the workload on its own shard with no
data-path collective (weak scaling: per-GPU work fixed); only the split-KV decode exchanges data.

`--impl reference` times the CPU restatement of the reference's rayon flash-attention path (the
reference is Rust and cannot be built on this machine) on all host cores, on a bounded sample of the
same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CFG2 = dict(B=4, H=32, N=4096, D=128)
CFG4 = dict(B=64, Hq=32, Hkv=8, D=128, S=8192, lo=1024, hi=8192)
CFG5_TOKENS_PER_GPU = 131072  # 1,048,576 / 8

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    except Exception:
        return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0, source="fallback")


def load_traffic():
    """DRAM bytes per launch of the dominant kernels, taken from the committed ncu summaries."""
    out = {}
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.txt")) as f:
            for line in f:
                parts = line.split()
                if len(parts) == 2 and not line.startswith("#"):
                    out[parts[0]] = int(parts[1])
    except Exception:
        pass
    return out


def prefill_flops(B, H, N, D):
    return 4.0 * D * B * H * (N * (N + 1) / 2.0)


# ------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while a timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nv = None

    def _loop(self):
        nv = self._nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self._nv:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# ------------------------------------------------------------------------------------------ CPU arm
def cpu_flash_sample(steps: int, warmup: int, target_seconds: float | None):
    """Times the oracle's tiled flash forward (one task per (b,h), all host threads) on `slabs`
    (b,h) slabs of the headline workload.  Returns (TFLOP/s algorithmic, cores, slabs, s/step)."""
    import numpy as np
    from oracle import oracle as orc

    # torchrun exports OMP_NUM_THREADS=1; the CPU arm uses every core this process may run on.
    orc.set_threads(len(os.sched_getaffinity(0)))
    cores = orc.get_threads()
    N, D = CFG2["N"], CFG2["D"]
    slabs = min(CFG2["B"] * CFG2["H"], max(8, cores))
    q, k, v = (orc.round_to_bf16(orc.fill_normal((1, slabs, N, D), s)) for s in (0xC0FFEE, 0xBADBEEF, 0xCAFE00))
    for _ in range(max(0, warmup)):
        orc.flash_forward_ext(q, k, v, causal=True)
    times = []
    t_begin = time.perf_counter()
    for i in range(max(1, steps)):
        t0 = time.perf_counter()
        rc, _, _ = orc.flash_forward_ext(q, k, v, causal=True)
        times.append(time.perf_counter() - t0)
        assert rc == 0
        if target_seconds is not None and time.perf_counter() - t_begin > target_seconds:
            break
    per_step = float(np.mean(times))
    return prefill_flops(1, slabs, N, D) / per_step / 1e12, cores, slabs, per_step, len(times)


def cpu_decode_sample(n_seq: int = 8, reps: int = 3):
    """Times the oracle's cache decode (decode_attn_row over (sequence, head), gqa.rs:216-270) on `n_seq`
    sequences of the config-4 geometry, serial as the reference runs seq_q == 1 (gqa.rs:190-198) and
    over all host threads.  Bytes are counted as for the GPU (bf16 K and V once per cached token)."""
    import numpy as np
    from oracle import oracle as orc
    orc.set_threads(len(os.sched_getaffinity(0)))
    cores = orc.get_threads()
    c = CFG4
    lens = orc.fill_uniform_int(n_seq, 0x5EED, c["lo"], c["hi"])
    q = orc.round_to_bf16(orc.fill_normal((n_seq, c["Hq"], c["D"]), 0xC0FFEE))
    k = orc.round_to_bf16(orc.fill_normal((n_seq, c["Hkv"], c["S"], c["D"]), 0xBADBEEF))
    v = orc.round_to_bf16(orc.fill_normal((n_seq, c["Hkv"], c["S"], c["D"]), 0xCAFE00))
    kv_bytes = 2.0 * c["Hkv"] * c["D"] * 2 * float(lens.sum())
    out = {}
    for label, par in (("all_cores", True), ("serial_as_written", False)):
        orc.gqa_decode_cache(q, k, v, lens, parallel=par)
        ts = []
        for _ in range(reps):
            t0 = time.perf_counter()
            rc, _, _ = orc.gqa_decode_cache(q, k, v, lens, parallel=par)
            ts.append(time.perf_counter() - t0)
            assert rc == 0
        out[label] = kv_bytes / float(np.median(ts)) / 1e9
    return out, cores, n_seq


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    tf, cores, slabs, per_step, done = cpu_flash_sample(args.steps, args.warmup, None)
    sample = (f"{slabs} of {CFG2['B'] * CFG2['H']} (b,h) slabs of the workload per step (N={CFG2['N']} D={CFG2['D']} "
              f"causal, f32 math on bf16-rounded inputs), C restatement of the reference's rayon path, {cores} threads")
    line = {
        "impl": "reference", "metric": "attn_prefill_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": done, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "causal prefill B=4 H=32 N=4096 D=128 (BASELINE config 2), bounded sample",
                   "sample_slabs": slabs},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ------------------------------------------------------------------------------------------ GPU arm
def timed(fn, steps, warmup, dist_mod, torch):
    """W untimed + K timed calls bracketed by barrier + synchronize; CUDA events on the launch stream;
    returns the max over ranks of the average ms per step."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist_mod is not None:
        dist_mod.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if dist_mod is not None:
        dist_mod.barrier()
    ms = e0.elapsed_time(e1) / steps
    if dist_mod is not None:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist_mod.all_reduce(t, op=dist_mod.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-cpu", action="store_true", help="skip the cpu_baseline leg (profiling runs)")
    ap.add_argument("--only", default="", help="comma list of legs: prefill,e2e,decode,splitkv,backward,published (default all)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        return run_reference_arm(args)

    import torch
    import rustorch_b200 as rt
    from rustorch_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist = dist_mod
    n_gpus = world
    legs = set(args.only.split(",")) if args.only else {"prefill", "e2e", "decode", "splitkv", "backward", "published"}
    peaks = load_peaks()
    traffic = load_traffic()
    lib = _lib.lib()
    out_line = {}

    # ---------------------------------------------------------------- prefill (headline)
    B, H, N, D = CFG2["B"], CFG2["H"], CFG2["N"], CFG2["D"]
    g = torch.Generator(device="cuda").manual_seed(0xC0FFEE + rank)
    q, k, v = (torch.randn((B, H, N, D), device="cuda", generator=g).to(torch.bfloat16) for _ in range(3))
    o = torch.empty_like(q)
    lse = torch.empty((B, H, N), dtype=torch.float32, device="cuda")
    flops = prefill_flops(B, H, N, D)

    def step_prefill():
        rt.prefill_bf16(q, k, v, causal=True, out=o, lse=lse)

    with ClockSampler(local_rank) as clk:
        ms = timed(step_prefill, args.steps, args.warmup, dist, torch)
    status = _lib.device_status()
    if status != 0:
        raise RuntimeError(f"device status word {status}: a bounded wait expired inside the prefill kernel")
    per_gpu_tflops = flops / (ms * 1e-3) / 1e12
    value = per_gpu_tflops * n_gpus
    clocks = clk.summary()

    # ---------------------------------------------------------------- e2e through the C-ABI host entry
    e2e = None
    if "e2e" in legs:
        hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
        ho = torch.empty_like(hq).pin_memory()
        hl = torch.empty((B, H, N), dtype=torch.float32).pin_memory()

        def step_e2e():
            rc = lib.rt_attn_prefill_bf16_host(hq.data_ptr(), hk.data_ptr(), hv.data_ptr(), ho.data_ptr(),
                                               hl.data_ptr(), B, H, N, D, _lib.RT_MASK_CAUSAL, None, -1.0)
            _lib.check(rc, "rt_attn_prefill_bf16_host")

        e2e_steps = max(3, min(args.steps, 10))
        for _ in range(2):
            step_e2e()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            step_e2e()  # blocks until the result is back in host memory
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
        if dist is not None:
            t = torch.tensor([e2e_ms], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
        e2e = {"value": n_gpus * flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": int(3 * q.numel() * 2), "d2h_bytes_per_step": int(o.numel() * 2 + lse.numel() * 4),
               "steps": e2e_steps, "api": "rt_attn_prefill_bf16_host (pinned host buffers, copies inside the timed region)"}
        assert torch.equal(ho.cuda(), o), "host entry and device entry disagree"
        del hq, hk, hv, ho, hl
    del q, k, v, o, lse
    torch.cuda.empty_cache()

    # ---------------------------------------------------------------- decode (HBM-bound half of the metric)
    decode = None
    if "decode" in legs:
        c = CFG4
        g = torch.Generator(device="cuda").manual_seed(0x5EED + rank)
        qd = torch.randn((c["B"], c["Hq"], c["D"]), device="cuda", generator=g).to(torch.bfloat16)
        kc = torch.randn((c["B"], c["Hkv"], c["S"], c["D"]), device="cuda", generator=g).to(torch.bfloat16)
        vc = torch.randn((c["B"], c["Hkv"], c["S"], c["D"]), device="cuda", generator=g).to(torch.bfloat16)
        lens = torch.randint(c["lo"], c["hi"] + 1, (c["B"],), device="cuda", generator=g, dtype=torch.int32)
        kv_bytes = 2.0 * c["Hkv"] * c["D"] * 2 * float(lens.sum().item())

        def step_decode():
            rt.gqa_decode(qd, kc, vc, kv_lens=lens)

        with ClockSampler(local_rank) as dclk:
            dms = timed(step_decode, args.steps, args.warmup, dist, torch)
        gbs = kv_bytes / (dms * 1e-3) / 1e9
        decode = {"metric": "kv_read_gbs", "value": gbs * n_gpus, "unit": "GB/s", "ms_per_step": dms,
                  "config": {"workload": "batched GQA decode B=64 Hq=32 Hkv=8 D=128 max_seq=8192 lens~U[1024,8192] per GPU "
                                         "(BASELINE config 4)", "kv_bytes_per_step": kv_bytes,
                             "l2": "1.2 GB of KV streamed per step, far larger than L2"},
                  "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                               "frac": gbs / peaks["hbm_gbs"], "peak_source": peaks["source"],
                               "traffic": traffic.get("gqa_decode_tc_kernel")},
                  "gpu_launches": args.steps, "clocks": dclk.summary()}
        if rank == 0 and n_gpus == 1 and not args.skip_cpu:
            gb, cores_d, nseq = cpu_decode_sample()
            decode["cpu_baseline"] = {"value": gb["all_cores"], "unit": "GB/s", "cores": cores_d, "kind": "port",
                                      "serial_as_written": gb["serial_as_written"],
                                      "sample": f"{nseq} of 64 sequences of the workload, median of 3; C restatement of "
                                                f"decode_attn_row over (sequence, head), f32 caches read by the CPU, "
                                                f"bytes counted as bf16 K and V once per cached token"}
        del qd, kc, vc
        torch.cuda.empty_cache()

    # ---------------------------------------------------------------- long-context split-KV decode (N>1 only)
    splitkv = None
    if "splitkv" in legs and dist is not None:
        Hq, Hkv, Dd, T = 32, 8, 128, CFG5_TOKENS_PER_GPU
        g = torch.Generator(device="cuda").manual_seed(0xBEEF)  # the same q on every rank
        q1 = torch.randn((1, Hq, Dd), device="cuda", generator=g).to(torch.bfloat16)
        g = torch.Generator(device="cuda").manual_seed(0xF00D + rank)
        k1 = torch.randn((1, Hkv, T, Dd), device="cuda", generator=g).to(torch.bfloat16)
        v1 = torch.randn((1, Hkv, T, Dd), device="cuda", generator=g).to(torch.bfloat16)
        from rustorch_b200 import sharding
        ws = torch.empty(rt.decode_workspace_bytes(1, Hq, Hkv, Dd, T), dtype=torch.uint8, device="cuda")

        def step_splitkv_nccl():
            # local shard -> packed (O | LSE) record; one 16.5 KB record per rank over NCCL; local merge
            rec = rt.gqa_decode_record(q1, k1, v1, kv_len=T, workspace=ws)
            return rt.merge_records(sharding.all_gather_partials(rec))

        # The same exchange over peer memory: the record is decoded straight into this rank's slot, pushed
        # to every peer with NVLink stores + a flag, and the merge kernel waits (bounded) for all flags.
        exchange, exchange_note = None, "peer stores over NVLink (symmetric memory) + flag, merge waits in-kernel; value = the faster of the copy-kernel and fused-in-merge forms"
        try:
            exchange = sharding.PeerRecordExchange.create(Hq, Dd)
        except Exception as exc:  # symmetric memory not available: keep the NCCL form, and say so
            exchange_note = f"NCCL all-gather (peer exchange unavailable: {type(exc).__name__}: {exc})"[:200]

        def step_splitkv_p2p():
            rt.gqa_decode_record(q1, k1, v1, kv_len=T, workspace=ws, record=exchange.next_epoch())
            exchange.push()   # copy kernel: 16-byte peer stores, then the flags
            return exchange.merge()

        def step_splitkv_p2p_fused():
            exchange.decode_push(q1, k1, v1, kv_len=T, workspace=ws)  # the merge kernel stores the record on every peer
            return exchange.merge()

        nccl_ms = timed(step_splitkv_nccl, args.steps, args.warmup, dist, torch)
        sms = nccl_ms
        if exchange is not None:
            a, b = step_splitkv_nccl(), step_splitkv_p2p()
            torch.cuda.synchronize()
            assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]), "peer exchange and NCCL exchange disagree"
            c = step_splitkv_p2p_fused()
            torch.cuda.synchronize()
            assert torch.equal(a[0], c[0]) and torch.equal(a[1], c[1]), "fused peer exchange and NCCL exchange disagree"
            sms_copy = timed(step_splitkv_p2p, args.steps, args.warmup, dist, torch)
            sms_fused = timed(step_splitkv_p2p_fused, args.steps, args.warmup, dist, torch)
            sms = min(sms_copy, sms_fused)
            from rustorch_b200 import _lib
            assert _lib.device_status() == 0, "a bounded wait of the peer exchange expired"
        total_bytes = 2.0 * Hkv * Dd * 2 * T * world
        splitkv = {"metric": "kv_read_gbs", "value": total_bytes / (sms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": sms,
                   "config": {"workload": f"split-KV decode B=1 Hq=32 Hkv=8 D=128, {T} KV positions per GPU "
                                          f"(BASELINE config 5 sharding), exchange of (O,LSE) records + merge",
                              "kv_len_total": T * world, "exchange": exchange_note},
                   "per_gpu_gbs": total_bytes / world / (sms * 1e-3) / 1e9,
                   "nccl_all_gather_ms_per_step": nccl_ms,
                   "peer_copy_kernel_ms_per_step": sms_copy if exchange is not None else None,
                   "peer_fused_in_merge_ms_per_step": sms_fused if exchange is not None else None}
        del k1, v1
        torch.cuda.empty_cache()

    # ---------------------------------------------------------------- backward (auxiliary line)
    backward = None
    if "backward" in legs and n_gpus == 1:
        g = torch.Generator(device="cuda").manual_seed(0xBAC0 + rank)
        qb, kb, vb, dob = (torch.randn((B, H, N, D), device="cuda", generator=g).to(torch.bfloat16) for _ in range(4))
        ob, lseb = rt.prefill_bf16(qb, kb, vb, causal=True)

        def step_backward():
            rt.backward_bf16(qb, kb, vb, ob, dob, lseb, causal=True)

        bsteps = max(3, min(args.steps, 20))
        bms = timed(step_backward, bsteps, 3, dist, torch)
        # five N x N x D products (S, dP, dV, dQ, dK) over the unmasked pairs, 2 flops per multiply-add
        btf = 2.5 * flops / (bms * 1e-3) / 1e12
        # the exact f32 companion on a smaller shape (CUDA cores)
        Bf, Hf, Nf, Df = 2, 8, 2048, 64
        qf, kf, vf, dof = (torch.randn((Bf, Hf, Nf, Df), device="cuda", generator=g) for _ in range(4))
        of, lsef = rt.prefill_f32(qf, kf, vf, causal=True)
        fms = timed(lambda: rt.backward_f32(qf, kf, vf, of, dof, lsef, causal=True), 3, 2, dist, torch)
        ftf = 10.0 * Df * Bf * Hf * (Nf * (Nf + 1) / 2) / (fms * 1e-3) / 1e12
        backward = {"metric": "attn_backward_tflops", "value": btf, "unit": "TFLOP/s", "ms_per_step": bms, "dtype": "bf16",
                    "steps": bsteps,
                    "config": {"workload": f"causal backward bf16 B={B} H={H} N={N} D={D} (dQ, dK, dV f32 from saved O, LSE)",
                               "flop_convention": "10*D*unmasked (q,k) pairs; the two-pass kernel executes 14*D (scores "
                                                  "and dP are recomputed in the second pass)",
                               "l2": "Q,K,V,O,dO bf16 + dQ,dK,dV f32 = 1 GiB per step, larger than the 126 MB L2"},
                    "roofline": {"bound": "tensor", "achieved": btf * 1.4, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                                 "frac": btf * 1.4 / peaks["bf16_tflops"], "peak_source": peaks["source"],
                                 "note": "mma.sync path (no tcgen05 yet); achieved counts the executed 14*D flops"},
                    "f32_companion": {"value": ftf, "unit": "TFLOP/s", "ms_per_step": fms,
                                      "workload": f"causal backward f32 B={Bf} H={Hf} N={Nf} D={Df}, CUDA cores"},
                    "gpu_launches": 3 * bsteps}
        del qb, kb, vb, dob, ob, lseb, qf, kf, vf, dof, of, lsef
        torch.cuda.empty_cache()

    # ---------------------------------------------------------------- the shapes the reference publishes numbers for
    published = None
    if "published" in legs and n_gpus == 1:
        g = torch.Generator(device="cuda").manual_seed(0x9B)
        rows = []

        def graph_ms(fn, iters=50):
            """The same call captured once into a CUDA graph and replayed: device-side time without the
            Python/ctypes cost of each enqueue.  None if the capture is refused."""
            try:
                fn()
                torch.cuda.synchronize()
                cg = torch.cuda.CUDAGraph()
                with torch.cuda.graph(cg):
                    fn()
                return timed(cg.replay, iters, 5, dist, torch)
            except Exception:
                return None

        # flash forward, unmasked, flops = 4*B*H*N^2*D (bench-vs-pytorch/benches/compare.rs:191); M4 Max CPU best runs
        for (Bp, Hp, Np, Dp, ref_ms) in ((2, 4, 2048, 64, 13.09), (1, 4, 1024, 64, 3.40), (1, 1, 512, 64, 0.783)):
            qf, kf, vf = (torch.randn((Bp, Hp, Np, Dp), device="cuda", generator=g) for _ in range(3))
            qh, kh, vh = (t.to(torch.bfloat16) for t in (qf, kf, vf))
            t16 = timed(lambda: rt.prefill_bf16(qh, kh, vh, causal=False), 20, 5, dist, torch)
            g16 = graph_ms(lambda: rt.prefill_bf16(qh, kh, vh, causal=False))
            t32 = timed(lambda: rt.prefill_f32(qf, kf, vf, causal=False), 5, 2, dist, torch)
            fl = 4.0 * Bp * Hp * Np * Np * Dp
            rows.append({"workload": f"flash forward B={Bp} H={Hp} N={Np} D={Dp}, no mask", "reference_ms": ref_ms,
                         "reference_hw": "Apple M4 Max CPU (published)", "bf16_tcgen05_ms": t16, "bf16_tcgen05_graph_replay_ms": g16,
                         "bf16_gflops": fl / t16 / 1e6, "f32_cuda_core_ms": t32})
        # Metal decode microbenchmarks: Hq=16 Hkv=2 D=256 f32 on the M4 Max GPU (rustorch-metal/src/kernels.rs:14314-14319)
        for kv, ref_us in ((64, 18.5), (256, 62.0), (1024, 238.0), (4096, 1474.0)):
            qd1 = torch.randn((1, 16, 256), device="cuda", generator=g).to(torch.bfloat16)
            kc1 = torch.randn((1, 2, 4096, 256), device="cuda", generator=g).to(torch.bfloat16)
            vc1 = torch.randn((1, 2, 4096, 256), device="cuda", generator=g).to(torch.bfloat16)
            td = timed(lambda: rt.gqa_decode(qd1, kc1, vc1, kv_len=kv), 50, 5, dist, torch)
            gd = graph_ms(lambda: rt.gqa_decode(qd1, kc1, vc1, kv_len=kv))
            rows.append({"workload": f"GQA decode Hq=16 Hkv=2 D=256 kv_len={kv}, batch 1", "reference_us": ref_us,
                         "reference_hw": "Apple M4 Max GPU, Metal NSG2 kernel (published)", "bf16_us": td * 1e3,
                         "bf16_graph_replay_us": None if gd is None else gd * 1e3,
                         "note": "bf16_us includes the Python/ctypes cost of each enqueue; graph replay is the same call "
                                 "captured once"})
        # the reference model's own decode call (LlamaModelCuda::decode_step, batch 1): no published number exists
        qd2 = torch.randn((1, 32, 128), device="cuda", generator=g).to(torch.bfloat16)
        kc2 = torch.randn((1, 8, 8192, 128), device="cuda", generator=g).to(torch.bfloat16)
        vc2 = torch.randn((1, 8, 8192, 128), device="cuda", generator=g).to(torch.bfloat16)
        od2 = torch.empty((1, 32, 128), device="cuda", dtype=torch.bfloat16)
        for kv in (1024, 4096, 8192):
            td = timed(lambda: rt.gqa_decode(qd2, kc2, vc2, kv_len=kv, out=od2, return_lse=False), 50, 5, dist, torch)
            gd = graph_ms(lambda: rt.gqa_decode(qd2, kc2, vc2, kv_len=kv, out=od2, return_lse=False))
            rows.append({"workload": f"GQA decode Hq=32 Hkv=8 D=128 kv_len={kv}, batch 1 (the reference model's call shape)",
                         "reference_us": None, "reference_hw": "not published", "bf16_us": td * 1e3,
                         "bf16_graph_replay_us": None if gd is None else gd * 1e3,
                         "kv_gbs_graph_replay": None if gd is None else 2.0 * 8 * 128 * 2 * kv / (gd * 1e-3) / 1e9})
        published = rows

    # ---------------------------------------------------------------- CPU baseline (rank 0, N = 1 only)
    cpu = None
    if rank == 0 and n_gpus == 1 and not args.skip_cpu:
        tf, cores, slabs, per_step, reps = cpu_flash_sample(8, 1, 12.0)
        cpu = {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port",
               "sample": f"{slabs} of {B * H} (b,h) slabs of the workload, {reps} repetitions, {per_step:.2f} s each; "
                         f"C restatement of the reference's rayon tiled path (visits every KV tile), all host threads"}

    if rank == 0:
        out_line = {
            "metric": "attn_prefill_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": n_gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "causal prefill bf16 B=4 H=32 N=4096 D=128 per GPU (BASELINE config 2), out bf16 + f32 LSE",
                       "flops_per_step_per_gpu": flops, "flop_convention": "4*D*unmasked (q,k) pairs",
                       "sharding": "independent (b,h) units per rank, no collective",
                       "l2": "Q,K,V,O = 512 MiB per step, larger than the 126 MB L2"},
            "roofline": {"bound": "tensor", "achieved": per_gpu_tflops, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": per_gpu_tflops / peaks["bf16_tflops"], "peak_source": peaks["source"],
                         "frac_of_sustained": per_gpu_tflops / peaks["bf16_tflops_sustained"],
                         "traffic": traffic.get("prefill_tc_kernel")},
            "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": args.steps, "clocks": clocks,
            "decode": decode, "decode_splitkv": splitkv, "backward": backward,
            "published_shapes": published,
        }
        print(json.dumps(out_line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
