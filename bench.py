#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py --gpus N --steps K --warmup W            (N>1: launched under torch.distributed.run)
    python bench.py --impl reference --gpus N --steps K --warmup W

Headline workload (one "step" = one pass of the hot path over one batch of synthetic input):
causal prefill, bf16, B=4 H=32 N=4096 D=128 per GPU, Q,K,V ~ N(0,1) from a seed, scale 1/sqrt(128),
output bf16 + f32 LSE.  `value` is attention TFLOP/s with inputs resident in HBM, counting only the
unmasked (query,key) pairs: FLOPs = 4*D*B*H*N(N+1)/2.  `e2e` is the same metric through the C-ABI
host entry (pinned host buffers, H2D and D2H inside the timed region).

The same JSON line carries every workload of the metric under "legs" (small prefill, headline
prefill, variable-length prefill, batched GQA decode, one GPU's shard of the long-context decode),
each with its time, achieved rate, roofline fraction and its parity against the CPU oracle measured
in the same run on a sample (outside every timed region); "decode" holds the HBM-bound half in full
(KV-read GB/s = 4096 B * sum(len) / time); on N>1 GPUs "decode_splitkv" is the long-context decode
with its KV range sharded over the ranks and the (O,LSE) records exchanged, and "strong" is the
fixed-size workloads partitioned over the ranks.

Multi-GPU: (b,h) units are independent, so every rank runs the workload on its own shard with no
data-path collective (weak scaling: per-GPU work fixed); only the split-KV decode exchanges data.

`--impl reference` times the CPU restatement of the reference's rayon flash-attention path (the
reference is Rust and cannot be built on this machine) on all host cores, on a bounded sample of the
same workload, with its tile products on register-blocked FMA micro-kernels (the stand-in for the
`gemm` crate the reference calls).
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

CFG1 = dict(B=1, H=8, N=2048, D=64)
CFG2 = dict(B=4, H=32, N=4096, D=128)
CFG3 = dict(B=16, H=16, N=2048, D=64, lo=256, hi=2048)
CFG4 = dict(B=64, Hq=32, Hkv=8, D=128, S=8192, lo=1024, hi=8192)
CFG5_TOKENS_PER_GPU = 131072  # 1,048,576 / 8
SEED_Q, SEED_K, SEED_V, SEED_LEN = 0xC0FFEE, 0xBADBEEF, 0xCAFE00, 0x5EED
HEADLINE = "causal prefill B=4 H=32 N=4096 D=128 (BASELINE config 2)"

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
    """DRAM bytes per launch of the dominant kernels, as captured once with ncu and committed under
    profiles/ (a static figure from that capture, not measured in this run)."""
    out = {}
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.txt")) as f:
            for line in f:
                parts = line.split()
                if len(parts) >= 2 and not line.startswith("#"):
                    out[parts[0]] = int(parts[1])
    except Exception:
        pass
    return out


TRAFFIC_SOURCE = {"prefill_tc_kernel": "ncu capture, committed: profiles/prefill_tc_kernel_cfg2.md",
                  "gqa_decode_tc_kernel": "ncu capture, committed: profiles/gqa_decode_tc_kernel_cfg4.md"}


def prefill_flops(B, H, N, D):
    return 4.0 * D * B * H * (N * (N + 1) / 2.0)


def varlen_flops(lens, H, N, D):
    """(all computed rows, valid rows only): padded query rows see every valid key (they are computed, as
    in the reference); valid rows see their causal prefix."""
    all_rows = sum(H * (l * (l + 1) / 2.0 + (N - l) * l) for l in lens)
    valid = sum(H * (l * (l + 1) / 2.0) for l in lens)
    return 4.0 * D * all_rows, 4.0 * D * valid


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
    """Times the CPU restatement of the reference's tiled flash forward (one task per (b,h), all host
    threads, every KV tile visited under the causal mask as the reference does) on `slabs` (b,h) slabs
    of the headline workload, tile products on the register-blocked micro-kernels.  Returns a dict."""
    import numpy as np
    from oracle import oracle as orc

    # torchrun exports OMP_NUM_THREADS=1; the CPU arm uses every core this process may run on.
    orc.set_threads(len(os.sched_getaffinity(0)))
    cores = orc.get_threads()
    N, D = CFG2["N"], CFG2["D"]
    slabs = min(CFG2["B"] * CFG2["H"], max(8, cores))
    q, k, v = (orc.round_to_bf16(orc.fill_normal((1, slabs, N, D), s)) for s in (SEED_Q, SEED_K, SEED_V))
    orc.set_gemm_kernel(1)
    try:
        for _ in range(max(0, warmup)):
            orc.flash_forward_ext(q, k, v, causal=True)
        times = []
        t_begin = time.perf_counter()
        for _ in range(max(1, steps)):
            t0 = time.perf_counter()
            rc, _, _ = orc.flash_forward_ext(q, k, v, causal=True)
            times.append(time.perf_counter() - t0)
            assert rc == 0
            if target_seconds is not None and time.perf_counter() - t_begin > target_seconds:
                break
    finally:
        orc.set_gemm_kernel(0)
    per_step = float(np.mean(times))
    executed = 4.0 * D * slabs * float(N) * N  # the reference multiplies every tile, masked or not
    peak = orc.fma_peak_gflops()
    per_core = executed / per_step / 1e9 / cores
    tile = orc.tile_gemm_gflops(D, 4000)
    return {"tflops": prefill_flops(1, slabs, N, D) / per_step / 1e12, "cores": cores, "slabs": slabs,
            "s_per_step": per_step, "reps": len(times), "executed_gflops_per_core": per_core,
            "fma_peak_gflops_per_core": peak, "isa": orc.micro_isa(), "tile_gemm_gflops_one_core": tile}


def cpu_sample_text(c):
    frac = c["executed_gflops_per_core"] / c["fma_peak_gflops_per_core"] if c["fma_peak_gflops_per_core"] else 0.0
    tfrac = c["tile_gemm_gflops_one_core"] / c["fma_peak_gflops_per_core"] if c["fma_peak_gflops_per_core"] else 0.0
    return (f"{c['slabs']} of {CFG2['B'] * CFG2['H']} (b,h) slabs of the workload per step, {c['reps']} repetitions, "
            f"{c['s_per_step']:.2f} s each; C restatement of the reference's rayon tiled path (visits every KV tile, "
            f"scalar expf and mask pass as the reference), {c['cores']} threads; tile GEMMs on {c['isa']} micro-kernels: "
            f"{c['tile_gemm_gflops_one_core']:.0f} GFLOP/s on one core alone = {tfrac:.2f} of its measured "
            f"{c['fma_peak_gflops_per_core']:.0f} GFLOP/s FMA peak; whole path executes "
            f"{c['executed_gflops_per_core']:.1f} GFLOP/s/core = {frac:.2f} of that peak")


def cpu_decode_sample(n_seq: int = 8, reps: int = 3):
    """Times the oracle's cache decode (decode_attn_row over (sequence, head), gqa.rs:216-270) on `n_seq`
    sequences of the batched-decode geometry, serial as the reference runs seq_q == 1 (gqa.rs:190-198) and
    over all host threads.  Bytes are counted as for the GPU (bf16 K and V once per cached token)."""
    import numpy as np
    from oracle import oracle as orc
    orc.set_threads(len(os.sched_getaffinity(0)))
    cores = orc.get_threads()
    c = CFG4
    lens = orc.fill_uniform_int(n_seq, SEED_LEN, c["lo"], c["hi"])
    q = orc.round_to_bf16(orc.fill_normal((n_seq, c["Hq"], c["D"]), SEED_Q))
    k = orc.round_to_bf16(orc.fill_normal((n_seq, c["Hkv"], c["S"], c["D"]), SEED_K))
    v = orc.round_to_bf16(orc.fill_normal((n_seq, c["Hkv"], c["S"], c["D"]), SEED_V))
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
    c = cpu_flash_sample(args.steps, args.warmup, None)
    line = {
        "impl": "reference", "metric": "attn_prefill_tflops", "value": c["tflops"], "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": c["reps"], "warmup": args.warmup, "ms_per_step": c["s_per_step"] * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": HEADLINE, "sample": f"{c['slabs']} of 128 (b,h) slabs per step; a rate, so the sample "
                                                   f"size does not enter the value", "sample_slabs": c["slabs"]},
        "cpu_baseline": {"value": c["tflops"], "unit": "TFLOP/s", "cores": c["cores"], "kind": "port",
                         "sample": cpu_sample_text(c)},
        "e2e": {"value": c["tflops"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ------------------------------------------------------------------------------------------ GPU arm
def timed(fn, steps, warmup, dist_mod, torch, per_rank=False):
    """W untimed + K timed calls bracketed by barrier + synchronize; CUDA events on the launch stream;
    returns the max over ranks of the average ms per step (and every rank's own figure if asked)."""
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
    ranks = [ms]
    if dist_mod is not None:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        allt = [torch.zeros_like(t) for _ in range(dist_mod.get_world_size())]
        dist_mod.all_gather(allt, t)
        ranks = [float(x.item()) for x in allt]
        ms = max(ranks)
    return (ms, ranks) if per_rank else ms


def timed_graph(fn, steps, warmup, dist_mod, torch):
    """The same K steps captured once into a CUDA graph and replayed once (each instantiated graph is replayed a
    single time: the exchange epochs baked into its launches must not repeat).  Removes the host from the timed
    region: with eight processes per box the Python enqueue of a 0.1 ms step is no longer negligible.
    Returns the max over ranks of the average ms per step."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist_mod is not None:
        dist_mod.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(steps):
            fn()
    torch.cuda.synchronize()
    if dist_mod is not None:
        dist_mod.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    if dist_mod is not None:
        dist_mod.barrier()
    ms = e0.elapsed_time(e1) / steps
    if dist_mod is not None:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist_mod.all_reduce(t, op=dist_mod.ReduceOp.MAX)
        ms = float(t.item())
    del g
    return ms


def rank_spread(ranks):
    s = sorted(ranks)
    return {"min": s[0], "median": s[len(s) // 2], "max": s[-1]}


def parity(got, ref, got_lse=None, ref_lse=None, bf16_out=True):
    """max-abs / relative-L2 / LSE error of a sample against the oracle, and whether they are inside the
    target tolerances (tests/util.py holds the same rule: 1e-2 max-abs, widened by half a bf16 ulp where
    |o| >= 4; 5e-3 relative L2; 1e-3 LSE)."""
    import numpy as np
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    ok = ~np.isnan(ref)
    nan_match = bool(np.array_equal(np.isnan(got), np.isnan(ref)))
    d = np.abs(got[ok] - ref[ok])
    a = np.abs(ref[ok])
    half_ulp = np.where(a >= 4.0, 2.0 ** (np.floor(np.log2(np.maximum(a, 1e-30))) - 8), 0.0) if bf16_out else 0.0
    within = bool(np.all(d <= 1e-2 + half_ulp)) if d.size else True
    rel = float(np.sqrt((d ** 2).sum()) / max(np.sqrt((ref[ok] ** 2).sum()), 1e-30)) if d.size else 0.0
    out = {"max_abs": float(d.max()) if d.size else 0.0, "rel_l2": rel, "ok": within and rel <= 5e-3 and nan_match}
    if got_lse is not None:
        gl, rl = np.asarray(got_lse, dtype=np.float64), np.asarray(ref_lse, dtype=np.float64)
        fin = np.isfinite(rl)
        out["lse_err"] = float(np.abs(gl[fin] - rl[fin]).max()) if fin.any() else 0.0
        out["ok"] = out["ok"] and out["lse_err"] <= 1e-3 and bool(np.array_equal(np.isfinite(gl), fin))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-cpu", action="store_true", help="skip the cpu_baseline and in-run parity legs (profiling runs)")
    ap.add_argument("--only", default="", help="comma list of legs: prefill,sustained,e2e,small,varlen,decode,shard,"
                                               "splitkv,strong,backward,published (default all)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        return run_reference_arm(args)

    import numpy as np
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
    all_legs = {"prefill", "sustained", "e2e", "small", "varlen", "decode", "shard", "splitkv", "strong", "backward",
                "published"}
    legs = set(args.only.split(",")) if args.only else all_legs
    check = not args.skip_cpu  # in-run parity against the oracle (outside every timed region)
    orc = None
    if check or (rank == 0 and n_gpus == 1 and not args.skip_cpu):
        from oracle import oracle as orc
        orc.set_threads(max(1, len(os.sched_getaffinity(0)) // max(1, world)))
    peaks = load_peaks()
    traffic = load_traffic()
    lib = _lib.lib()
    leg_map = {}

    def to_dev(x):
        return torch.from_numpy(np.ascontiguousarray(x)).cuda().to(torch.bfloat16).contiguous()

    def to_dev_f32(x):
        return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).cuda().contiguous()

    def f32(t):
        return t.detach().to(torch.float32).cpu().numpy()

    def tensor_leg(ms, flops, par, extra=None):
        tf = flops / (ms * 1e-3) / 1e12
        d = {"ms": ms, "achieved": tf, "unit": "TFLOP/s", "frac": tf / peaks["bf16_tflops"], "bound": "tensor"}
        if par:
            d.update({k: par[k] for k in ("max_abs", "lse_err", "rel_l2", "ok") if k in par})
        if extra:
            d.update(extra)
        return d

    def hbm_leg(ms, nbytes, par, extra=None):
        gb = nbytes / (ms * 1e-3) / 1e9
        d = {"ms": ms, "achieved": gb, "unit": "GB/s", "frac": gb / peaks["hbm_gbs"], "bound": "hbm"}
        if par:
            d.update({k: par[k] for k in ("max_abs", "lse_err", "rel_l2", "ok") if k in par})
        if extra:
            d.update(extra)
        return d

    # ---------------------------------------------------------------- prefill (headline)
    B, H, N, D = CFG2["B"], CFG2["H"], CFG2["N"], CFG2["D"]
    g = torch.Generator(device="cuda").manual_seed(SEED_Q + rank)
    q, k, v = (torch.randn((B, H, N, D), device="cuda", generator=g).to(torch.bfloat16) for _ in range(3))
    o = torch.empty_like(q)
    lse = torch.empty((B, H, N), dtype=torch.float32, device="cuda")
    flops = prefill_flops(B, H, N, D)

    def step_prefill():
        rt.prefill_bf16(q, k, v, causal=True, out=o, lse=lse)

    with ClockSampler(local_rank) as clk:
        ms, prefill_ranks = timed(step_prefill, args.steps, args.warmup, dist, torch, per_rank=True)
    status = _lib.device_status()
    if status != 0:
        raise RuntimeError(f"device status word {status}: a bounded wait expired inside the prefill kernel")
    per_gpu_tflops = flops / (ms * 1e-3) / 1e12
    value = per_gpu_tflops * n_gpus
    clocks = clk.summary()
    par2 = None
    if check:  # two (b,h) slabs of the step's own output against the oracle
        sel = [(0, 0), (B - 1, H - 1)]
        qs, ks, vs = (np.stack([f32(t[b, h]) for b, h in sel])[None] for t in (q, k, v))
        rc, ref, ref_lse = orc.flash_forward_ext(qs, ks, vs, causal=True)
        assert rc == 0
        par2 = parity(np.stack([f32(o[b, h]) for b, h in sel])[None], ref,
                      np.stack([f32(lse[b, h]) for b, h in sel])[None], ref_lse)
    leg_map["cfg2"] = tensor_leg(ms, flops, par2, {"parity_sample": "2 of 128 (b,h) slabs"})

    # ---------------------------------------------------------------- sustained: the same step back to back for >= 2 s
    sustained = None
    if "sustained" in legs:
        sus_steps = max(args.steps, int(2200.0 / ms) + 1)
        with ClockSampler(local_rank) as sclk:
            sus_ms = timed(step_prefill, sus_steps, 3, dist, torch)
        ss = sclk.summary()
        sus_tf = flops / (sus_ms * 1e-3) / 1e12
        sustained = {"value": sus_tf * n_gpus, "per_gpu": sus_tf, "unit": "TFLOP/s", "ms_per_step": sus_ms,
                     "steps": sus_steps, "seconds": sus_ms * sus_steps / 1e3, "sm_mhz_median": ss["sm_mhz"],
                     "reasons": ss["reasons"], "clock_samples": ss["samples"], "peak": peaks["bf16_tflops_sustained"],
                     "frac": sus_tf / peaks["bf16_tflops_sustained"],
                     "sm_clocks_per_step": None if not ss["sm_mhz"] else sus_ms * 1e-3 * ss["sm_mhz"] * 1e6,
                     "note": "frac divides a seconds-long measurement by the seconds-long cuBLAS peak; roofline.frac "
                             "divides the short timed region by the burst peak"}

    # ---------------------------------------------------------------- e2e through the C-ABI host entries
    e2e = None
    if "e2e" in legs:
        hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
        ho = torch.empty_like(hq).pin_memory()
        hl = torch.empty((B, H, N), dtype=torch.float32).pin_memory()

        def step_e2e():
            rc = lib.rt_attn_prefill_bf16_host(hq.data_ptr(), hk.data_ptr(), hv.data_ptr(), ho.data_ptr(),
                                               hl.data_ptr(), B, H, N, D, _lib.RT_MASK_CAUSAL, None, -1.0)
            _lib.check(rc, "rt_attn_prefill_bf16_host")

        def wall(fn, steps_):
            for _ in range(2):
                fn()
            if dist is not None:
                dist.barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(steps_):
                fn()  # blocks until the result is back in host memory
            torch.cuda.synchronize()
            w = (time.perf_counter() - t0) * 1e3 / steps_
            if dist is not None:
                t = torch.tensor([w], dtype=torch.float64, device="cuda")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                w = float(t.item())
            return w

        e2e_steps = max(3, min(args.steps, 10))
        e2e_ms = wall(step_e2e, e2e_steps)
        e2e = {"value": n_gpus * flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": int(3 * q.numel() * 2), "d2h_bytes_per_step": int(o.numel() * 2 + lse.numel() * 4),
               "steps": e2e_steps, "api": "rt_attn_prefill_bf16_host (pinned host buffers, copies inside the timed region)"}
        # The host entry runs the same kernel on (batch element, head range) chunks; small chunks take the
        # small-launch schedule, whose summation order differs, so the results agree to a bf16 ulp, not bit for bit.
        hd, od = ho.cuda().float(), o.float()
        host_dev_diff = float(((hd - od).abs() / od.abs().clamp(min=1.0)).max())
        assert host_dev_diff <= 2.0 ** -7, f"host entry and device entry disagree: {host_dev_diff}"
        e2e["max_rel_diff_vs_device_entry"] = host_dev_diff
        del hd, od
        del hq, hk, hv, ho, hl
        # The reference's own signature: flash_forward_masked(&AttentionShape, &[f32] q, k, v, &Mask, &mut [f32] out)
        # (cpu_forward.rs:193-200) -> rt_flash_forward_f32_host, f32 host slices in and out, bf16 tensor-core math.
        if n_gpus == 1:
            sig = {"api": "rt_flash_forward_f32_host(precision = BF16): f32 host slices in and out (pinned), causal"}
            for name, cfg in (("cfg1", CFG1), ("cfg2", CFG2)):
                shp = rt.AttentionShape.new(cfg["B"], cfg["H"], cfg["N"], cfg["D"])
                n_el = shp.buffer_len()
                bufs = [torch.randn(n_el, dtype=torch.float32).pin_memory() for _ in range(3)]
                outb = torch.empty(n_el, dtype=torch.float32).pin_memory()
                arrs = [b.numpy() for b in bufs]
                out_np = outb.numpy()

                def step_sig():
                    rt.flash_forward_masked(shp, arrs[0], arrs[1], arrs[2], rt.Mask.causal(), out_np, precision="bf16")

                w = wall(step_sig, 3 if name == "cfg2" else 10)
                fl = prefill_flops(cfg["B"], cfg["H"], cfg["N"], cfg["D"])
                sig[name] = {"ms_per_step": w, "tflops": fl / (w * 1e-3) / 1e12, "h2d_bytes_per_step": 3 * n_el * 4,
                             "d2h_bytes_per_step": n_el * 4}
                if name == "cfg1":  # the same call with the reference's default precision: exact f32 arithmetic
                    def step_sig_f32():
                        rt.flash_forward_masked(shp, arrs[0], arrs[1], arrs[2], rt.Mask.causal(), out_np, precision="f32")

                    w32 = wall(step_sig_f32, 10)
                    sig["cfg1_f32_precision"] = {"ms_per_step": w32, "tflops": fl / (w32 * 1e-3) / 1e12,
                                                 "h2d_bytes_per_step": 3 * n_el * 4, "d2h_bytes_per_step": n_el * 4}
                del bufs, outb, arrs, out_np
            e2e["reference_signature"] = sig

    # ---------------------------------------------------------------- backward (auxiliary line)
    backward = None
    if "backward" in legs and n_gpus == 1:
        gb = torch.Generator(device="cuda").manual_seed(0xBAC0 + rank)
        dob = torch.randn((B, H, N, D), device="cuda", generator=gb).to(torch.bfloat16)

        def step_backward():
            rt.backward_bf16(q, k, v, o, dob, lse, causal=True)

        bsteps = max(3, min(args.steps, 20))
        bms = timed(step_backward, bsteps, 3, dist, torch)
        # five N x N x D products (S, dP, dV, dQ, dK) over the unmasked pairs, 2 flops per multiply-add
        btf = 2.5 * flops / (bms * 1e-3) / 1e12
        backward = {"metric": "attn_backward_tflops", "value": btf, "unit": "TFLOP/s", "ms_per_step": bms, "dtype": "bf16",
                    "steps": bsteps,
                    "config": {"workload": f"causal backward bf16 B={B} H={H} N={N} D={D} (dQ, dK, dV f32 from saved O, LSE)",
                               "flop_convention": "10*D*unmasked (q,k) pairs",
                               "l2": "Q,K,V,O,dO bf16 + dQ,dK,dV f32 = 1 GiB per step, larger than the 126 MB L2"},
                    "roofline": {"bound": "tensor", "achieved": btf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                                 "frac": btf / peaks["bf16_tflops"], "peak_source": peaks["source"],
                                 "executed_frac": 1.4 * btf / peaks["bf16_tflops"],
                                 "note": "tcgen05 kernel, two deterministic passes: 14*D flops executed per pair (scores "
                                         "and dP are recomputed on the key side) for the 10*D counted"},
                    "gpu_launches": 3 * bsteps}
        del dob
    del q, k, v, o, lse
    torch.cuda.empty_cache()

    # ---------------------------------------------------------------- small prefill (B=1 H=8 N=2048 D=64, causal)
    if "small" in legs and n_gpus == 1:
        c = CFG1
        from oracle import oracle as orc_gen
        qn, kn, vn = (orc_gen.round_to_bf16(orc_gen.fill_normal((c["B"], c["H"], c["N"], c["D"]), s))
                      for s in (SEED_Q, SEED_K, SEED_V))
        # 48 rotating copies of the 3 MiB input set (144 MiB > the 126 MB L2): every step reads cold inputs
        R = 48
        qs = [to_dev(qn) for _ in range(R)]
        ks = [to_dev(kn) for _ in range(R)]
        vs = [to_dev(vn) for _ in range(R)]
        o1 = torch.empty_like(qs[0])
        l1 = torch.empty((c["B"], c["H"], c["N"]), dtype=torch.float32, device="cuda")
        it = [0]

        def step_small():
            i = it[0] = (it[0] + 1) % R
            rt.prefill_bf16(qs[i], ks[i], vs[i], causal=True, out=o1, lse=l1)

        ms1 = timed(step_small, max(args.steps, 20), 5, dist, torch)
        cg = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        with torch.cuda.graph(cg):
            for i in range(R):
                rt.prefill_bf16(qs[i], ks[i], vs[i], causal=True, out=o1, lse=l1)
        ms1g = timed(cg.replay, 4, 2, dist, torch) / R
        par1 = None
        if check:
            rc, ref, ref_lse = orc.flash_forward_ext(qn, kn, vn, causal=True)
            par1 = parity(f32(o1), ref, f32(l1), ref_lse)
        fl1 = prefill_flops(c["B"], c["H"], c["N"], c["D"])
        # The reference's literal arithmetic on this configuration is f32: the exact-f32 CUDA-core kernel
        # (held to the oracle at 1e-4) on f32 inputs of the same values, timed the same way (the f32 inputs
        # are the unrounded fill, so this row's parity is against the oracle on those).
        qf, kf, vf = (to_dev_f32(orc_gen.fill_normal((c["B"], c["H"], c["N"], c["D"]), s))
                      for s in (SEED_Q, SEED_K, SEED_V))
        of32, lf32 = rt.prefill_f32(qf, kf, vf, causal=True)
        ms_f32 = timed(lambda: rt.prefill_f32(qf, kf, vf, causal=True), max(args.steps, 20), 3, dist, torch)
        f32_row = {"ms": ms_f32, "tflops": fl1 / (ms_f32 * 1e-3) / 1e12,
                   "kernel": "prefill_f32_tiled_kernel (CUDA cores, f32 in / f32 accumulate / f32 out, rt_attn_prefill_f32)"}
        if check:
            qh, kh, vh = (orc_gen.fill_normal((c["B"], c["H"], c["N"], c["D"]), s) for s in (SEED_Q, SEED_K, SEED_V))
            rc32, ref32, ref_lse32 = orc.flash_forward_ext(qh, kh, vh, causal=True)
            f32_row["max_abs_vs_oracle"] = float(np.abs(of32.cpu().numpy() - ref32).max())
            f32_row["lse_err_vs_oracle"] = float(np.abs(lf32.cpu().numpy() - ref_lse32).max())
            f32_row["tolerance"] = 1e-4
            assert f32_row["max_abs_vs_oracle"] <= 1e-4, f32_row
            del qh, kh, vh
        del qf, kf, vf, of32, lf32
        leg_map["cfg1"] = tensor_leg(ms1g, fl1, par1, {
            "f32_exact": f32_row,
            "ms_per_call_from_python": ms1, "ms": ms1g,
            "note": "ms = device time per launch (48 launches on rotating inputs replayed from one CUDA graph); "
                    "ms_per_call_from_python adds the enqueue cost of one ctypes call per launch",
            "flops_reference_convention": 4.0 * c["B"] * c["H"] * c["N"] * c["N"] * c["D"]})
        del qs, ks, vs, o1, l1
        torch.cuda.empty_cache()

    # ---------------------------------------------------------------- variable-length prefill (B=16 H=16 N=2048 D=64)
    varlen_full_ms = None
    if "varlen" in legs:
        c = CFG3
        from oracle import oracle as orc_gen
        lens3 = orc_gen.fill_uniform_int(c["B"], SEED_LEN, c["lo"], c["hi"])
        shape3 = (c["B"], c["H"], c["N"], c["D"])
        q3n, k3n, v3n = (orc_gen.round_to_bf16(orc_gen.fill_normal(shape3, s)) for s in (SEED_Q, SEED_K, SEED_V))
        q3, k3, v3 = to_dev(q3n), to_dev(k3n), to_dev(v3n)
        l3d = torch.from_numpy(lens3).cuda()
        o3 = torch.empty_like(q3)
        ls3 = torch.empty(shape3[:3], dtype=torch.float32, device="cuda")

        def step_varlen():
            rt.prefill_bf16(q3, k3, v3, causal=True, kv_lens=l3d, out=o3, lse=ls3)

        ms3 = timed(step_varlen, args.steps, args.warmup, dist, torch)
        varlen_full_ms = ms3
        fl_all, fl_valid = varlen_flops([int(x) for x in lens3], c["H"], c["N"], c["D"])
        par3 = None
        if check:
            bsel = [int(np.argmin(lens3)), int(np.argmax(lens3))]
            hs = [0, c["H"] - 1]
            qq, kk, vv = (np.ascontiguousarray(t[bsel][:, hs]) for t in (q3n, k3n, v3n))
            rc, ref, ref_lse = orc.flash_forward_ext(qq, kk, vv, causal=True, kv_lens=lens3[bsel])
            par3 = parity(f32(o3)[bsel][:, hs], ref, f32(ls3)[bsel][:, hs], ref_lse)
        leg_map["cfg3"] = tensor_leg(ms3, fl_all, par3, {
            "achieved_valid_rows_only": fl_valid / (ms3 * 1e-3) / 1e12, "flops_all_computed_rows": fl_all,
            "flops_valid_rows_only": fl_valid, "parity_sample": "shortest and longest sequence x 2 heads",
            "l2": "Q,K,V,O = 256 MiB per step, larger than L2"})
        if dist is None:
            del q3, k3, v3, o3, ls3
        torch.cuda.empty_cache()

    # ---------------------------------------------------------------- decode (HBM-bound half of the metric)
    decode = None
    dms = None
    if "decode" in legs:
        c = CFG4
        # the same lengths on every rank (weak scaling: every GPU streams the same number of bytes), own values
        gl = torch.Generator(device="cuda").manual_seed(SEED_LEN)
        lens = torch.randint(c["lo"], c["hi"] + 1, (c["B"],), device="cuda", generator=gl, dtype=torch.int32)
        g = torch.Generator(device="cuda").manual_seed(SEED_LEN + 1 + rank)
        qd = torch.randn((c["B"], c["Hq"], c["D"]), device="cuda", generator=g).to(torch.bfloat16)
        kc = torch.randn((c["B"], c["Hkv"], c["S"], c["D"]), device="cuda", generator=g).to(torch.bfloat16)
        vc = torch.randn((c["B"], c["Hkv"], c["S"], c["D"]), device="cuda", generator=g).to(torch.bfloat16)
        kv_bytes = 2.0 * c["Hkv"] * c["D"] * 2 * float(lens.sum().item())
        od = torch.empty_like(qd)
        ld = torch.empty((c["B"], c["Hq"]), dtype=torch.float32, device="cuda")

        def step_decode():
            rt.gqa_decode(qd, kc, vc, kv_lens=lens, out=od, lse=ld)

        with ClockSampler(local_rank) as dclk:
            dms, dranks = timed(step_decode, args.steps, args.warmup, dist, torch, per_rank=True)
        gbs = kv_bytes / (dms * 1e-3) / 1e9
        par4 = None
        if check:
            sel = [0, c["B"] - 1]
            ln = lens.cpu().numpy()[sel]
            rc, ref, ref_lse = orc.gqa_decode_cache(f32(qd[sel]), f32(kc[sel]), f32(vc[sel]), ln)
            par4 = parity(f32(od[sel]), ref, f32(ld[sel]), ref_lse)
        decode = {"metric": "kv_read_gbs", "value": gbs * n_gpus, "unit": "GB/s", "ms_per_step": dms,
                  "config": {"workload": "batched GQA decode B=64 Hq=32 Hkv=8 D=128 max_seq=8192 lens~U[1024,8192] per GPU "
                                         "(BASELINE config 4)", "kv_bytes_per_step": kv_bytes,
                             "l2": "1.2 GB of KV streamed per step, far larger than L2"},
                  "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                               "frac": gbs / peaks["hbm_gbs"], "peak_source": peaks["source"],
                               "traffic": traffic.get("gqa_decode_tc_kernel"),
                               "traffic_source": TRAFFIC_SOURCE["gqa_decode_tc_kernel"]},
                  "gpu_launches": args.steps, "clocks": dclk.summary()}
        if dist is not None:
            # every rank streams its own 1.2 GB; ms_per_step is the slowest rank's average over the timed region
            decode["per_rank_ms"] = rank_spread(dranks)
            decode["per_rank_gbs_fastest"] = kv_bytes / (min(dranks) * 1e-3) / 1e9
            decode["per_rank_note"] = ("every rank streams the same byte count (same lengths, own values); value divides "
                                       "all ranks' bytes by the slowest rank's time, so the spread below is the spread "
                                       "of the GPUs' own HBM rates")
            t = torch.tensor([kv_bytes], dtype=torch.float64, device="cuda")
            allb = [torch.zeros_like(t) for _ in range(world)]
            dist.all_gather(allb, t)
            per_rank_gb = [float(x.item()) / (r * 1e-3) / 1e9 for x, r in zip(allb, dranks)]
            decode["per_rank_gbs"] = rank_spread(per_rank_gb)
            decode["value"] = sum(float(x.item()) for x in allb) / (dms * 1e-3) / 1e9
        if rank == 0 and n_gpus == 1 and not args.skip_cpu:
            gb, cores_d, nseq = cpu_decode_sample()
            decode["cpu_baseline"] = {"value": gb["all_cores"], "unit": "GB/s", "cores": cores_d, "kind": "port",
                                      "serial_as_written": gb["serial_as_written"],
                                      "sample": f"{nseq} of 64 sequences of the workload, median of 3; C restatement of "
                                                f"decode_attn_row over (sequence, head), f32 caches read by the CPU, "
                                                f"bytes counted as bf16 K and V once per cached token"}
        leg_map["cfg4"] = hbm_leg(dms, kv_bytes, par4, {"parity_sample": "2 of 64 sequences"})
        if dist is None or "strong" not in legs:
            del qd, kc, vc
        torch.cuda.empty_cache()

    # ---------------------------------------------------------------- strong scaling of the fixed-size workloads (N>1)
    strong = None
    if "strong" in legs and dist is not None:
        from rustorch_b200 import sharding
        strong = {"note": "the fixed-size workloads partitioned over the ranks with no collective; ms = slowest rank; "
                          "efficiency = full-workload time on one GPU (measured in this run on every rank) / (N * ms)"}
        # headline prefill: 128 (b,h) units, contiguous slabs per rank
        u0, u1 = sharding.shard_units(B * H, world, rank)
        g = torch.Generator(device="cuda").manual_seed(SEED_Q + rank)
        qs_, ks_, vs_ = (torch.randn((1, u1 - u0, N, D), device="cuda", generator=g).to(torch.bfloat16) for _ in range(3))
        os_ = torch.empty_like(qs_)
        sms, sr = timed(lambda: rt.prefill_bf16(qs_, ks_, vs_, causal=True, out=os_, return_lse=False), args.steps,
                        args.warmup, dist, torch, per_rank=True)
        strong["cfg2"] = {"units_per_rank": u1 - u0, "ms": sms, "tflops_aggregate": flops / (sms * 1e-3) / 1e12,
                          "efficiency": ms / (world * sms), "imbalance": max(sr) / (sum(sr) / len(sr)),
                          "bound": "tensor pipe; with 16 units per rank the grid is 128 CTAs < 148 SMs at N=8"}
        del qs_, ks_, vs_, os_
        if "decode" in legs:
            # batched decode: sequences balanced on their lengths (every rank derives the same assignment)
            c = CFG4
            g = torch.Generator(device="cuda").manual_seed(SEED_LEN)  # the same workload on every rank
            qd0 = torch.randn((c["B"], c["Hq"], c["D"]), device="cuda", generator=g).to(torch.bfloat16)
            kc.copy_(torch.randn(kc.shape, device="cuda", generator=g).to(torch.bfloat16))
            vc.copy_(torch.randn(vc.shape, device="cuda", generator=g).to(torch.bfloat16))
            lens0 = torch.randint(c["lo"], c["hi"] + 1, (c["B"],), device="cuda", generator=g, dtype=torch.int32)
            ln0 = [int(x) for x in lens0.cpu().numpy()]
            mine = sharding.balance_sequences(ln0, world)[rank]
            ix = torch.tensor(mine, device="cuda")
            qm, km, vm, lm = qd0[ix].contiguous(), kc[ix].contiguous(), vc[ix].contiguous(), lens0[ix].contiguous()
            full_ms = timed(lambda: rt.gqa_decode(qd0, kc, vc, kv_lens=lens0), args.steps, args.warmup, dist, torch)
            sms, sr = timed(lambda: rt.gqa_decode(qm, km, vm, kv_lens=lm), args.steps, args.warmup, dist, torch,
                            per_rank=True)
            tot = 2.0 * c["Hkv"] * c["D"] * 2 * float(sum(ln0))
            strong["cfg4"] = {"sequences_per_rank": len(mine), "ms": sms, "gbs_aggregate": tot / (sms * 1e-3) / 1e9,
                              "efficiency": full_ms / (world * sms), "imbalance": max(sr) / (sum(sr) / len(sr)),
                              "full_workload_ms_one_gpu": full_ms,
                              "bound": "HBM; 150 MB per rank at N=8 is 25 us of streaming, the launch and the tail count"}
            del qd0, qm, km, vm, qd, kc, vc
        if "varlen" in legs:
            c = CFG3
            cost = [float(l) * float(l) for l in lens3]
            mine = sharding.balance_sequences(cost, world)[rank]
            ix = torch.tensor(mine, device="cuda")
            qm, km, vm, lm = q3[ix].contiguous(), k3[ix].contiguous(), v3[ix].contiguous(), l3d[ix].contiguous()
            om = torch.empty_like(qm)
            sms, sr = timed(lambda: rt.prefill_bf16(qm, km, vm, causal=True, kv_lens=lm, out=om, return_lse=False),
                            args.steps, args.warmup, dist, torch, per_rank=True)
            fl_all, _ = varlen_flops([int(x) for x in lens3], c["H"], c["N"], c["D"])
            strong["cfg3"] = {"sequences_per_rank": len(mine), "ms": sms, "tflops_aggregate": fl_all / (sms * 1e-3) / 1e12,
                              "efficiency": varlen_full_ms / (world * sms), "imbalance": max(sr) / (sum(sr) / len(sr)),
                              "assignment": "longest-processing-time on len^2",
                              "bound": "2 sequences x 16 heads per rank at N=8: too few CTAs to fill 148 SMs"}
            del q3, k3, v3, o3, ls3, qm, km, vm, om
        torch.cuda.empty_cache()

    # ---------------------------------------------------------------- one GPU's shard of the long-context decode
    Hq, Hkv, Dd, T = 32, 8, 128, CFG5_TOKENS_PER_GPU
    shard_bytes = 2.0 * Hkv * Dd * 2 * T
    q1 = k1 = v1 = ws = None
    if "shard" in legs or ("splitkv" in legs and dist is not None):
        g = torch.Generator(device="cuda").manual_seed(0xBEEF)  # the same q on every rank
        q1 = torch.randn((1, Hq, Dd), device="cuda", generator=g).to(torch.bfloat16)
        g = torch.Generator(device="cuda").manual_seed(0xF00D + rank)
        k1 = torch.randn((1, Hkv, T, Dd), device="cuda", generator=g).to(torch.bfloat16)
        v1 = torch.randn((1, Hkv, T, Dd), device="cuda", generator=g).to(torch.bfloat16)
        ws = torch.empty(rt.decode_workspace_bytes(1, Hq, Hkv, Dd, T), dtype=torch.uint8, device="cuda")
    if "shard" in legs:
        rec = torch.empty((Hq, Dd + 1), dtype=torch.float32, device="cuda")

        def step_shard():
            rt.gqa_decode_record(q1, k1, v1, kv_len=T, workspace=ws, record=rec)

        ms5 = timed(step_shard, args.steps, args.warmup, dist, torch)
        par5 = None
        if check and rank == 0:
            rc, ref, ref_lse = orc.gqa_decode_cache(f32(q1), f32(k1), f32(v1), np.array([T], dtype=np.int32))
            r = f32(rec)
            par5 = parity(r[:, :Dd][None], ref, r[:, Dd][None], ref_lse, bf16_out=False)
        leg_map["cfg5_shard"] = hbm_leg(ms5, shard_bytes, par5, {
            "note": "B=1, 131072 cached positions (512 MiB of K and V) on one GPU: decode + chunk merge into the "
                    "(O | LSE) record a rank contributes to the exchange; parity on the whole shard"})
        del rec

    # ---------------------------------------------------------------- long-context split-KV decode (N>1 only)
    splitkv = None
    if "splitkv" in legs and dist is not None:
        from rustorch_b200 import sharding

        def step_splitkv_nccl():
            # local shard -> packed (O | LSE) record; one 16.5 KB record per rank over NCCL; local merge
            r = rt.gqa_decode_record(q1, k1, v1, kv_len=T, workspace=ws)
            return rt.merge_records(sharding.all_gather_partials(r))

        # The same exchange over peer memory: the record is decoded straight into this rank's slot, pushed
        # to every peer with NVLink stores + a flag, and the merge kernel waits (bounded) for all flags.
        exchange, exchange_note = None, ("peer stores over NVLink (symmetric memory), flags or flag-in-word rows, the merge waits in-kernel; "
                                         "value = the fastest of the forms timed below")
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

        def step_splitkv_rows():
            # decode kernel, then ONE kernel: chunk merge, row delivery, per-row wait, cross-rank merge
            return exchange.decode_exchange(q1, k1, v1, kv_len=T, workspace=ws)

        def step_splitkv_ll():
            # the same, every element as an 8-byte {value, epoch} word: no fence, no flag store, the reader spins on the words
            return exchange.decode_exchange(q1, k1, v1, kv_len=T, workspace=ws, ll=True)

        # Verification over real peer memory, before anything is timed: every rank holds the SAME small cache
        # (4096 positions per rank), decodes only its own KV range, exchanges, and compares the merged result
        # with its own single-GPU decode of the whole range.
        verified, verify_err = None, None
        if exchange is not None:
            Tv = 4096 * world
            g = torch.Generator(device="cuda").manual_seed(0xACE)
            kv_ = torch.randn((1, Hkv, Tv, Dd), device="cuda", generator=g).to(torch.bfloat16)
            vv_ = torch.randn((1, Hkv, Tv, Dd), device="cuda", generator=g).to(torch.bfloat16)
            whole, whole_lse = rt.gqa_decode(q1, kv_, vv_, kv_len=Tv, out_dtype=torch.float32)
            b0, b1 = sharding.kv_shard(Tv, world, rank, align=16)
            errs = []
            for form in ("copy", "fused", "rows", "ll"):
                if form == "copy":
                    rt.gqa_decode_record(q1, kv_, vv_, kv_len=Tv, kv_begin=b0, kv_end=b1, record=exchange.next_epoch())
                    exchange.push()
                elif form == "fused":
                    exchange.decode_push(q1, kv_, vv_, kv_len=Tv, kv_begin=b0, kv_end=b1)
                if form in ("rows", "ll"):
                    got, got_lse = exchange.decode_exchange(q1, kv_, vv_, kv_len=Tv, kv_begin=b0, kv_end=b1,
                                                            out_dtype=torch.float32, ll=(form == "ll"))
                else:
                    got, got_lse = exchange.merge(out_dtype=torch.float32)
                torch.cuda.synchronize()
                errs.append(max((got - whole.reshape(Hq, Dd)).abs().max().item(),
                                (got_lse - whole_lse.reshape(Hq)).abs().max().item()))
            t = torch.tensor([max(errs)], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            verify_err = float(t.item())
            verified = bool(verify_err <= 1e-3 and _lib.device_status() == 0)
            del kv_, vv_

        nccl_ms = timed(step_splitkv_nccl, args.steps, args.warmup, dist, torch)
        sms = nccl_ms
        sms_copy = sms_fused = sms_rows = sms_rows_graph = sms_copy_graph = sms_ll = sms_ll_graph = None
        if exchange is not None:
            a, b = step_splitkv_nccl(), step_splitkv_p2p()
            torch.cuda.synchronize()
            assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]), "peer exchange and NCCL exchange disagree"
            cc = step_splitkv_p2p_fused()  # chunks merged inside the decode kernel: another summation order
            torch.cuda.synchronize()
            assert (a[0].float() - cc[0].float()).abs().max().item() <= 2e-2 and (a[1] - cc[1]).abs().max().item() <= 1e-5, \
                "fused peer exchange and NCCL exchange disagree"
            sms_copy = timed(step_splitkv_p2p, args.steps, args.warmup, dist, torch)
            sms_fused = timed(step_splitkv_p2p_fused, args.steps, args.warmup, dist, torch)
            dd = step_splitkv_rows()
            torch.cuda.synchronize()
            assert (a[0].float() - dd[0].float()).abs().max().item() <= 2e-2 and (a[1] - dd[1]).abs().max().item() <= 1e-5, \
                "row exchange and NCCL exchange disagree"
            sms_rows = timed(step_splitkv_rows, args.steps, args.warmup, dist, torch)
            # the two best forms again with the steps replayed from one CUDA graph per rank (no host in the loop)
            def graph_or_none(step):
                # a refused capture must not cost the line: the step-by-step timing of the same form stands.  Every
                # rank takes the same branch (the capture fails on all or none: same code, same library).
                try:
                    return timed_graph(step, args.steps, args.warmup, dist, torch)
                except Exception as exc:
                    sys.stderr.write(f"[bench] graph replay of {step.__name__} not timed: {type(exc).__name__}: {exc}\n")
                    torch.cuda.synchronize()
                    return None

            sms_rows_graph = graph_or_none(step_splitkv_rows)
            sms_copy_graph = graph_or_none(step_splitkv_p2p)
            ee = step_splitkv_ll()
            torch.cuda.synchronize()
            assert (a[0].float() - ee[0].float()).abs().max().item() <= 2e-2 and (a[1] - ee[1]).abs().max().item() <= 1e-5, \
                "word exchange and NCCL exchange disagree"
            sms_ll = timed(step_splitkv_ll, args.steps, args.warmup, dist, torch)
            sms_ll_graph = graph_or_none(step_splitkv_ll)
            sms = min(x for x in (sms_copy, sms_fused, sms_rows, sms_rows_graph, sms_copy_graph, sms_ll, sms_ll_graph)
                      if x is not None)
            assert _lib.device_status() == 0, "a bounded wait of the peer exchange expired"
        total_bytes = shard_bytes * world
        splitkv = {"metric": "kv_read_gbs", "value": total_bytes / (sms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": sms,
                   "config": {"workload": f"split-KV decode B=1 Hq=32 Hkv=8 D=128, {T} KV positions per GPU "
                                          f"(BASELINE config 5 sharding), exchange of (O,LSE) records + merge",
                              "kv_len_total": T * world, "exchange": exchange_note},
                   "per_gpu_gbs": total_bytes / world / (sms * 1e-3) / 1e9,
                   "frac_of_hbm_per_gpu": total_bytes / world / (sms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                   "nccl_all_gather_ms_per_step": nccl_ms, "peer_copy_kernel_ms_per_step": sms_copy,
                   "peer_fused_in_merge_ms_per_step": sms_fused, "peer_row_exchange_one_kernel_ms_per_step": sms_rows,
                   "peer_row_exchange_graph_replay_ms_per_step": sms_rows_graph,
                   "peer_copy_kernel_graph_replay_ms_per_step": sms_copy_graph,
                   "peer_word_exchange_one_kernel_ms_per_step": sms_ll,
                   "peer_word_exchange_graph_replay_ms_per_step": sms_ll_graph,
                   "timing_note": "graph_replay rows: the K steps of a rank captured once into a CUDA graph and replayed "
                                  "once, CUDA events around the replay, max over ranks; the others are enqueued step by "
                                  "step from Python (3 to 1 ctypes calls per step on each of the N processes)",
                   "splitkv_verified": verified, "splitkv_verify_max_err": verify_err,
                   "splitkv_verify": "every rank decodes its range of a shared 4096*N-position cache, exchanges over real "
                                     "peer memory (every form) and compares with its own single-GPU decode (max |diff| "
                                     "of O and LSE over ranks, f32)"}
    del q1, k1, v1, ws
    torch.cuda.empty_cache()

    # ---------------------------------------------------------------- the shapes the reference publishes numbers for
    published = None
    if "published" in legs and n_gpus == 1:
        g = torch.Generator(device="cuda").manual_seed(0x9B)
        rows = []
        ref_cuda = None
        try:
            from oracle import ref_cuda as _rc
            if _rc.available():
                ref_cuda = _rc
        except Exception:
            ref_cuda = None

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
            oh = torch.empty_like(qh)
            t16 = timed(lambda: rt.prefill_bf16(qh, kh, vh, causal=False, out=oh, return_lse=False), 20, 5, dist, torch)
            g16 = graph_ms(lambda: rt.prefill_bf16(qh, kh, vh, causal=False, out=oh, return_lse=False))
            rows.append({"shape": f"flash fwd B{Bp} H{Hp} N{Np} D{Dp} no mask", "ref_ms": ref_ms, "ref_hw": "M4 Max CPU",
                         "ms": t16, "graph_ms": g16, "gflops": 4.0 * Bp * Hp * Np * Np * Dp / t16 / 1e6})
        # Metal decode microbenchmarks: Hq=16 Hkv=2 D=256 f32 on the M4 Max GPU (rustorch-metal/src/kernels.rs:14314-14319),
        # then the reference model's own decode call (LlamaModelCuda::decode_step, batch 1): no published number
        # exists for it, so the reference's CUDA kernel itself is timed here on the same GPU (reference_cuda_us).
        for (hq, hkv, dd, cases) in ((16, 2, 256, ((64, 18.5), (256, 62.0), (1024, 238.0), (4096, 1474.0))),
                                     (32, 8, 128, ((1024, None), (4096, None), (8192, None)))):
            qd1 = torch.randn((1, hq, dd), device="cuda", generator=g).to(torch.bfloat16)
            kc1 = torch.randn((1, hkv, 8192, dd), device="cuda", generator=g).to(torch.bfloat16)
            vc1 = torch.randn((1, hkv, 8192, dd), device="cuda", generator=g).to(torch.bfloat16)
            od1 = torch.empty_like(qd1)
            for kv, ref_us in cases:
                td = timed(lambda: rt.gqa_decode(qd1, kc1, vc1, kv_len=kv, out=od1, return_lse=False), 50, 5, dist, torch)
                gd = graph_ms(lambda: rt.gqa_decode(qd1, kc1, vc1, kv_len=kv, out=od1, return_lse=False))
                row = {"shape": f"GQA decode Hq{hq} Hkv{hkv} D{dd} kv{kv} batch 1", "ref_us": ref_us,
                       "ref_hw": "M4 Max GPU (Metal)" if ref_us else "not published", "us": td * 1e3,
                       "graph_us": None if gd is None else gd * 1e3}
                if ref_cuda is not None:
                    ro = torch.empty_like(qd1[0])
                    rus = graph_ms(lambda: ref_cuda.gqa_decode_online_bf16(qd1[0], kc1[0], vc1[0], kv, out=ro), iters=10)
                    row["reference_cuda_us"] = None if rus is None else rus * 1e3
                    row["reference_cuda_max_abs_diff"] = float((ro.float() - od1[0].float()).abs().max().item())
                rows.append(row)
        # One layer's attention step of the reference's decode loop (cuda_backend.rs:917-987): rope on q and on the new
        # K row, append of K and V, attention.  Four launches there, two here (rope + append fused; the decode is
        # scheduled while the append still runs and waits for it on the device).
        hq, hkv, dd, kv = 32, 8, 128, 4096
        qd1 = torch.randn((1, hq, dd), device="cuda", generator=g).to(torch.bfloat16)
        kc1 = torch.randn((1, hkv, 8192, dd), device="cuda", generator=g).to(torch.bfloat16)
        vc1 = torch.randn((1, hkv, 8192, dd), device="cuda", generator=g).to(torch.bfloat16)
        kn1 = torch.randn((1, hkv, dd), device="cuda", generator=g).to(torch.bfloat16)
        vn1 = torch.randn((1, hkv, dd), device="cuda", generator=g).to(torch.bfloat16)
        od1 = torch.empty_like(qd1)
        inv = rt.rope_inv_freq(dd, 10000.0)

        def layer_step():
            rt.rope_kv_append(qd1, kn1, vn1, kc1, vc1, inv, pos=kv - 1, style="adjacent")
            rt.gqa_decode(qd1, kc1, vc1, kv_len=kv, out=od1, return_lse=False)

        row = {"shape": f"decode step of one layer (rope q, rope k, append, attention) Hq{hq} Hkv{hkv} D{dd} kv{kv} batch 1",
               "ref_hw": "not published", "us": timed(layer_step, 50, 5, dist, torch) * 1e3, "launches": 2}
        gl = graph_ms(layer_step)
        row["graph_us"] = None if gl is None else gl * 1e3
        if ref_cuda is not None:
            ro = torch.empty_like(qd1[0])

            def ref_layer_step():
                ref_cuda.rope_half_split_bf16(qd1[0], inv, kv - 1)
                ref_cuda.rope_half_split_bf16(kn1[0], inv, kv - 1)
                ref_cuda.kv_append_bf16(kc1[0], vc1[0], kn1[0], vn1[0], kv - 1)
                ref_cuda.gqa_decode_online_bf16(qd1[0], kc1[0], vc1[0], kv, out=ro)

            rus = graph_ms(ref_layer_step, iters=10)
            row["reference_cuda_us"] = None if rus is None else rus * 1e3
            row["reference_launches"] = 4
        rows.append(row)
        published = {"rows": rows, "note": "ms/us = one call per step from Python (includes the ctypes enqueue); graph_* = "
                                           "the same call replayed from a CUDA graph; reference_cuda_us = the reference's "
                                           "own gqa_decode_online_bf16 CUDA kernel (llm_kernels.rs:376-458) on this GPU, "
                                           "graph replay"}

    # ---------------------------------------------------------------- CPU baseline (rank 0, N = 1 only)
    cpu = None
    if rank == 0 and n_gpus == 1 and not args.skip_cpu:
        c = cpu_flash_sample(8, 1, 12.0)
        cpu = {"value": c["tflops"], "unit": "TFLOP/s", "cores": c["cores"], "kind": "port", "sample": cpu_sample_text(c),
               "executed_gflops_per_core": c["executed_gflops_per_core"],
               "fma_peak_gflops_per_core": c["fma_peak_gflops_per_core"],
               "tile_gemm_gflops_one_core": c["tile_gemm_gflops_one_core"]}

    if rank == 0:
        out_line = {
            "metric": "attn_prefill_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": n_gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": HEADLINE, "detail": "bf16, per GPU, out bf16 + f32 LSE, all 128 (b,h) slabs per step",
                       "flops_per_step_per_gpu": flops, "flop_convention": "4*D*unmasked (q,k) pairs",
                       "sharding": "independent (b,h) units per rank, no collective",
                       "l2": "Q,K,V,O = 512 MiB per step, larger than the 126 MB L2"},
            "roofline": {"bound": "tensor", "achieved": per_gpu_tflops, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": per_gpu_tflops / peaks["bf16_tflops"], "peak_source": peaks["source"],
                         "peak_kind": "burst (the timed region is tens of ms); see sustained for the seconds-long figure",
                         "traffic": traffic.get("prefill_tc_kernel"),
                         "traffic_source": TRAFFIC_SOURCE["prefill_tc_kernel"]},
            "sustained": sustained, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": args.steps, "clocks": clocks,
            "per_rank_ms": rank_spread(prefill_ranks) if dist is not None else None,
            "published_shapes": published, "backward": backward, "strong": strong,
            "decode_splitkv": splitkv, "decode": decode, "legs": leg_map,
        }
        print(json.dumps(out_line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
