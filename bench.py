#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference] [--workload NAME]

Default workload (the headline): BASELINE config 2 -- flash_attention forward, bf16, MHA,
B=8 H=32 S=4096 D=128, causal; FLOPs = 2*B*H*S^2*D.  One "step" is one forward pass over the
batch.  With N > 1 (torchrun, one rank per GPU) every rank runs its own full-size shard of
(batch x head) units -- the path has no exchange step, so there is no collective in the timed
region -- and `value` is the work of all ranks over the slowest rank's device time.

Prints ONE JSON line.  `--impl reference` times the CPU restatement of the reference's own
CPU path (oracle/) on a bounded sample of the same workload, on rank 0 only.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (kind, params)
    "prefill_fwd_c2": ("fwd", dict(B=8, Hq=32, Hkv=32, S=4096, D=128, dtype="bf16", seed=1)),
    # same kernel and tile shapes as config 2 on a quarter of the batch: the case ncu --set full captures
    "prefill_fwd_profile": ("fwd", dict(B=2, Hq=32, Hkv=32, S=4096, D=128, dtype="bf16", seed=1)),
    "bwd_profile": ("bwd", dict(B=2, Hq=32, Hkv=4, S=8192, D=128, dtype="bf16", seed=2)),
    "decode_profile": ("decode", dict(B=8, Hq=32, Hkv=8, cap=32768, D=128, dtype="bf16", seed=3, lens="uniform")),
    "prefill_fwd_s8192": ("fwd", dict(B=4, Hq=64, Hkv=8, S=8192, D=128, dtype="bf16", seed=2)),
    "fwdbwd_c3": ("bwd", dict(B=4, Hq=64, Hkv=8, S=8192, D=128, dtype="bf16", seed=2)),
    # RoPE on the query tensor of config 3, (B,S,H,D) layout, positions from 0: bytes = read + write of x
    "rope_c3": ("rope", dict(B=4, H=64, S=8192, D=128, dtype="bf16", seed=2)),
    "decode_c4": ("decode", dict(B=64, Hq=32, Hkv=8, cap=32768, D=128, dtype="bf16", seed=3, lens="uniform")),
    "decode_c5": ("decode", dict(B=16, Hq=64, Hkv=1, cap=131072, D=128, dtype="fp16", seed=4, lens="full", std=0.5)),
    # head dimension 256: the one-tile tcgen05 kernel in prefill and in decode mode (profiles/tile_kernel_d256.md)
    "prefill_fwd_d256": ("fwd", dict(B=2, Hq=32, Hkv=8, S=4096, D=256, dtype="bf16", seed=5)),
    "decode_d256": ("decode", dict(B=16, Hq=32, Hkv=8, cap=16384, D=256, dtype="bf16", seed=6, lens="uniform")),
    # fp32 tensors through the tensor cores as TF32 (opt-in), and the same shape on the default exact fp32 kernels
    "prefill_fwd_fp32_tf32": ("fwd", dict(B=2, Hq=32, Hkv=8, S=4096, D=128, dtype="fp32", seed=7, impl="sm100")),
    "prefill_fwd_fp32_exact": ("fwd", dict(B=2, Hq=32, Hkv=8, S=4096, D=128, dtype="fp32", seed=7)),
}
DT = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernel per launch, from the ncu
# captures summarised under profiles/ (taken on a smaller case of the same kernel and scaled by the units).
NCU_TRAFFIC_BYTES = {
    "prefill_fwd_c2": 4 * 254.5e6,        # profiles/fwd_sm100_prefill_bf16_d128.md
    "prefill_fwd_profile": 254.5e6,
    "fwdbwd_c3": 4 * 1136.6e6,            # profiles/bwd_sm100_bf16_d128.md
    "bwd_profile": 1136.6e6,
    "decode_c4": 8 * 855.5e6,             # profiles/decode_group_bf16_d128.md
    "decode_profile": 855.5e6,
    "decode_c5": 1.0830e9,               # profiles/decode_tc_fp16_d128.md (read 1.0741 GB + write 8.9 MB)
}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm=float(d["hbm_gbs"]), tf=float(d["bf16_tflops"]), tf_sus=float(d["bf16_tflops_sustained"]),
                    src="measured")
    return dict(hbm=6650.0, tf=1590.0, tf_sus=1400.0, src="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML every few milliseconds while the timed
    region runs (read-only queries; falls back to one nvidia-smi query if NVML is unavailable)."""

    def __init__(self, gpu_index, period_s=0.004):
        self.idx, self.period = gpu_index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop, self._thr, self._nv = False, None, None

    def _loop(self):
        nv, h = self._nv, self._h
        bits = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown if hasattr(nv, "nvmlClocksEventReasonHwSlowdown")
                else nv.nvmlClocksThrottleReasonHwSlowdown,
                "hw_thermal_slowdown": nv.nvmlClocksThrottleReasonHwThermalSlowdown,
                "sw_thermal_slowdown": nv.nvmlClocksThrottleReasonSwThermalSlowdown,
                "sw_power_cap": nv.nvmlClocksThrottleReasonSwPowerCap}
        while not self._stop:
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for name, bit in bits.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            # NVML enumerates physical GPUs; honour CUDA_VISIBLE_DEVICES when it lists indices
            vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            phys = self.idx
            if vis and all(x.strip().isdigit() for x in vis.split(",")):
                phys = int(vis.split(",")[self.idx])
            self._h = nv.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(self._h, nv.NVML_CLOCK_SM)
            self._nv = nv
            import threading
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()
        except Exception:
            self._nv = None

    def stop(self):
        if self._nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable"], "samples": 0}
        self._stop = True
        self._thr.join(timeout=2)
        sm = sorted(self.samples)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(sm)}


def make_inputs(kind, p, device, pinned_host=False):
    """Seeded synthetic inputs: fp32 randn on the CPU generator in the order q, k, v, (dO), then cast."""
    torch.manual_seed(p["seed"])
    dt, std = DT[p["dtype"]], p.get("std", 1.0)

    def draw(*shape):
        return (torch.randn(*shape, dtype=torch.float32) * std).to(dt)
    if kind == "rope":
        return [draw(p["B"], p["S"], p["H"], p["D"])], None
    if kind in ("fwd", "bwd"):
        host = [draw(p["B"], p["Hq"], p["S"], p["D"]), draw(p["B"], p["Hkv"], p["S"], p["D"]),
                draw(p["B"], p["Hkv"], p["S"], p["D"])]
        if kind == "bwd":
            host.append(draw(p["B"], p["Hq"], p["S"], p["D"]))
        extra = None
    else:
        host = [draw(p["B"], p["Hq"], 1, p["D"])]
        if p["lens"] == "uniform":
            extra = torch.randint(16384, p["cap"] + 1, (p["B"],), dtype=torch.int32)   # upper end inclusive
        else:
            extra = torch.full((p["B"],), p["cap"], dtype=torch.int32)
        # the cache (2 x 4.3 GB for config 4) is drawn on the device from the same seed
        g = torch.Generator(device=device).manual_seed(p["seed"])
        for _ in range(2):
            c = torch.empty((p["B"], p["Hkv"], p["cap"], p["D"]), dtype=dt, device=device)
            c.normal_(0.0, std, generator=g)
            host.append(c)
    if pinned_host:
        host = [t.pin_memory() if not t.is_cuda else t for t in host]
    return host, extra


def work_units(kind, p, lens=None):
    """Algorithmic work of one step on one GPU: FLOPs (prefill/backward) or KV bytes (decode)."""
    if kind == "rope":
        return 2.0 * p["B"] * p["S"] * p["H"] * p["D"] * (2 if p["dtype"] != "fp32" else 4)
    if kind == "fwd":
        return 2.0 * p["B"] * p["Hq"] * p["S"] ** 2 * p["D"]             # causal half of 4*B*H*S^2*D
    if kind == "bwd":
        return 2.5 * 2.0 * p["B"] * p["Hq"] * p["S"] ** 2 * p["D"]
    es = 2 if p["dtype"] != "fp32" else 4
    return float(lens.sum().item()) * p["Hkv"] * p["D"] * es * 2         # K and V rows actually attended


def time_steps(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    t_all0, t_all1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_all0.record()
    for a, b in evs:
        a.record()
        fn()
        b.record()
    t_all1.record()
    torch.cuda.synchronize()
    return t_all0.elapsed_time(t_all1), [a.elapsed_time(b) for a, b in evs]


def run_native(args):
    import torch.distributed as dist
    from stackkernels_b200 import _lib
    from stackkernels_b200 import flash_attention, flash_attention_host, flash_decode
    from stackkernels_b200.launchers import flash_attn_bwd, flash_attn_fwd
    from stackkernels_b200.launchers import flash_decode as core_decode

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()
    peaks = load_peaks()

    def measure(name, steps, warmup, with_e2e):
        kind, p = WORKLOADS[name]
        host, lens = make_inputs(kind, p, dev, pinned_host=with_e2e)
        d = [t.to(dev, non_blocking=True) for t in host]
        lens_d = None if lens is None else lens.to(dev)
        launches = 1
        if kind == "rope":
            from stackkernels_b200.embedding import precompute_freqs, rope_launch
            cos, sin = precompute_freqs(p["D"], p["S"], device=dev)
            fn = lambda: rope_launch(d[0], cos, sin, 0)
        elif kind == "fwd":
            fn = lambda: flash_attn_fwd(d[0], d[1], d[2], is_causal=True, impl=p.get("impl", "auto"))
        elif kind == "bwd":
            o, lse = flash_attn_fwd(d[0], d[1], d[2], is_causal=True)
            fn = lambda: flash_attn_bwd(d[3], d[0], d[1], d[2], o, lse, is_causal=True)
            launches = 3
        else:
            fn = lambda: core_decode(d[0], d[1], d[2], cache_seqlens=lens_d)
            launches = 2
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        sampler = ClockSampler(local)
        sampler.start()
        total_ms, per = time_steps(fn, steps, 0)
        clocks = sampler.stop()
        if world > 1:
            dist.barrier()
            t = torch.tensor([total_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            total_ms = t.item()
        units = work_units(kind, p, lens)
        ms_step = total_ms / steps
        res = dict(kind=kind, p=p, units=units, ms_step=ms_step, ms_kernel=statistics.mean(per), clocks=clocks,
                   launches=launches * steps, e2e=None)
        if with_e2e:
            # end to end through the public API: host (pinned) -> device, compute, result -> host
            def e2e_step():
                if kind == "fwd":
                    # host q, k, v -> chunked H2D / kernel / D2H pipeline -> host O
                    flash_attention_host(host[0], host[1], host[2], out=out_host, causal=True)
                    torch.cuda.current_stream().synchronize()
                    return out_host
                dd = [t.to(dev, non_blocking=True) if not t.is_cuda else t for t in host]
                if kind == "decode":
                    out = flash_decode(dd[0], dd[1], dd[2], cache_seqlens=lens_d)
                else:
                    raise NotImplementedError
                out_host.copy_(out, non_blocking=True)
                torch.cuda.current_stream().synchronize()
                return out_host
            out_host = torch.empty(host[0].shape, dtype=host[0].dtype).pin_memory()
            for _ in range(2):
                e2e_step()
            torch.cuda.synchronize()
            n_e2e = max(3, min(steps, 5))
            if world > 1:
                dist.barrier()
            t0 = time.perf_counter()
            for _ in range(n_e2e):
                e2e_step()
            torch.cuda.synchronize()
            dt_ = time.perf_counter() - t0
            if world > 1:
                t = torch.tensor([dt_], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                dt_ = t.item()
            h2d = sum(t.numel() * t.element_size() for t in host if not t.is_cuda)
            d2h = host[0].numel() * host[0].element_size()
            res["e2e"] = dict(s_step=dt_ / n_e2e, h2d=h2d, d2h=d2h)
        return res

    name = args.workload
    r = measure(name, args.steps, args.warmup, with_e2e=not args.no_e2e)
    kind, p = r["kind"], r["p"]
    is_decode = kind in ("decode", "rope")          # bandwidth-bound workloads report GB/s
    scale = 1e-9 if is_decode else 1e-12
    unit = "GB/s" if is_decode else "TFLOP/s"
    value = world * r["units"] * scale / (r["ms_step"] * 1e-3)
    achieved = r["units"] * scale / (r["ms_kernel"] * 1e-3)
    long_region = r["ms_step"] * args.steps > 1000.0      # seconds-long loops run under the power cap
    peak = peaks["hbm"] if is_decode else (peaks["tf_sus"] if long_region else peaks["tf"])
    line = {
        "metric": {"fwd": "attn_fwd_tflops", "bwd": "attn_bwd_tflops", "decode": "flash_decode_hbm_gbs",
                   "rope": "rope_hbm_gbs"}[kind],
        "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": r["ms_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": p["dtype"], "data": "synthetic",
        "config": {"workload": name, **{k: v for k, v in p.items() if k not in ("seed",)}, "causal": not is_decode,
                   "per_gpu": "one full-size shard per GPU, units = (batch x kv-head group), no collective",
                   "l2": "inputs_exceed_l2"},
        "roofline": {"bound": "hbm" if is_decode else "tensor", "achieved": achieved, "peak": peak, "unit": unit,
                     "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES.get(name),
                     "peak_source": f"{peaks['src']} ({'copy bandwidth' if is_decode else ('bf16 sustained' if long_region else 'bf16 burst')})",
                     "frac_of_burst": None if is_decode else achieved / peaks["tf"],
                     "frac_of_sustained": None if is_decode else achieved / peaks["tf_sus"],
                     # nominal B200 figures, for context: 8 TB/s HBM3e, 2250 TFLOP/s dense bf16
                     "frac_of_nominal": achieved / (8000.0 if is_decode else 2250.0)},
        "clocks": r["clocks"], "gpu_launches": r["launches"],
    }
    if r["e2e"] is not None:
        line["e2e"] = {"value": world * r["units"] * scale / r["e2e"]["s_step"], "unit": unit,
                       "h2d_bytes_per_step": r["e2e"]["h2d"], "d2h_bytes_per_step": r["e2e"]["d2h"]}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(name, limit_s=args.cpu_seconds)
    if world == 1 and not args.no_extras:
        extras = {}
        for en, st in (("prefill_fwd_s8192", 5), ("fwdbwd_c3", 3), ("decode_c4", 10), ("decode_c5", 10), ("rope_c3", 10)):
            if en == name:
                continue
            torch.cuda.empty_cache()
            e = measure(en, st, 3, with_e2e=False)
            dec = e["kind"] in ("decode", "rope")
            sc = 1e-9 if dec else 1e-12
            a = e["units"] * sc / (e["ms_step"] * 1e-3)
            pk = peaks["hbm"] if dec else peaks["tf"]
            extras[en] = {"value": a, "unit": "GB/s" if dec else "TFLOP/s", "ms_per_step": e["ms_step"],
                          "frac_of_measured_peak": a / pk}
        line["extras"] = extras
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def cpu_baseline(name, limit_s=15.0):
    """The CPU restatement of the reference's CPU path, timed on a bounded sample of the workload."""
    from oracle import attention_oracle as orc
    kind, p = WORKLOADS[name]
    torch.manual_seed(p["seed"])
    dt = DT[p["dtype"]]
    # all host cores, whatever the launcher put into OMP_NUM_THREADS (torchrun sets it to 1 per process)
    torch.set_num_threads(max(1, len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)))
    threads = torch.get_num_threads()
    done_units, t_used, n = 0.0, 0.0, 0
    if kind in ("fwd", "bwd"):
        g = p["Hq"] // p["Hkv"]
        S, D = p["S"], p["D"]
        per_slice = (2.0 if kind == "fwd" else 5.0) * g * S * S * D
        while t_used < limit_s and n < p["B"] * p["Hkv"]:
            q = torch.randn(1, g, S, D).to(dt)
            k, v = torch.randn(1, 1, S, D).to(dt), torch.randn(1, 1, S, D).to(dt)
            t0 = time.perf_counter()
            if kind == "fwd":
                orc.attention_forward(q, k, v, causal=True)
            else:
                orc.attention_backward(torch.randn(1, g, S, D).to(dt), q, k, v, causal=True)
            t_used += time.perf_counter() - t0
            done_units += per_slice
            n += 1
        sample = f"{n} of {p['B'] * p['Hkv']} (batch, kv-head) units of {name}, one call each"
        scale, unit = 1e-12, "TFLOP/s"
    else:
        es = 2 if p["dtype"] != "fp32" else 4
        ln = p["cap"] if p["lens"] == "full" else (16384 + p["cap"]) // 2
        while t_used < limit_s and n < p["B"]:
            q = torch.randn(1, p["Hq"], 1, p["D"]).to(dt)
            k, v = torch.randn(1, p["Hkv"], ln, p["D"]).to(dt), torch.randn(1, p["Hkv"], ln, p["D"]).to(dt)
            t0 = time.perf_counter()
            orc.attention_forward(q, k, v)
            t_used += time.perf_counter() - t0
            done_units += ln * p["Hkv"] * p["D"] * es * 2
            n += 1
        sample = f"{n} of {p['B']} sequences of {name} at {ln} cached tokens"
        scale, unit = 1e-9, "GB/s"
    return {"value": done_units * scale / t_used, "unit": unit, "cores": threads, "kind": "port", "sample": sample,
            "seconds": t_used}


def run_reference(args):
    """Reference arm: the reference's CPU implementation of the path (its Python source cannot travel
    to the GPU box, so the pinned restatement in oracle/ is what runs), all host threads, rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    name = args.workload
    kind, p = WORKLOADS[name]
    per_step = max(2.0, min(20.0, 120.0 / max(1, args.steps + args.warmup)))
    for _ in range(args.warmup):
        cpu_baseline(name, limit_s=per_step / 4)
    vals, secs = [], 0.0
    for _ in range(args.steps):
        r = cpu_baseline(name, limit_s=per_step)
        vals.append(r["value"])
        secs += r["seconds"]
    v = statistics.mean(vals)
    is_decode = kind == "decode"
    line = {
        "impl": "reference",
        "metric": {"fwd": "attn_fwd_tflops", "bwd": "attn_bwd_tflops", "decode": "flash_decode_hbm_gbs"}[kind],
        "value": v, "unit": r["unit"], "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * secs / max(1, args.steps), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": p["dtype"], "data": "synthetic",
        "config": {"workload": name, **{k: vv for k, vv in p.items() if k != "seed"}, "causal": not is_decode},
        "cpu_baseline": {"value": v, "unit": r["unit"], "cores": r["cores"], "kind": "port",
                         "sample": r["sample"] + f" per step ({per_step:.0f} s per step)"},
        "e2e": {"value": v, "unit": r["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default="prefill_fwd_c2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary workloads reported under 'extras'")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "native":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
