"""Benchmark of the HiP attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload (``prefill_128k``, benchmark configuration 2): one Llama-3.1-8B-shaped layer, bf16, the last
32768 queries against 131072 keys, 32 / 8 heads, head dim 128, three scan stages
(chunks 256 / 32 / 8 keeping 32768 / 8192 / 2048 tokens), sink 256, window 1024.  A step is one
``hip_attention_12`` call (mask estimation + block-sparse attention).  With N > 1 the KV heads are
split over the ranks (strong scaling) and every scan stage ends in a MAX all-reduce.

Prints one JSON line (rank 0).  ``value`` is queries per second with inputs resident in HBM,
``e2e`` the same through the public call with pinned host buffers copied in and the output copied
out every step, ``roofline`` describes the scan kernel (the dominant one), ``cpu_baseline`` times the
CPU oracle on a bounded sample of the same workload.  ``--impl reference`` times the CPU restatement
of the reference operator on the host cores (the reference itself is Triton code for GPUs; its
checkout does not travel to the benchmark box).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # benchmark configuration 2
    "prefill_128k": dict(kind="prefill", B=1, TQ=32768, T=131072, H=32, HKV=8, D=128, dtype="bf16", theta=5e5,
                         bq=64, chunks=[256, 32, 8], keep=[32768, 8192, 2048], strides=[4, 4, 1], sink=256, sw=1024,
                         heavy=0.01, seed=1235),
    # benchmark configuration 1 (fp32, CPU-runnable)
    "prefill_4k_fp32": dict(kind="prefill", B=1, TQ=4096, T=4096, H=8, HKV=2, D=64, dtype="fp32", theta=1e4,
                            bq=64, chunks=[32, 8], keep=[1024, 512], strides=[4, 1], sink=64, sw=256, heavy=0.0,
                            seed=1234),
    # benchmark configuration 3: batched decode over a paged cache, mask refreshed every 8 steps
    "decode_128k": dict(kind="decode", B=32, TQ=1, T=131072, H=32, HKV=8, D=128, dtype="bf16", theta=5e5,
                        bq=64, chunks=[256, 32, 8], keep=[32768, 8192, 2048], strides=[4, 4, 1], sink=256, sw=1024,
                        heavy=0.01, seed=1236, page=64, refresh=8),
    # benchmark configuration 4: million-token decode in 8 logical sequence shards
    "decode_1m": dict(kind="decode_sharded", B=1, TQ=1, T=1048576, H=32, HKV=8, D=128, dtype="bf16", theta=5e5,
                      bq=64, chunks=[256, 32, 8], keep=[32768, 8192, 512], strides=[4, 4, 1], sink=256, sw=1024,
                      heavy=0.0, seed=1237, page=64, shards=8, needles=64),
}
_DT = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}
# dram__bytes_read.sum + dram__bytes_write.sum per scan launch (mean of the three stages), from the ncu capture
# summarised in profiles/prefill128k_dram_traffic.md; keyed by (workload, GPUs, queries)
NCU_DRAM_BYTES_PER_SCAN_LAUNCH = {("prefill_128k", 1, 32768): (563160320 + 582162688 + 357693696) / 3}


# ----------------------------------------------------------------------------------------------
# synthetic inputs
# ----------------------------------------------------------------------------------------------
def rope(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    """Rotate-half RoPE; x [B, T, H, D] fp32, pos [T] or [B, T]."""
    D = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, device=x.device, dtype=torch.float64) / D))
    ang = pos.to(torch.float64)[..., None] * inv
    ang = torch.cat([ang, ang], -1)
    cos, sin = ang.cos().float(), ang.sin().float()
    if cos.ndim == 2:
        cos, sin = cos[None], sin[None]
    cos, sin = cos[:, :, None, :], sin[:, :, None, :]
    xr = torch.cat([-x[..., D // 2:], x[..., : D // 2]], -1)
    return x * cos + xr * sin


def make_qkv(w: dict, device, kv_heads: slice = None, step: int = 0):
    """Seeded synthetic q, k, v of the workload's shape and value distribution (N(0,1), RoPE, 1 % heavy
    keys scaled x4; q carries the softmax scale).  ``kv_heads`` keeps only one rank's heads."""
    g = torch.Generator(device=device)
    g.manual_seed(w["seed"])
    B, TQ, T, H, HKV, D = w["B"], w["TQ"], w["T"], w["H"], w["HKV"], w["D"]
    dt = _DT[w["dtype"]]
    k = torch.randn((B, T, HKV, D), generator=g, device=device, dtype=torch.float32)
    k = rope(k, torch.arange(T, device=device), w["theta"])
    if w["heavy"] > 0:
        hh = torch.rand((B, T), generator=g, device=device) < w["heavy"]
        k = torch.where(hh[:, :, None, None], k * 4.0, k)
    k = k.to(dt)
    v = torch.randn((B, T, HKV, D), generator=g, device=device, dtype=torch.float32).to(dt)
    gq = torch.Generator(device=device)
    gq.manual_seed(w["seed"] * 1000 + step)
    q = torch.randn((B, TQ, H, D), generator=gq, device=device, dtype=torch.float32)
    q = rope(q, torch.arange(T - TQ, T, device=device), w["theta"]) * (D ** -0.5)
    q = q.to(dt)
    if kv_heads is not None:
        gq_ = H // HKV
        q = q[:, :, kv_heads.start * gq_: kv_heads.stop * gq_].contiguous()
        k = k[:, :, kv_heads].contiguous()
        v = v[:, :, kv_heads].contiguous()
    return q, k, v


def make_args(w: dict, **kw):
    from hip_attention_b200 import HiPAttentionArgs, ScanStage
    stages = []
    for i, c in enumerate(w["chunks"]):
        stages.append(ScanStage(stage_block_size_q=w["bq"], stage_block_stride_q=w["strides"][i], stage_chunk_size=c,
                                stage_k=None if i == 0 else w["keep"][i - 1], stage_stride=1))
    return HiPAttentionArgs(sink_token_size=w["sink"], sliding_window_size=w["sw"], second_stage_k=w["keep"][-1],
                            stages=stages, block_sparse_block_size_q=w["bq"], require_cache_statistics=False, **kw)


def oracle_config(w: dict):
    from oracle import hip_oracle as O
    st = [O.OracleStage(w["bq"], w["strides"][i], c, None if i == 0 else w["keep"][i - 1]) for i, c in enumerate(w["chunks"])]
    return O.OracleConfig(stages=st, sink=w["sink"], sw=w["sw"], second_stage_k=w["keep"][-1])


def scan_bytes(w: dict, heads: int) -> float:
    """Algorithmic bytes of the scan stages of one call: active chunks x (log2(chunk) + 1) rounds x 2 key
    rows x D x element size, summed over (batch, query block, head, stage)."""
    eb = 4 if w["dtype"] == "fp32" else 2
    B, TQ, T, D, bq = w["B"], w["TQ"], w["T"], w["D"], w["bq"]
    c0 = w["chunks"][0]
    n0 = -(-max(0, T - w["sink"] - w["sw"]) // c0)
    sw_r = max(0, w["sw"] - c0)
    total = 0.0
    for d in range(-(-TQ // bq)):
        pmin = d * bq + T - TQ
        pt = max(pmin - sw_r, 0)
        act = min(n0, max(0, (pt - w["sink"]) // c0 + 1)) if pt >= w["sink"] else 0
        n = n0
        for i, c in enumerate(w["chunks"]):
            total += act * (int(math.log2(c)) + 1) * 2 * D * eb
            if i + 1 < len(w["chunks"]):
                keep = min(w["keep"][i] // c, n)
                split = c // w["chunks"][i + 1]
                act = min(act, keep) * split
                n = keep * split
    return total * B * heads


def scan_flops(w: dict, heads: int) -> float:
    """Tensor-core FLOPs of the scan stages: every gathered key row is multiplied with the pooled query rows
    of its (query block, head): 2 * rows * D per key row."""
    eb = 4 if w["dtype"] == "fp32" else 2
    total = 0.0
    for i, c in enumerate(w["chunks"]):
        w1 = dict(w, chunks=w["chunks"][:i + 1], keep=w["keep"][:max(i, 1)])
        w0 = dict(w, chunks=w["chunks"][:i], keep=w["keep"][:max(i - 1, 1)]) if i else None
        stage_bytes = scan_bytes(w1, heads) - (scan_bytes(w0, heads) if w0 else 0.0)
        rows = w["bq"] // w["strides"][i]
        total += stage_bytes / (w["D"] * eb) * 2.0 * rows * w["D"]
    return total


def attention_flops(w: dict, heads: int) -> float:
    return 4.0 * w["D"] * w["B"] * heads * w["TQ"] * (w["keep"][-1] + w["sink"] + w["sw"])


# ----------------------------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            f = [x.strip() for x in s.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for nme, val in zip(names, f[2:6]):
                if val == "Active":
                    reasons.add(nme)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ----------------------------------------------------------------------------------------------
# CPU arm (oracle = restatement of the reference operator)
# ----------------------------------------------------------------------------------------------
def cpu_sample(w: dict, n_blocks: int, block0: int = None):
    """Run the CPU oracle on ``n_blocks`` query blocks of the workload; returns (seconds, tokens)."""
    from oracle import hip_oracle as O
    q, k, v = make_qkv(w, "cpu")
    cfg = oracle_config(w)
    bq, TQ, T = w["bq"], w["TQ"], w["T"]
    nb = -(-TQ // bq)
    b0 = (nb - n_blocks) if block0 is None else block0  # the last blocks see the longest context
    r0, r1 = b0 * bq, min(TQ, (b0 + n_blocks) * bq)
    qs = q[:, r0:r1].contiguous()
    pos = (torch.arange(r0, r1) + (T - TQ))[None].expand(w["B"], -1).contiguous()
    t0 = time.perf_counter()
    O.hip_attention_oracle(qs, k, v, pos, cfg, out_dtype=torch.float32)
    return time.perf_counter() - t0, (r1 - r0) * w["B"]


def run_reference_arm(a, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    secs = []
    for i in range(a.warmup + a.steps):
        dt, toks = cpu_sample(w, 1)
        if i >= a.warmup:
            secs.append(dt)
    ms = 1e3 * float(np.mean(secs))
    val = toks / (ms / 1e3)
    sample = f"1 query block ({toks} queries, the last of {w['TQ']}) per step against all {w['T']} keys"
    line = {"impl": "reference", "metric": "hip_prefill_tokens_per_s", "value": val, "unit": "tokens/s", "n_gpus": a.gpus,
            "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": {"workload": a.workload, **{k_: w[k_] for k_ in ("B", "TQ", "T", "H", "HKV", "D")}},
            "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="prefill_128k", choices=list(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--tq", type=int, default=0, help="profiling aid: shrink the number of queries (not a bench value)")
    ap.add_argument("--batch", type=int, default=0, help="profiling aid: shrink the batch (not a bench value)")
    ap.add_argument("--cpu-blocks", type=int, default=6, help="query blocks of the CPU baseline sample")
    a = ap.parse_args()
    w = dict(WORKLOADS[a.workload])
    if a.tq:
        w["TQ"] = a.tq
    if a.batch:
        w["B"] = a.batch
    if a.impl == "reference":
        return run_reference_arm(a, w)
    if w["kind"] != "prefill":
        import bench_decode
        return bench_decode.run(a, w)

    import torch.distributed as dist
    from hip_attention_b200 import PhaseTimer, hip_attention_impl, read_status
    from hip_attention_b200.sharded import kv_head_slice, make_score_reduce

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != a.gpus:
        raise SystemExit(f"--gpus {a.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    hs, kvs = kv_head_slice(rank, world, w["H"], w["HKV"])
    q, k, v = make_qkv(w, dev, kvs)
    args = make_args(w)
    reduce = make_score_reduce()
    heads_local = hs.stop - hs.start

    def step(timer=None):
        return hip_attention_impl(q, k, v, args, score_reduce=reduce, timer=timer)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def check_status(where: str):
        # a kernel that gave up on a bounded on-chip wait, or clamped a bad index, says so in the device status word:
        # a number measured on such a run is not a measurement
        st = read_status(dev)
        if st != 0:
            raise SystemExit(f"bench.py: device status word {st:#x} after {where}; the run is invalid")

    read_status(dev)
    for _ in range(max(a.warmup, 3)):
        out, md = step()
    barrier()
    check_status("the warm-up steps")

    # ---- device-resident timing -------------------------------------------------------------
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    timers = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(a.steps):
        t = PhaseTimer()
        out, md = step(t)
        timers.append(t)
    e1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    check_status("the timed steps")
    ms_total = e0.elapsed_time(e1)
    tms = torch.tensor([ms_total], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    ms_step = float(tms.item()) / a.steps
    phases = {}
    for t in timers:
        for name, val in t.milliseconds().items():
            phases[name] = phases.get(name, 0.0) + val / a.steps
    scan_ms = sum(vv for kk, vv in phases.items() if kk.startswith("scan"))
    n_scan = sum(1 for kk in phases if kk.startswith("scan"))

    # ---- end to end: pinned host inputs in, output back, every step ---------------------------
    # Three streams (copy in, compute, copy out) and two sets of device buffers: the host-to-device
    # copy of step i + 1 and the device-to-host copy of step i - 1 overlap the kernels of step i.
    hq, hk, hv = (x.cpu().pin_memory() for x in (q, k, v))
    houts = [torch.empty(out.shape, dtype=out.dtype).pin_memory() for _ in range(2)]
    dbuf = [tuple(torch.empty_like(x) for x in (q, k, v)) for _ in range(2)]
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    s_main = torch.cuda.current_stream(dev)

    def e2e_run(n):
        ev_in = [None, None]      # inputs of buffer set j are on the device
        ev_free = [None, None]    # kernels that read buffer set j are done
        ev_out = [None, None]     # result j has been copied out
        keep = []
        for i in range(n):
            j = i & 1
            with torch.cuda.stream(s_in):
                if ev_free[j] is not None:
                    s_in.wait_event(ev_free[j])
                # q and k first: the estimator starts on them while v is still on its way
                dbuf[j][0].copy_(hq, non_blocking=True)
                dbuf[j][1].copy_(hk, non_blocking=True)
                ev_in[j] = torch.cuda.Event()
                ev_in[j].record(s_in)
                dbuf[j][2].copy_(hv, non_blocking=True)
                ev_v = torch.cuda.Event()
                ev_v.record(s_in)
            s_main.wait_event(ev_in[j])
            o, _ = hip_attention_impl(*dbuf[j], args, score_reduce=reduce, v_ready=ev_v)
            ev_free[j] = torch.cuda.Event()
            ev_free[j].record(s_main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_free[j])
                if ev_out[j] is not None:
                    s_out.wait_event(ev_out[j])
                houts[j].copy_(o, non_blocking=True)
                o.record_stream(s_out)
                ev_out[j] = torch.cuda.Event()
                ev_out[j].record(s_out)
            keep.append(o)
        s_main.wait_stream(s_in)
        s_main.wait_stream(s_out)

    e2e_run(2)
    barrier()
    e0.record()
    e2e_run(a.steps)
    e1.record()
    barrier()
    check_status("the end-to-end steps")
    tms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    e2e_ms = float(tms.item()) / a.steps
    h2d = sum(x.numel() * x.element_size() for x in (hq, hk, hv)) * world
    d2h = houts[0].numel() * houts[0].element_size() * world

    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except OSError:
            pass
        peak, peak_src = (peaks["hbm_gbs"], "measured") if "hbm_gbs" in peaks else (6650.0, "fallback")
        sb = scan_bytes(w, heads_local)
        achieved = sb / 1e9 / (scan_ms / 1e3) if scan_ms > 0 else None
        tokens = w["B"] * w["TQ"]
        line = {
            "metric": "hip_prefill_tokens_per_s", "value": tokens / (ms_step / 1e3), "unit": "tokens/s",
            "n_gpus": world, "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": {"workload": a.workload, **{k_: w[k_] for k_ in ("B", "TQ", "T", "H", "HKV", "D")},
                       "stages": {"chunk": w["chunks"], "keep": w["keep"], "stride_q": w["strides"]},
                       "sink": w["sink"], "window": w["sw"], "parallelism": f"kv-head x{world}",
                       "l2": "inputs (q 268 MB, k 268 MB, v 268 MB at N=1) exceed the 126 MB L2"},
            "clocks": clocks,
            "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": (4 + len(w["chunks"]) + 3 * (len(w["chunks"]) - 1)) * a.steps,
            "phases_ms": {k_: round(v_, 4) for k_, v_ in phases.items() if k_ != "start"},
            # `algorithmic` counts the key rows the rounds of the scan gather; in prefill nearly all of them are L2 hits
            # (one KV head's keys, 33.5 MB, are swept by all its query blocks), so `achieved` can exceed the HBM
            # copy peak: `traffic` (measured DRAM bytes per launch) is the part that reaches HBM.  The tensor-core
            # side of the same launches is given beside it.
            "roofline": {"kernel": "scan_stage_tcgen05_kernel", "bound": "hbm", "achieved": achieved, "peak": peak,
                         "peak_source": peak_src, "unit": "GB/s", "frac": achieved / peak if achieved else None,
                         "traffic": NCU_DRAM_BYTES_PER_SCAN_LAUNCH.get((a.workload, world, w["TQ"])),
                         "algorithmic_bytes_per_launch": sb / max(1, n_scan),
                         "launch_ms": scan_ms / max(1, n_scan),
                         "served_by": "L2 (DRAM traffic per launch is `traffic`, about 1.3 % of the gathered bytes)",
                         "tensor": {"achieved": scan_flops(w, heads_local) / 1e12 / (scan_ms / 1e3) if scan_ms > 0 else None,
                                    "peak": peaks.get("bf16_tflops"), "unit": "TFLOP/s",
                                    "frac": scan_flops(w, heads_local) / 1e12 / (scan_ms / 1e3) / peaks["bf16_tflops"]
                                    if scan_ms > 0 and "bf16_tflops" in peaks else None},
                         "note": "algorithmic = key-row gathers issued by the three scan launches; achieved = their bytes / "
                                 "their summed CUDA-event time; a fraction above 1 means the gathers are served from L2, "
                                 "not that work is skipped (tests compare every stage's output with the strict kernel)"},
            "attention_roofline": {"kernel": "bsa_tcgen05_ws_kernel", "bound": "tensor",
                                   "achieved": attention_flops(w, heads_local) / 1e12 / (phases.get("attention", 0) / 1e3)
                                   if phases.get("attention") else None,
                                   "peak": peaks.get("bf16_tflops"), "unit": "TFLOP/s",
                                   "frac": (attention_flops(w, heads_local) / 1e12 / (phases.get("attention", 0) / 1e3)) /
                                   peaks["bf16_tflops"] if phases.get("attention") and "bf16_tflops" in peaks else None,
                                   "flops_per_launch": attention_flops(w, heads_local), "launch_ms": phases.get("attention")},
        }
        if world == 1 and not a.no_cpu_baseline:
            cores = len(os.sched_getaffinity(0))
            torch.set_num_threads(cores)
            dt, toks = cpu_sample(w, a.cpu_blocks)
            line["cpu_baseline"] = {"value": toks / dt, "unit": "tokens/s", "cores": cores, "kind": "port",
                                    "sample": f"the last {a.cpu_blocks} query blocks ({toks} queries) against all "
                                              f"{w['T']} keys, {dt:.1f} s"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
