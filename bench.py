"""Benchmark of the HiP attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload (``prefill_128k``, benchmark configuration 2): one Llama-3.1-8B-shaped layer, bf16, the last
32768 queries against 131072 keys, 32 / 8 heads, head dim 128, three scan stages
(chunks 256 / 32 / 8 keeping 32768 / 8192 / 2048 tokens), sink 256, window 1024.  A step is one
``hip_attention_12`` call (mask estimation + block-sparse attention).  With N > 1 the KV heads are
split over the ranks (strong scaling) and every scan stage ends in a MAX all-reduce.

Prints one JSON line (rank 0).  ``value`` is queries per second with inputs resident in HBM,
``e2e`` the same through the public call with pinned host buffers copied in and the output copied
out every step, ``roofline`` describes the dominant kernel, ``cpu_baseline`` times the CPU oracle on a
bounded sample of the same workload and ``parity`` compares that sample's mask and output with what the
GPU produced for the same query blocks (a mismatch ends the run with a non-zero exit code).
``mask_sha256`` hashes the mask of the first head: all heads share the mask, so the value must not
depend on the number of GPUs.  The default run also carries the decode workloads as sub-records:
``decode`` (configuration 3, one GPU) and ``decode_1m`` (configuration 4, sequence shards over the N ranks),
and, on one GPU, ``triton_reference``: the unmodified reference operator from ``baseline/_ref`` running its
Triton kernels on the same device and inputs.  ``--impl reference`` times the CPU restatement of the
reference operator on the host cores.
"""
from __future__ import annotations

import argparse
import hashlib
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
    # benchmark configuration 5: large-GQA prefill, query blocks of 128 rows, 64 / 8 heads
    "prefill_256k_gqa": dict(kind="prefill", B=2, TQ=262144, T=262144, H=64, HKV=8, D=128, dtype="bf16", theta=1e6,
                             bq=128, chunks=[256, 32, 8], keep=[65536, 16384, 4096], strides=[4, 4, 1], sink=256, sw=2048,
                             heavy=0.01, seed=1238),
}
_DT = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}
# dram__bytes_read.sum + dram__bytes_write.sum per scan launch (mean of the three stages) from one ncu capture of
# this command; a capture is valid for the (workload, GPUs, queries) it was taken on only, hence the key
NCU_DRAM_BYTES_PER_SCAN_LAUNCH = {("prefill_128k", 1, 32768): (563160320 + 582162688 + 357693696) / 3}
NCU_TRAFFIC_SOURCE = "ncu capture (dram__bytes_read.sum + dram__bytes_write.sum), prefill_128k, 1 GPU, 32768 queries only"


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


def scan_bytes(w: dict, heads: int, fetched: bool = False) -> float:
    """Algorithmic bytes of the scan stages of one call: active chunks x (log2(chunk) + 1) rounds x 2 key
    rows x D x element size, summed over (batch, query block, head, stage).  ``fetched``: the rows the kernels
    actually gather -- a candidate that repeats the previous round's winner is not fetched again, which removes
    three of the 2 (log2(chunk) + 1) rows of a chunk."""
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
            rows = (int(math.log2(c)) + 1) * 2
            if fetched:
                rows -= 3 if c >= 4 else (2 if c >= 2 else 0)
            total += act * rows * D * eb
            if i + 1 < len(w["chunks"]):
                keep = min(w["keep"][i] // c, n)
                split = c // w["chunks"][i + 1]
                act = min(act, keep) * split
                n = keep * split
    return total * B * heads


def scan_flops(w: dict, heads: int, fetched: bool = False) -> float:
    """Tensor-core FLOPs of the scan stages: every gathered key row is multiplied with the pooled query rows
    of its (query block, head): 2 * rows * D per key row."""
    eb = 4 if w["dtype"] == "fp32" else 2
    total = 0.0
    for i, c in enumerate(w["chunks"]):
        w1 = dict(w, chunks=w["chunks"][:i + 1], keep=w["keep"][:max(i, 1)])
        w0 = dict(w, chunks=w["chunks"][:i], keep=w["keep"][:max(i - 1, 1)]) if i else None
        stage_bytes = scan_bytes(w1, heads, fetched) - (scan_bytes(w0, heads, fetched) if w0 else 0.0)
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
        self.index, self.samples, self.proc, self.t0 = index, [], None, 0.0

    def mark(self):
        """Samples received before this call are dropped: nvidia-smi is started early because it needs a moment to
        deliver its first line, and only what it reports from here on describes the GPU under load."""
        self.t0 = time.perf_counter()

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.perf_counter(), line.strip()))

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.03)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for when, s in self.samples:
            if when < self.t0:
                continue
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
def cpu_sample(w: dict, n_blocks: int, qkv=None):
    """Run the CPU oracle on the last ``n_blocks`` query blocks of the workload (they see the longest context).
    ``qkv`` = CPU tensors to use (default: drawn here).  Returns (seconds, tokens, output, mask, first row)."""
    from oracle import hip_oracle as O
    q, k, v = qkv if qkv is not None else make_qkv(w, "cpu")
    cfg = oracle_config(w)
    bq, TQ, T = w["bq"], w["TQ"], w["T"]
    nb = -(-TQ // bq)
    b0 = max(0, nb - n_blocks)
    r0, r1 = b0 * bq, TQ
    qs = q[:, r0:r1].contiguous()
    pos = (torch.arange(r0, r1) + (T - TQ))[None].expand(w["B"], -1).contiguous()
    t0 = time.perf_counter()
    out, m = O.hip_attention_oracle(qs, k, v, pos, cfg, out_dtype=torch.float32)
    return time.perf_counter() - t0, (r1 - r0) * w["B"], out, m, r0


def config_of(a, w: dict, world: int) -> dict:
    """The ``config`` object of the JSON line; both arms print the same one."""
    if w["kind"] != "prefill":
        cfg = {"workload": a.workload, **{k_: w[k_] for k_ in ("B", "TQ", "T", "H", "HKV", "D")}, "page": w["page"]}
        if w["kind"] == "decode":
            cfg["mask_refresh_every"] = w["refresh"]
        else:
            cfg.update(logical_shards=w["shards"], per_shard_top_k=w["keep"][-1])
        return cfg
    mb = lambda n: round(n * (4 if w["dtype"] == "fp32" else 2) / 1e6)
    return {"workload": a.workload, **{k_: w[k_] for k_ in ("B", "TQ", "T", "H", "HKV", "D")},
            "block_size_q": w["bq"], "stages": {"chunk": w["chunks"], "keep": w["keep"], "stride_q": w["strides"]},
            "sink": w["sink"], "window": w["sw"], "parallelism": f"kv-head x{world}",
            "l2": f"inputs (q {mb(w['B'] * w['TQ'] * w['H'] * w['D'])} MB, k and v {mb(w['B'] * w['T'] * w['HKV'] * w['D'])} MB "
                  f"each over all GPUs) exceed the 126 MB L2"}


def run_reference_arm(a, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    if w["kind"] != "prefill":
        import bench_decode
        return bench_decode.run_reference_arm(a, w, cores)
    secs = []
    qkv = make_qkv(w, "cpu")
    for i in range(a.warmup + a.steps):
        dt, toks, _, _, _ = cpu_sample(w, 1, qkv)
        if i >= a.warmup:
            secs.append(dt)
    ms = 1e3 * float(np.mean(secs))
    val = toks / (ms / 1e3)
    sample = f"1 query block ({toks} queries, the last of {w['TQ']}) per step against all {w['T']} keys"
    line = {"impl": "reference", "metric": "hip_prefill_tokens_per_s", "value": val, "unit": "tokens/s", "n_gpus": a.gpus,
            "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic", "config": config_of(a, w, a.gpus),
            "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# the reference's own Triton kernels on the same GPU (from baseline/_ref; nothing of this project on that path)
# ----------------------------------------------------------------------------------------------
def triton_reference_leg(w: dict, ours, steps: int = 10) -> dict:
    """Times the unmodified reference operator on the workload (warm-up 3, then ``steps`` timed calls, CUDA events,
    the pattern of the reference's own benchmark, tests/v1_2/test_attention_extend.py:300-320) and compares its
    mask and output with ``ours`` = (out, metadata) of this project on the same tensors."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import reference_loader as R
        if not R.available():
            return {"unavailable": "no copy of the reference under baseline/_ref"}
        op, Args, ScanStage = R.load_reference()
        import triton
        q, k, v = make_qkv(w, "cuda")
        ra = R.reference_args(Args, ScanStage, bq=w["bq"], strides=w["strides"], chunks=w["chunks"], keep=w["keep"],
                              sink=w["sink"], sw=w["sw"])
        for _ in range(3):
            o_ref, md_ref = op(q, k, v, args=ra)
        torch.cuda.synchronize()
        ts = []
        for _ in range(steps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            o_ref, md_ref = op(q, k, v, args=ra)
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ms = float(np.median(ts))
        rec = {"ms_per_step": ms, "best_ms": float(min(ts)), "tokens_per_s": w["B"] * w["TQ"] / (ms / 1e3), "steps": steps,
               "triton": triton.__version__, "torch": torch.__version__, "autotune": "off (HIP_DISABLE_AUTOTUNE=1)"}
        if ours is not None:
            rec["agreement"] = mask_agreement(ours[1], md_ref, ours[0], o_ref)
        return rec
    except Exception as e:  # noqa: BLE001 - whatever stops the reference is reported, not raised
        return {"unavailable": f"{type(e).__name__}: {str(e)[:300]}"}


def mask_agreement(md, md_ref, out, out_ref) -> dict:
    """How far two runs of the operator agree: share of (head, query block) rows whose selected block set is identical,
    overlap of the sets over all rows, and the output difference.  The reference orders equal scores arbitrarily and
    accumulates its dot products in tensor-core order, so single blocks at the selection threshold may differ."""
    a, b = md.indices, md_ref.indices
    ka, kb = md.ks, md_ref.ks
    n = min(a.shape[-1], b.shape[-1])
    ar = torch.arange(n, device=a.device)
    va, vb = ar[None, None, :] < ka[..., None], ar[None, None, :] < kb[..., None]
    sa = torch.where(va, a[..., :n], torch.full_like(a[..., :n], -1))
    sb = torch.where(vb, b[..., :n], torch.full_like(b[..., :n], -1))
    rows_equal = (sa == sb).all(-1)
    # both lists are ascending: count common entries through a merged sort
    cat = torch.cat([torch.where(va, a[..., :n], torch.full_like(a[..., :n], -1)),
                     torch.where(vb, b[..., :n], torch.full_like(b[..., :n], -2))], -1).sort(-1).values
    common = ((cat[..., 1:] == cat[..., :-1]) & (cat[..., 1:] >= 0)).sum()
    total = torch.maximum(ka, kb).sum().clamp(min=1)
    d = (out.float() - out_ref.float()).abs()
    return {"rows_identical": float(rows_equal.float().mean()), "block_overlap": float(common / total),
            "out_max_abs": float(d.max()), "out_mean_abs": float(d.mean())}


def gpu_numa_cpus(index: int):
    """CPUs of the NUMA node the GPU hangs off (sysfs), or None: pinned staging buffers are then allocated and
    first touched by a thread running there."""
    try:
        p = torch.cuda.get_device_properties(index)
        path = f"/sys/bus/pci/devices/{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0/numa_node"
        node = int(open(path).read())
        if node < 0:
            return None
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            if "-" in part:
                lo, hi = part.split("-")
                cpus.update(range(int(lo), int(hi) + 1))
            elif part:
                cpus.add(int(part))
        cpus &= os.sched_getaffinity(0)
        return cpus or None
    except (OSError, ValueError, AttributeError):
        return None


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
    ap.add_argument("--no-decode", action="store_true", help="skip the decode sub-records of the default run")
    ap.add_argument("--no-triton", action="store_true", help="skip the reference's Triton kernels")
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

    import torch.distributed as dist
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != a.gpus:
        raise SystemExit(f"--gpus {a.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    try:
        if w["kind"] != "prefill":
            import bench_decode
            line = bench_decode.run(a, w, dev, rank, world)
        else:
            line = run_prefill(a, w, dev, rank, world)
            default_run = a.workload == "prefill_128k" and not a.tq and not a.batch
            if default_run and not a.no_decode:
                import bench_decode
                torch.cuda.empty_cache()
                sub = argparse.Namespace(**{**vars(a), "steps": 64, "no_cpu_baseline": a.no_cpu_baseline})
                if world == 1:
                    sub.workload = "decode_128k"
                    rec = bench_decode.run(sub, dict(WORKLOADS["decode_128k"]), dev, rank, world, triton=not a.no_triton)
                    if rank == 0:
                        line["decode"] = rec
                    torch.cuda.empty_cache()
                if WORKLOADS["decode_1m"]["shards"] % world == 0:
                    sub.workload = "decode_1m"
                    rec = bench_decode.run(sub, dict(WORKLOADS["decode_1m"]), dev, rank, world)
                    if rank == 0:
                        line["decode_1m"] = rec
        if rank == 0:
            print(json.dumps(line), flush=True)
    finally:
        if world > 1:
            dist.destroy_process_group()


def run_prefill(a, w, dev, rank, world):
    import torch.distributed as dist
    from hip_attention_b200 import PhaseTimer, _lib, hip_attention_impl, read_status
    from hip_attention_b200.sharded import kv_head_slice, make_score_reduce
    lib = _lib.load()
    local = dev.index
    hs, kvs = kv_head_slice(rank, world, w["H"], w["HKV"])
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
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
    # clocks and throttle reasons: the samples from the first warm-up step to the end of the timed steps count
    sampler.mark()
    for _ in range(max(a.warmup, 3)):
        out, md = step()
    barrier()
    check_status("the warm-up steps")

    # ---- device-resident timing -------------------------------------------------------------
    timers = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    launches0 = lib.hipattn_launch_count()
    e0.record()
    for _ in range(a.steps):
        t = PhaseTimer()
        out, md = step(t)
        timers.append(t)
    e1.record()
    barrier()
    launches = lib.hipattn_launch_count() - launches0
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
    mask_hash = hashlib.sha256(md.indices[0].cpu().numpy().tobytes() + md.ks[0].cpu().numpy().tobytes()).hexdigest()

    # ---- end to end: pinned host inputs in, output back, every step ---------------------------
    # Three streams (copy in, compute, copy out) and two sets of device buffers: the host-to-device
    # copy of step i + 1 and the device-to-host copy of step i - 1 overlap the kernels of step i.
    # Each rank stages only its own heads, in pinned memory allocated and first touched on the GPU's NUMA node.
    affinity = os.sched_getaffinity(0)
    near = gpu_numa_cpus(local)
    if near:
        os.sched_setaffinity(0, near)
    hq, hk, hv = (torch.empty(x.shape, dtype=x.dtype).pin_memory() for x in (q, k, v))
    for h_, d_ in ((hq, q), (hk, k), (hv, v)):
        h_.copy_(d_)
    houts = [torch.empty(out.shape, dtype=out.dtype).pin_memory() for _ in range(2)]
    for h_ in houts:
        h_.zero_()
    if near:
        os.sched_setaffinity(0, affinity)
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
    h2d_rank = sum(x.numel() * x.element_size() for x in (hq, hk, hv))
    h2d = h2d_rank * world
    d2h = houts[0].numel() * houts[0].element_size() * world
    del dbuf, hq, hk, hv, houts

    if rank != 0:
        return None
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    hbm_peak, peak_src = (peaks["hbm_gbs"], "measured") if "hbm_gbs" in peaks else (6650.0, "fallback")
    tc_peak = peaks.get("bf16_tflops", 1590.0)
    sb = scan_bytes(w, heads_local)
    sf = scan_flops(w, heads_local)
    af = attention_flops(w, heads_local)
    att_ms = phases.get("attention", 0.0)
    tokens = w["B"] * w["TQ"]
    scan_tf = sf / 1e12 / (scan_ms / 1e3) if scan_ms > 0 else None
    att_tf = af / 1e12 / (att_ms / 1e3) if att_ms > 0 else None
    # The scan launches are the larger share of the step.  Their key-row gathers are served by L2 (one KV head's keys are
    # swept by all its query blocks; the DRAM traffic measured under ncu is about 1 % of the gathered bytes), so the bound
    # that applies is the tensor pipe their dot products run on; the gather rate and the DRAM traffic are side figures.
    scan_roof = {"kernel": "scan stage kernels (%d launches per step)" % n_scan, "bound": "tensor", "achieved": scan_tf,
                 "peak": tc_peak, "peak_source": peak_src, "unit": "TFLOP/s", "frac": scan_tf / tc_peak if scan_tf else None,
                 "traffic": NCU_DRAM_BYTES_PER_SCAN_LAUNCH.get((a.workload, world, w["TQ"])),
                 "traffic_source": NCU_TRAFFIC_SOURCE if (a.workload, world, w["TQ"]) in NCU_DRAM_BYTES_PER_SCAN_LAUNCH else None,
                 "flops_per_launch": sf / max(1, n_scan), "launch_ms": scan_ms / max(1, n_scan),
                 "algorithm": "flops and bytes of the reference's rounds (two key rows per chunk, head and round); the "
                              "kernels skip rows whose score is already known, see the *_executed figures",
                 "flops_executed_per_launch": scan_flops(w, heads_local, True) / max(1, n_scan),
                 "executed_tflops": scan_flops(w, heads_local, True) / 1e12 / (scan_ms / 1e3) if scan_ms > 0 else None,
                 "gathered_bytes_per_launch": scan_bytes(w, heads_local, True) / max(1, n_scan),
                 "gather_gbs": scan_bytes(w, heads_local, True) / 1e9 / (scan_ms / 1e3) if scan_ms > 0 else None,
                 "gather_served_by": "L2; the gather rate is not an HBM figure and may exceed the HBM copy peak",
                 "hbm_peak_gbs": hbm_peak}
    att_roof = {"kernel": "bsa_tcgen05 prefill attention kernel", "bound": "tensor", "achieved": att_tf, "peak": tc_peak,
                "peak_source": peak_src, "unit": "TFLOP/s", "frac": att_tf / tc_peak if att_tf else None, "traffic": None,
                "flops_per_launch": af, "launch_ms": att_ms}
    scan_dominant = scan_ms >= att_ms
    line = {
        "metric": "hip_prefill_tokens_per_s", "value": tokens / (ms_step / 1e3), "unit": "tokens/s",
        "n_gpus": world, "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
        "config": config_of(a, w, world), "clocks": clocks,
        "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "h2d_gbs_per_gpu_if_copies_alone_set_the_pace": h2d_rank / 1e9 / (e2e_ms / 1e3),
                "staging": "pinned host buffers on the GPU's NUMA node" if near else "pinned host buffers"},
        "gpu_launches": int(launches), "gpu_launches_counted_by": "hipattn_launch_count() around the timed steps (rank 0)",
        "phases_ms": {k_: round(v_, 4) for k_, v_ in phases.items() if k_ != "start"},
        "mask_sha256": mask_hash,
        "roofline": scan_roof if scan_dominant else att_roof,
        ("attention_roofline" if scan_dominant else "scan_roofline"): att_roof if scan_dominant else scan_roof,
    }
    if world == 1 and not a.no_cpu_baseline:
        cores = len(os.sched_getaffinity(0))
        torch.set_num_threads(cores)
        dt, toks, ref_out, m, r0 = cpu_sample(w, a.cpu_blocks, (q.cpu(), k.cpu(), v.cpu()))
        line["cpu_baseline"] = {"value": toks / dt, "unit": "tokens/s", "cores": cores, "kind": "port",
                                "sample": f"the last {a.cpu_blocks} query blocks ({toks} queries) against all "
                                          f"{w['T']} keys, {dt:.1f} s"}
        # the sample's mask and output against what the GPU produced for the same query blocks
        d0 = r0 // w["bq"]
        gi, gk = md.indices[:, d0:].cpu(), md.ks[:, d0:].cpu()
        mask_equal = bool(torch.equal(gi, m.indices) and torch.equal(gk, m.ks))
        err = (out[:, r0:].float().cpu() - ref_out.float()).abs()
        line["parity"] = {"blocks": a.cpu_blocks, "mask_equal": mask_equal, "out_max_abs": float(err.max()),
                          "out_mean_abs": float(err.mean()), "tolerance": {"max_abs": 2e-2, "mean_abs": 2e-3},
                          "against": "CPU oracle on the same tensors"}
        if not mask_equal or err.max().item() > 2e-2 or err.mean().item() > 2e-3:
            print(json.dumps(line), flush=True)
            raise SystemExit("bench.py: the GPU result differs from the CPU oracle on the sampled query blocks")
    if world == 1 and not a.no_triton and not a.tq and not a.batch:
        ours = (out, md)
        del q, k, v
        torch.cuda.empty_cache()
        line["triton_reference"] = triton_reference_leg(w, ours)
    return line


if __name__ == "__main__":
    main()
