"""Decode workloads of bench.py (benchmark configurations 3 and 4); selected with ``bench.py --workload decode_128k | decode_1m``.

``decode_128k``: 32 sequences of 131072 tokens in a paged cache (page 64, permuted page table); one step
is one ``hip_attention_12`` call with one query row per sequence; the mask is re-estimated every 8th
step and reused in between (``cached_metadata``), 64 steps are averaged.  The sequence length is held
constant so that every step costs the same.
``decode_1m``: one sequence of 1048576 tokens cut into 8 logical shards of 131072 tokens; each shard is
an operator call on its pages (top-k 512 per shard, sink in the first, window in the last shard) and
the partial outputs are merged by log-sum-exp.  With N GPUs each rank runs 8 / N shards and the
partials are all-gathered.
"""
from __future__ import annotations

import hashlib
import json
import os
import time

import numpy as np
import torch

import bench


def _paged_pool(w, dev, kv_heads=None, seqs=None, t0=0, t1=None):
    """Build the page pool for sequences ``seqs`` (default all) over tokens [t0, t1)."""
    B, T, HKV, D, P = w["B"], w["T"], w["HKV"], w["D"], w["page"]
    t1 = T if t1 is None else t1
    dt = bench._DT[w["dtype"]]
    hk = range(HKV)[kv_heads] if kv_heads is not None else range(HKV)
    nh = len(hk)
    pages_per_seq = (t1 - t0) // P
    n_pages = B * pages_per_seq + 17
    g = torch.Generator(device="cpu")
    g.manual_seed(w["seed"] + 7)
    perm = torch.randperm(n_pages, generator=g)[: B * pages_per_seq].view(B, pages_per_seq).to(dev)
    kc = torch.zeros((n_pages, P, nh, D), dtype=dt, device=dev)
    vc = torch.zeros((n_pages, P, nh, D), dtype=dt, device=dev)
    needles = None
    for b in range(B):
        gg = torch.Generator(device=dev)
        gg.manual_seed(w["seed"] * 100 + b)
        step = 131072
        for s0 in range(0, T, step):  # full sequence is generated so that every slice sees the same values
            k = torch.randn((1, step, HKV, D), generator=gg, device=dev, dtype=torch.float32)
            k = bench.rope(k, torch.arange(s0, s0 + step, device=dev), w["theta"])
            if w["heavy"] > 0:
                hh = torch.rand((1, step), generator=gg, device=dev) < w["heavy"]
                k = torch.where(hh[:, :, None, None], k * 4.0, k)
            v = torch.randn((1, step, HKV, D), generator=gg, device=dev, dtype=torch.float32)
            lo, hi = max(s0, t0), min(s0 + step, t1)
            if lo < hi:
                ks = k[0, lo - s0: hi - s0][:, list(hk)].to(dt)
                vs = v[0, lo - s0: hi - s0][:, list(hk)].to(dt)
                pg = perm[b, (lo - t0) // P: (hi - t0) // P]
                kc[pg] = ks.view(-1, P, nh, D)
                vc[pg] = vs.view(-1, P, nh, D)
    return kc, vc, perm.to(torch.int32)


def _queries(w, dev, steps, heads=None):
    g = torch.Generator(device=dev)
    g.manual_seed(w["seed"] * 1000 + 1)
    q = torch.randn((steps, w["B"], 1, w["H"], w["D"]), generator=g, device=dev, dtype=torch.float32)
    pos = torch.full((1,), w["T"] - 1, device=dev)
    q = bench.rope(q.flatten(0, 1), pos.expand(1), w["theta"]).view_as(q) * (w["D"] ** -0.5)
    q = q.to(bench._DT[w["dtype"]])
    if heads is not None:
        q = q[:, :, :, heads].contiguous()
    return q


def _check_status(dev):
    # a kernel that gave up on a bounded on-chip wait, or clamped a bad index, says so in the device status word:
    # a number measured on such a run is not a measurement
    from hip_attention_b200 import read_status
    st = read_status(dev)
    if st != 0:
        raise SystemExit(f"bench_decode.py: device status word {st:#x} after the measured steps; the run is invalid")


def fetched_scan_bytes(w, heads):
    """Key-row bytes the scan of one refresh requests: per stage the rounds' rows (two per chunk, head and round),
    or, where the chunk is small enough for whole-chunk scoring (chunk <= 32 and <= heads-per-KV-head x 2 x rounds),
    every token of the active chunks once per KV head."""
    import math
    total = 0.0
    gq = w["H"] // w["HKV"]
    hb = 4 if gq % 4 == 0 else (2 if gq % 2 == 0 else 1)
    for i, c in enumerate(w["chunks"]):
        w1 = dict(w, chunks=w["chunks"][:i + 1], keep=w["keep"][:max(i, 1)])
        w0 = dict(w, chunks=w["chunks"][:i], keep=w["keep"][:max(i - 1, 1)]) if i else None
        rounds_bytes = bench.scan_bytes(w1, heads) - (bench.scan_bytes(w0, heads) if w0 else 0.0)
        r = int(math.log2(c)) + 1
        if 4 <= c <= 32 and c <= hb * 2 * r:
            total += rounds_bytes * c / (2.0 * r * hb)     # c rows per chunk and head batch instead of 2 r per head
        else:                                              # rounds: a candidate that repeats the last winner is not fetched
            total += bench.scan_bytes(w1, heads, True) - (bench.scan_bytes(w0, heads, True) if w0 else 0.0)
    return total


def run(a, w, dev, rank, world, triton=False):
    """Runs a decode workload on this rank; returns the JSON record on rank 0 (None elsewhere)."""
    import torch.distributed as dist
    from hip_attention_b200 import PhaseTimer, _lib, hip_attention_impl
    from hip_attention_b200.sharded import hip_attention_12_sequence_sharded
    lib = _lib.load()
    local = dev.index
    steps = a.steps if a.steps != 5 else 64
    B, T, H, HKV, D = w["B"], w["T"], w["H"], w["HKV"], w["D"]
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(bench.ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak, peak_src = (peaks["hbm_gbs"], "measured") if "hbm_gbs" in peaks else (6650.0, "fallback")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if w["kind"] == "decode":
        if world > 1:
            raise SystemExit("decode_128k is a single-GPU workload (independent sequences: run replicas)")
        kc, vc, table = _paged_pool(w, dev)
        seq = torch.full((B,), T, dtype=torch.int32, device=dev)
        pos = torch.full((B, 1), T - 1, dtype=torch.int64, device=dev)
        args = bench.make_args(w, k_cache=kc, v_cache=vc, block_table=table, cache_seq_lens=seq, position_ids=pos,
                               extend_context_length=T)
        qs = _queries(w, dev, steps)
        refresh = w["refresh"]

        def run_steps(n, timers=None, host=None):
            md = None
            for i in range(n):
                t = PhaseTimer() if timers is not None else None
                if host is not None:
                    q = host["dq"]
                    q.copy_(host["hq"][i % steps], non_blocking=True)
                else:
                    q = qs[i % steps]
                out, md = hip_attention_impl(q, None, None, args, None if i % refresh == 0 else md, timer=t)
                if host is not None:
                    host["ho"].copy_(out, non_blocking=True)
                if timers is not None:
                    timers.append(t)
            return out

        run_steps(max(a.warmup, 3) + refresh)  # at least one refresh + cached steps
        barrier()
        sampler = bench.ClockSampler(local)
        sampler.start()
        timers = []
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = lib.hipattn_launch_count()
        e0.record()
        run_steps(steps, timers)
        e1.record()
        barrier()
        launches = lib.hipattn_launch_count() - launches0
        clocks = sampler.stop()
        ms_step = e0.elapsed_time(e1) / steps
        ph_refresh, ph_cached, n_r, n_c = {}, {}, 0, 0
        for i, t in enumerate(timers):
            tgt = ph_refresh if i % refresh == 0 else ph_cached
            for k_, v_ in t.milliseconds().items():
                tgt[k_] = tgt.get(k_, 0.0) + v_
            n_r += i % refresh == 0
            n_c += i % refresh != 0
        ph_refresh = {k_: v_ / max(1, n_r) for k_, v_ in ph_refresh.items() if k_ != "start"}
        ph_cached = {k_: v_ / max(1, n_c) for k_, v_ in ph_cached.items() if k_ != "start"}
        host = {"hq": qs.cpu().pin_memory(), "dq": torch.empty_like(qs[0]),
                "ho": torch.empty(qs[0].shape, dtype=qs.dtype).pin_memory()}
        run_steps(refresh, host=host)
        barrier()
        e0.record()
        run_steps(steps, host=host)
        e1.record()
        barrier()
        e2e_ms = e0.elapsed_time(e1) / steps
        # ---- CUDA graphs: one graph for a refresh step, one for a cached-mask step, replayed on new queries ----
        q_static = qs[0].clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            _, md0 = hip_attention_impl(q_static, None, None, args)
            hip_attention_impl(q_static, None, None, args, md0)
        torch.cuda.current_stream().wait_stream(side)
        g_refresh, g_cached = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_refresh):
            out_g, md_g = hip_attention_impl(q_static, None, None, args)
        with torch.cuda.graph(g_cached):
            out_c, _ = hip_attention_impl(q_static, None, None, args, md_g)

        def run_graphs(n):
            for i in range(n):
                q_static.copy_(qs[i % steps], non_blocking=True)
                (g_refresh if i % refresh == 0 else g_cached).replay()

        run_graphs(refresh)
        barrier()
        e0.record()
        run_graphs(steps)
        e1.record()
        barrier()
        graph_ms = e0.elapsed_time(e1) / steps
        _check_status(dev)
        fetched = fetched_scan_bytes(w, H)
        scan_ms = sum(v_ for k_, v_ in ph_refresh.items() if k_.startswith("scan"))
        att_bytes = B * HKV * (w["keep"][-1] + w["sink"] + w["sw"]) * D * 2 * 2
        att_ms = ph_cached.get("attention", 0.0)
        scan_gbs = fetched / 1e9 / (scan_ms / 1e3) if scan_ms else None
        line = {
            "metric": "hip_decode_ms_per_step", "value": graph_ms, "unit": "ms/step", "n_gpus": 1, "steps": steps,
            "warmup": max(a.warmup, 3), "ms_per_step": graph_ms, "eager_ms_per_step": ms_step,
            "higher_is_better": False, "scaling": "weak",
            "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": {**bench.config_of(a, w, 1), "l2": "page pool of 2 x 8.6 GB exceeds the 126 MB L2",
                       "launch": "value: two CUDA graphs (refresh step, cached-mask step) replayed; eager_ms_per_step: plain calls"},
            "clocks": clocks,
            "e2e": {"value": e2e_ms, "unit": "ms/step", "h2d_bytes_per_step": qs[0].numel() * 2,
                    "d2h_bytes_per_step": qs[0].numel() * 2},
            "gpu_launches": int(launches), "gpu_launches_counted_by": "hipattn_launch_count() around the eager timed steps",
            "phases_ms": {"refresh_step": ph_refresh, "cached_step": ph_cached},
            # The bytes counted are the key rows the scan kernels request: the stages with small chunks fetch every
            # token of an active chunk once for the heads of a KV head, the others two rows per chunk, head and round.
            "roofline": {"kernel": "scan_stage_kernel + scan_chunks_strict_kernel (refresh steps)", "bound": "hbm",
                         "achieved": scan_gbs, "peak": peak, "peak_source": peak_src,
                         "unit": "GB/s", "frac": scan_gbs / peak if scan_gbs else None, "traffic": None,
                         "algorithmic_bytes_per_refresh": fetched,
                         "bytes_if_every_head_gathered_two_rows_per_round": bench.scan_bytes(w, H), "scan_ms_per_refresh": scan_ms},
            "attention_roofline": {"kernel": "bsa_decode_mma_kernel (split-KV decode)", "bound": "hbm",
                                   "achieved": att_bytes / 1e9 / (att_ms / 1e3) if att_ms else None, "peak": peak,
                                   "unit": "GB/s", "frac": (att_bytes / 1e9 / (att_ms / 1e3)) / peak if att_ms else None,
                                   "algorithmic_bytes_per_step": att_bytes},
        }
        if not a.no_cpu_baseline:
            # one sequence through the CPU oracle on the GPU's own tensors: the baseline, and the parity check
            k0 = kc[table[0].long()].reshape(1, T, HKV, D).cpu()
            v0 = vc[table[0].long()].reshape(1, T, HKV, D).cpu()
            out0, md0_ = hip_attention_impl(qs[0][:1], None, None, bench.make_args(
                w, k_cache=kc, v_cache=vc, block_table=table[:1], cache_seq_lens=seq[:1], position_ids=pos[:1],
                extend_context_length=T))
            rec, ref_out, m = _cpu_decode(w, qs[0][:1].cpu(), k0, v0)
            line["cpu_baseline"] = rec
            mask_equal = bool(torch.equal(md0_.indices.cpu(), m.indices) and torch.equal(md0_.ks.cpu(), m.ks))
            err = (out0.float().cpu() - ref_out.float()).abs()
            line["parity"] = {"sequences": 1, "mask_equal": mask_equal, "out_max_abs": float(err.max()),
                              "out_mean_abs": float(err.mean()), "tolerance": {"max_abs": 2e-2, "mean_abs": 2e-3},
                              "against": "CPU oracle on the same tensors (sequence 0, de-paged)"}
            if not mask_equal or err.max().item() > 2e-2 or err.mean().item() > 2e-3:
                print(json.dumps(line), flush=True)
                raise SystemExit("bench_decode.py: the GPU result differs from the CPU oracle on the sampled sequence")
        if triton:
            line["triton_reference"] = _triton_decode(w, kc, vc, table, qs, steps)
        return line

    # ---- sequence-sharded million-token decode -----------------------------------------------------
    S = w["shards"]
    if S % world:
        raise SystemExit(f"{S} shards cannot be split over {world} ranks")
    per = S // world
    L = T // S
    # one page pool per rank holding its shards; every shard has its own page table into it
    kc, vc, table = _paged_pool(w, dev, t0=rank * per * L, t1=(rank + 1) * per * L)
    pps = L // w["page"]
    shard_kv = [(kc, vc, table[:, j * pps:(j + 1) * pps].contiguous(), torch.full((B,), L, dtype=torch.int32, device=dev))
                for j in range(per)]
    qs = _queries(w, dev, steps)
    args = bench.make_args(w)

    def one(i, cached):
        return hip_attention_12_sequence_sharded(qs[i], shard_kv, args, n_shards=S, shard_len=L, per_shard_k=w["keep"][-1],
                                                 first_shard=rank * per, cached=cached)

    for i in range(max(a.warmup, 3)):
        out, mds = one(i, None)
    barrier()
    out0, _ = one(0, None)
    out_hash = hashlib.sha256(out0.float().cpu().numpy().tobytes()).hexdigest()
    sampler = bench.ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    launches0 = lib.hipattn_launch_count()
    e0.record()
    for i in range(steps):
        out, mds = one(i, None)   # every step re-estimates the mask: the worst case
    e1.record()
    barrier()
    launches = lib.hipattn_launch_count() - launches0
    tms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    e0.record()
    for i in range(steps):
        out, _ = one(i, mds)      # cached masks: attention + merge only
    e1.record()
    barrier()
    tms2 = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    # end to end: the query comes from pinned host memory and the merged output goes back, every step
    hq = qs.cpu().pin_memory()
    dq = torch.empty_like(qs[0])
    ho = torch.empty(qs[0].shape, dtype=qs.dtype).pin_memory()
    barrier()
    e0.record()
    for i in range(steps):
        dq.copy_(hq[i], non_blocking=True)
        o_, _ = hip_attention_12_sequence_sharded(dq, shard_kv, args, n_shards=S, shard_len=L, per_shard_k=w["keep"][-1],
                                                  first_shard=rank * per)
        ho.copy_(o_, non_blocking=True)
    e1.record()
    barrier()
    tms3 = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        for t_ in (tms, tms2, tms3):
            dist.all_reduce(t_, op=dist.ReduceOp.MAX)
    graph_ms = None
    if world == 1:
        q_static = qs[0].clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            hip_attention_12_sequence_sharded(q_static, shard_kv, args, n_shards=S, shard_len=L, per_shard_k=w["keep"][-1])
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out_g, _ = hip_attention_12_sequence_sharded(q_static, shard_kv, args, n_shards=S, shard_len=L,
                                                         per_shard_k=w["keep"][-1])
        for i in range(3):
            g.replay()
        barrier()
        e0.record()
        for i in range(steps):
            q_static.copy_(qs[i], non_blocking=True)
            g.replay()
        e1.record()
        barrier()
        graph_ms = e0.elapsed_time(e1) / steps
    _check_status(dev)
    if rank != 0:
        return None
    clocks = sampler.stop()
    ms_step = float(tms.item()) / steps
    wsh = dict(w, T=L)
    sb = fetched_scan_bytes(wsh, H) * S
    att_bytes = HKV * (S * w["keep"][-1] + w["sink"] + w["sw"] + (S - 1) * w["chunks"][0]) * D * 2 * 2
    gbs = (sb + att_bytes) / 1e9 / (ms_step / 1e3)
    return {"metric": "hip_decode_ms_per_step", "value": ms_step, "unit": "ms/step", "n_gpus": world, "steps": steps,
            "warmup": max(a.warmup, 3), "ms_per_step": ms_step, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": {**bench.config_of(a, w, world), "mask": "re-estimated every step", "parallelism": f"sequence shards x{world}",
                       "l2": "each step draws a new query; the 4.3 GB page pool exceeds the 126 MB L2"},
            "clocks": clocks, "cached_mask_ms_per_step": float(tms2.item()) / steps,
            "cuda_graph_ms_per_step": graph_ms,
            "e2e": {"value": float(tms3.item()) / steps, "unit": "ms/step", "h2d_bytes_per_step": qs[0].numel() * 2,
                    "d2h_bytes_per_step": qs[0].numel() * 2},
            "gpu_launches": int(launches), "gpu_launches_counted_by": "hipattn_launch_count() around the timed steps (rank 0)",
            "merged_output_sha256": out_hash,
            "roofline": {"kernel": "whole step (scan + selection + split-KV attention + merge of every shard)", "bound": "hbm",
                         "achieved": gbs, "peak": peak, "peak_source": peak_src, "unit": "GB/s", "frac": gbs / peak,
                         "traffic": None, "algorithmic_bytes_per_step": sb + att_bytes,
                         "note": "launch-latency bound: a step is a few tens of short launches on 1/Nth of 5 MB of key rows"}}


def run_reference_arm(a, w, cores):
    """CPU arm for the decode workloads: the oracle on one sequence (one refresh and one cached step per timed step)."""
    w1 = dict(w, B=1)
    if w["kind"] == "decode_sharded":
        w1["T"] = w["T"] // w["shards"]   # one logical shard per step
    q, k, v = bench.make_qkv(w1, "cpu")
    vals = []
    for i in range(a.warmup + a.steps):
        rec, _, _ = _cpu_decode(dict(w1, refresh=w.get("refresh", 1)), q, k, v)
        if i >= a.warmup:
            vals.append(rec["value"])
    scale = w["B"] if w["kind"] == "decode" else w["shards"]
    val = float(np.mean(vals)) * scale
    sample = (f"1 of {w['B']} sequences per step, scaled by {w['B']}" if w["kind"] == "decode"
              else f"1 of {w['shards']} sequence shards per step, scaled by {w['shards']}")
    line = {"impl": "reference", "metric": "hip_decode_ms_per_step", "value": val, "unit": "ms/step", "n_gpus": a.gpus,
            "steps": a.steps, "warmup": a.warmup, "ms_per_step": val, "higher_is_better": False,
            "scaling": "weak" if w["kind"] == "decode" else "strong", "vs_baseline": None, "dtype": w["dtype"],
            "data": "synthetic", "config": bench.config_of(a, w, a.gpus),
            "cpu_baseline": {"value": val, "unit": "ms/step", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "ms/step", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def _cpu_decode(w, q, k, v):
    """CPU oracle on one sequence (q [1, 1, H, D], dense k / v): one refresh step and one cached step, scaled to
    the batch and the refresh interval.  Returns (baseline record, output, mask)."""
    from oracle import hip_oracle as O
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    cfg = bench.oracle_config(w)
    T = k.shape[1]
    pos = torch.full((1, 1), T - 1, dtype=torch.int64)
    ks, vs = O.DenseKV(k), O.DenseKV(v)
    t0 = time.perf_counter()
    m = O.estimate_mask(q, ks, pos, cfg)
    t1 = time.perf_counter()
    out = O.attention_on_mask(q, ks, vs, pos, m, sink=cfg.sink, sw=max(cfg.sw, cfg.stages[0].chunk_size), dtype=torch.float32)
    t2 = time.perf_counter()
    r = w.get("refresh", 1)
    per_seq = ((t1 - t0) + r * (t2 - t1)) / r
    rec = {"value": 1e3 * per_seq * w["B"], "unit": "ms/step", "cores": cores, "kind": "port",
           "sample": f"1 of {w['B']} sequences (estimator {t1 - t0:.2f} s once per {r} steps, attention {t2 - t1:.3f} s per step), "
                     f"scaled by {w['B']}"}
    return rec, out, m


def _triton_decode(w, kc, vc, table, qs, steps):
    """The unmodified reference operator on the decode workload: dense K / V rebuilt from the page pool (the reference
    refuses pages of more than 32 tokens, attention_metadata.py:239), its own flash-decode kernels, the same refresh
    schedule, plain calls (no CUDA graph)."""
    import sys
    sys.path.insert(0, os.path.join(bench.ROOT, "baseline"))
    try:
        import reference_loader as R
        if not R.available():
            return {"unavailable": "no copy of the reference under baseline/_ref"}
        op, Args, ScanStage = R.load_reference()
        import triton
        B, T, HKV, D = w["B"], w["T"], w["HKV"], w["D"]
        k = kc[table.long()].reshape(B, T, HKV, D)
        v = vc[table.long()].reshape(B, T, HKV, D)
        pos = torch.full((B, 1), T - 1, dtype=torch.int64, device=k.device)
        ra = R.reference_args(Args, ScanStage, bq=w["bq"], strides=w["strides"], chunks=w["chunks"], keep=w["keep"],
                              sink=w["sink"], sw=w["sw"], position_ids=pos)
        refresh = w["refresh"]

        def run_steps(n):
            md = None
            for i in range(n):
                out, md = op(qs[i % steps], k, v, args=ra, cached_metadata=None if i % refresh == 0 else md)
            return out

        run_steps(2 * refresh)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run_steps(steps)
        e1.record()
        torch.cuda.synchronize()
        return {"ms_per_step": e0.elapsed_time(e1) / steps, "steps": steps, "kv": "dense (de-paged)", "launch": "plain calls",
                "triton": triton.__version__, "torch": torch.__version__, "autotune": "off (HIP_DISABLE_AUTOTUNE=1)"}
    except Exception as e:  # noqa: BLE001 - whatever stops the reference is reported, not raised
        return {"unavailable": f"{type(e).__name__}: {str(e)[:300]}"}
