#!/usr/bin/env python
"""Timings of the operator's variants on the benchmark shapes: paged prefill and the in-kernel RoPE backends.

    python bench_variants.py [--tq Q] [--page P] [--steps K] [--warmup W]

One GPU.  Prints one JSON line per variant (CUDA events around K calls after W warm-up calls, inputs resident in
HBM and larger than L2), each with the per-phase split of the last call:

* ``prefill dense`` / ``prefill paged``: benchmark configuration 2 with Q queries, K/V contiguous or behind a block
  table of shuffled P-token pages; the paged line also says whether mask and output equal the dense call's;
* ``prefill rope=...``: the same call with un-rotated K in the cache and the ``relative`` / ``streaming`` scan backends
  (rotation inside the scan and attention kernels);
* ``decode rope=...``: benchmark configuration 3's shape at batch 8, a mask-refresh step and a cached-mask step.

These are not the headline figures (``bench.py`` prints those); they put a number beside every variant the parity
tests cover.
"""
from __future__ import annotations

import argparse
import json

import numpy as np
import torch

import bench


def rope_tables(T: int, D: int, theta: float, device):
    """cos / sin tables [T, D], half-dimension frequencies repeated (rotate-half convention)."""
    inv = 1.0 / (theta ** (np.arange(0, D, 2, dtype=np.float64) / D))
    ang = np.arange(T, dtype=np.float64)[:, None] * inv[None, :]
    ang = np.concatenate([ang, ang], axis=-1)
    return (torch.from_numpy(np.cos(ang).astype(np.float32)).to(device),
            torch.from_numpy(np.sin(ang).astype(np.float32)).to(device))


def timed(fn, steps: int, warmup: int):
    """Milliseconds per call of ``fn`` and the result of the last call."""
    for _ in range(max(warmup, 3)):
        res = fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        res = fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps, res


def main():
    from hip_attention_b200 import PhaseTimer, hip_attention_impl, read_status
    ap = argparse.ArgumentParser()
    ap.add_argument("--tq", type=int, default=4096, help="queries of the prefill variants")
    ap.add_argument("--page", type=int, default=64, help="tokens per page of the paged variant")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    read_status(dev)

    def emit(name: str, ms: float, call, **extra):
        t = PhaseTimer()
        call(t)
        torch.cuda.synchronize()
        st = read_status(dev)
        if st != 0:
            raise SystemExit(f"bench_variants.py: device status word {st:#x} after {name}")
        phases = {k: round(v, 4) for k, v in t.milliseconds().items() if k != "start"}
        print(json.dumps({"variant": name, "ms_per_call": round(ms, 4), "steps": a.steps, "phases_ms": phases, **extra}),
              flush=True)

    # ---- prefill: dense and paged -------------------------------------------------------------------
    w = dict(bench.WORKLOADS["prefill_128k"], TQ=a.tq)
    q, k, v = bench.make_qkv(w, dev)
    B, T, HKV, D = k.shape
    shape = {"queries": a.tq, "keys": T, "dtype": w["dtype"]}
    args = bench.make_args(w)
    ms, (o0, md0) = timed(lambda: hip_attention_impl(q, k, v, args), a.steps, a.warmup)
    emit("prefill dense", ms, lambda t: hip_attention_impl(q, k, v, args, timer=t), **shape)

    n_pages = T // a.page
    perm = torch.randperm(n_pages, device=dev, generator=torch.Generator(device=dev).manual_seed(7))
    k_cache = torch.empty((n_pages + 1, a.page, HKV, D), dtype=k.dtype, device=dev)
    v_cache = torch.empty_like(k_cache)
    k_cache[perm + 1] = k[0].view(n_pages, a.page, HKV, D)
    v_cache[perm + 1] = v[0].view(n_pages, a.page, HKV, D)
    pargs = bench.make_args(w, k_cache=k_cache, v_cache=v_cache, block_table=(perm + 1).to(torch.int32).view(1, n_pages),
                            cache_seq_lens=torch.tensor([T], dtype=torch.int32, device=dev),
                            position_ids=torch.arange(T - a.tq, T, device=dev).view(1, a.tq), extend_context_length=T)
    ms, (o1, md1) = timed(lambda: hip_attention_impl(q, None, None, pargs), a.steps, a.warmup)
    emit("prefill paged", ms, lambda t: hip_attention_impl(q, None, None, pargs, timer=t), page=a.page, **shape,
         mask_equals_dense=bool(torch.equal(md0.indices, md1.indices)),
         out_max_abs_diff_to_dense=float((o0.float() - o1.float()).abs().max()))
    del k_cache, v_cache, o0, o1, md0, md1

    # ---- prefill and decode: RoPE inside the kernels ---------------------------------------------------
    cos, sin = rope_tables(T + 8, D, w["theta"], dev)

    def rope_kw(backend):
        if backend is None:
            return {}
        return dict(using_extend=True, need_apply_rope=True, rope_cos=cos, rope_sin=sin, scan_extend_backend=backend)

    for backend in (None, "relative", "streaming"):
        rargs = bench.make_args(w, **rope_kw(backend))
        ms, _ = timed(lambda: hip_attention_impl(q, k, v, rargs), a.steps, a.warmup)
        emit(f"prefill rope={backend or 'none'}", ms, lambda t: hip_attention_impl(q, k, v, rargs, timer=t), **shape)
    del q, k, v

    wd = dict(bench.WORKLOADS["decode_128k"], B=8, kind="prefill")
    qd, kd, vd = bench.make_qkv(wd, dev)
    for backend in (None, "relative", "streaming"):
        dargs = bench.make_args(wd, **rope_kw(backend))
        ms, (_, md) = timed(lambda: hip_attention_impl(qd, kd, vd, dargs), a.steps, a.warmup)
        ms_c, _ = timed(lambda: hip_attention_impl(qd, kd, vd, dargs, md), a.steps, a.warmup)
        emit(f"decode rope={backend or 'none'}", ms, lambda t: hip_attention_impl(qd, kd, vd, dargs, timer=t),
             batch=8, keys=wd["T"], dtype=wd["dtype"], ms_per_cached_mask_call=round(ms_c, 4))


if __name__ == "__main__":
    main()
