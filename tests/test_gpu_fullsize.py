"""Full-size checks on a B200: the benchmark configurations themselves, through properties that do not need the
CPU oracle (which would take hours at these sizes).

* structure of the mask: ascending, unique, aligned block starts inside [sink, T), padded with INT64_MAX, ``ks`` = the
  number of entries below the block's first position + block size, identical for all heads of a sequence;
* exactness at full size: the default tensor-core scan and the strict fp32 scan select the same blocks;
* idempotence: the cached mask reproduces the output bit for bit, the stage caches reproduce the mask;
* sampled rows of the output against an fp64 recomputation of the attention set (sink, selected blocks, window).
"""
import os

import pytest
import torch

import bench

pytestmark = pytest.mark.gpu
PAD = torch.iinfo(torch.int64).max


def _check_mask_structure(md, w, pos_first, TQ):
    B, H, bq, c_last = w["B"], w["H"], w["bq"], w["chunks"][-1]
    K = w["keep"][-1] // c_last
    BDST = -(-TQ // bq)
    idx, ks = md.indices, md.ks
    assert idx.shape == (B * H, BDST, K) and ks.shape == (B * H, BDST)
    real = idx != PAD
    assert bool(((idx[..., 1:] > idx[..., :-1]) | ~real[..., 1:]).all()), "indices must ascend (pads last)"
    assert bool((real.long().diff(dim=-1) <= 0).all()), "no real entry after a pad"
    vals = idx[real]
    assert bool((vals >= w["sink"]).all()) and bool((vals < w["T"]).all())
    assert bool((vals % c_last == 0).all()), "block starts are multiples of the last chunk size"
    limit = (pos_first + bq)[:, None, :, None]                     # [B, 1, BDST, 1]
    expect = ((idx.view(B, H, BDST, K) < limit)).sum(-1).view(B * H, BDST)
    assert torch.equal(ks, expect)
    v = idx.view(B, H, BDST, K)
    assert bool((v == v[:, :1]).all()), "the head max-reduce gives every head of a sequence the same blocks"


def _recompute_rows(q, k, v, md, w, rows, pos):
    """fp64 attention of sampled (b, t, h) rows over sink + selected blocks + window (the set the kernels attend)."""
    B, TQ, H, D = q.shape
    HKV, bq, c_last, sink = w["HKV"], w["bq"], w["chunks"][-1], w["sink"]
    W = max(w["sw"], w["chunks"][0])
    out = []
    for (b, t, h) in rows:
        p = int(pos[b, t])
        d = t // bq
        pmax = int(pos[b, min((d + 1) * bq, TQ) - 1])
        n_sel = int(md.ks[b * H + h, d])
        starts = md.indices[b * H + h, d, :n_sel]
        sel = (starts[:, None] + torch.arange(c_last, device=q.device)[None]).flatten()
        sel = sel[(sel >= sink) & (sel <= pmax) & (sel < w["T"]) & (sel <= p - W)]
        snk = torch.arange(0, min(sink, p + 1), device=q.device)
        snk = snk[snk <= p - W]
        win = torch.arange(max(0, p - W + 1), p + 1, device=q.device)
        keys = torch.cat([snk, sel, win])
        assert keys.unique().numel() == keys.numel()
        kk = k[b, keys, h // (H // HKV)].double()
        vv = v[b, keys, h // (H // HKV)].double()
        s = kk @ q[b, t, h].double()
        out.append(torch.softmax(s, 0) @ vv)
    return torch.stack(out)


def test_prefill_128k_full_size(monkeypatch):
    _prefill_full_size(dict(bench.WORKLOADS["prefill_128k"]), monkeypatch)


def test_prefill_256k_gqa_shape(monkeypatch):
    """The large-GQA configuration (query blocks of 128 rows, 64 query heads on 8 KV heads, 262144 keys, sink 256,
    window 2048, stages keeping 65536 / 16384 / 4096 tokens): one sequence and its last 32768 queries, which keeps
    every stage shape (32 / 32 / 128 pooled rows, 1015 / 2048 / 2048 chunks, 512 selected blocks) at a sixteenth of
    the work."""
    _prefill_full_size(dict(bench.WORKLOADS["prefill_256k_gqa"], B=1, TQ=32768), monkeypatch)


def _prefill_full_size(w, monkeypatch):
    from hip_attention_b200 import HiPAttentionOutputMetadata, hip_attention_12, hip_attention_impl, read_status
    q, k, v = bench.make_qkv(w, "cuda")
    args = bench.make_args(w)
    TQ, T = w["TQ"], w["T"]
    pos = (torch.arange(TQ, device="cuda") + T - TQ)[None]
    read_status("cuda")
    out, md = hip_attention_impl(q, k, v, args)
    torch.cuda.synchronize()
    assert read_status("cuda") == 0
    assert torch.isfinite(out.float()).all()
    _check_mask_structure(md, w, pos[:, ::w["bq"]], TQ)
    # the strict fp32 scan selects the same blocks (exactness of the tensor-core scan at full size)
    monkeypatch.setenv("HIPATTN_SCAN_MODE", "strict")
    _, md_strict = hip_attention_impl(q, k, v, args)
    monkeypatch.setenv("HIPATTN_SCAN_MODE", "auto")
    assert torch.equal(md_strict.indices, md.indices) and torch.equal(md_strict.ks, md.ks)
    # cached mask: same output; cached stage inputs: same mask
    out2, _ = hip_attention_12(q, k, v, args, cached_metadata=md)
    assert torch.equal(out2, out)
    part = HiPAttentionOutputMetadata(None, None, None, None, None, None, list(md.stage_caches[:2]))
    _, md3 = hip_attention_12(q, k, v, args, cached_metadata=part)
    assert torch.equal(md3.indices, md.indices)
    # sampled output rows against an fp64 recomputation on the same mask
    g = torch.Generator().manual_seed(5)
    rows = [(0, int(torch.randint(0, TQ, (1,), generator=g)), int(torch.randint(0, w["H"], (1,), generator=g))) for _ in range(24)]
    rows += [(0, 0, 0), (0, TQ - 1, w["H"] - 1), (0, w["bq"] - 1, 3), (0, w["bq"], 3)]
    ref = _recompute_rows(q, k, v, md, w, rows, pos)
    got = torch.stack([out[b, t, h].double() for (b, t, h) in rows])
    err = (got - ref).abs()
    assert err.max().item() <= 2e-2 and err.mean().item() <= 2e-3, (err.max().item(), err.mean().item())


def test_decode_128k_full_size(monkeypatch):
    """Batched decode at the benchmark size (the page pools take 17 GB): mask structure, whole-chunk scan = round-by-round
    scan, cached-mask idempotence, and the paged output of sampled heads against the fp64 recomputation."""
    import bench_decode
    from hip_attention_b200 import hip_attention_12, hip_attention_impl, read_status
    w = dict(bench.WORKLOADS["decode_128k"])
    dev = "cuda"
    kc, vc, table = bench_decode._paged_pool(w, dev)
    B, T, H, D, P = w["B"], w["T"], w["H"], w["D"], w["page"]
    g = torch.Generator(device=dev)
    g.manual_seed(99)
    q = (torch.randn((B, 1, H, D), generator=g, device=dev) * (D ** -0.5)).to(torch.bfloat16)
    pos = torch.full((B, 1), T - 1, dtype=torch.int64, device=dev)
    args = bench.make_args(w, position_ids=pos, k_cache=kc, v_cache=vc, block_table=table,
                           cache_seq_lens=torch.full((B,), T, dtype=torch.int32, device=dev), extend_context_length=T)
    read_status(dev)
    out, md = hip_attention_impl(q, None, None, args)
    torch.cuda.synchronize()
    assert read_status(dev) == 0
    _check_mask_structure(md, w, pos[:, :1], 1)
    monkeypatch.setenv("HIPATTN_DECODE_SCAN", "rounds")
    out_r, md_r = hip_attention_impl(q, None, None, args)
    monkeypatch.delenv("HIPATTN_DECODE_SCAN")
    assert torch.equal(md_r.indices, md.indices) and torch.equal(md_r.ks, md.ks) and torch.equal(out_r, out)
    out2, _ = hip_attention_12(q, None, None, args, cached_metadata=md)
    assert torch.equal(out2, out)
    # de-page two sequences and recompute sampled heads in fp64
    for b in (0, B - 1):
        kd = kc[table[b].long()].reshape(1, T, w["HKV"], D)
        vd = vc[table[b].long()].reshape(1, T, w["HKV"], D)
        rows = [(0, 0, h) for h in (0, 5, H - 1)]
        sub = type(md)(indices=md.indices[b * H:(b + 1) * H], ks=md.ks[b * H:(b + 1) * H], ks_count=None, ks_start_end=None,
                       mask_cache_statistics=None, sa_cache_statistics=None, stage_caches=None)
        ref = _recompute_rows(q[b:b + 1], kd, vd, sub, dict(w, B=1), rows, pos[b:b + 1])
        got = torch.stack([out[b, 0, h].double() for (_, _, h) in rows])
        err = (got - ref).abs()
        assert err.max().item() <= 2e-2 and err.mean().item() <= 2e-3, (b, err.max().item())
