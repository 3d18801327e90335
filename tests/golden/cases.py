"""Shared definitions of the golden parity cases.

Each case fixes shapes, dtype, estimator stages and a seed.  Inputs are drawn from
``numpy.random.RandomState`` (a frozen stream) so that the generator script, the
CPU oracle tests and the GPU parity tests all see bit-identical tensors without
storing them.  ``gen_golden.py`` runs the reference operator on these inputs and
stores its outputs next to this file as ``<name>.npz``.
"""
from __future__ import annotations

import numpy as np
import torch

_DT = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}

# stages: list of (stage_block_size_q, stage_block_stride_q, stage_chunk_size, stage_k)
CASES = {
    # fp32, three stages, Tq < Tk (chunked prefill)
    "prefill_fp32": dict(B=1, TQ=256, T=2048, H=4, HKV=2, D=64, dtype="fp32", sink=32, sw=128,
                         second_k=128, stages=[(64, 4, 64, None), (64, 2, 16, 512), (64, 1, 4, 256)], seed=11),
    # fp16, ragged last query block, two stages
    "ragged_fp16": dict(B=2, TQ=100, T=1024, H=4, HKV=2, D=64, dtype="fp16", sink=32, sw=128,
                        second_k=128, stages=[(64, 2, 32, None), (64, 1, 8, 256)], seed=12),
    # fp16 decode (one query row), flash-decode back end in the reference
    "decode_fp16": dict(B=2, TQ=1, T=2048, H=8, HKV=2, D=64, dtype="fp16", sink=32, sw=128,
                        second_k=128, stages=[(64, 4, 64, None), (64, 4, 16, 512), (64, 1, 4, 256)], seed=13),
    # Tq == Tk: early query blocks see only inactive chunks (ties at -32000)
    "square_fp16": dict(B=1, TQ=1024, T=1024, H=2, HKV=1, D=64, dtype="fp16", sink=16, sw=64,
                        second_k=64, stages=[(64, 4, 32, None), (64, 1, 8, 128)], seed=14),
    # exactly representable arithmetic: D=256 (scales 4 and 1/4), values on a 1/4 grid
    "exact_fp32": dict(B=1, TQ=192, T=1536, H=4, HKV=2, D=256, dtype="fp32", sink=32, sw=128,
                       second_k=128, stages=[(64, 4, 64, None), (64, 1, 8, 512)], seed=15, quant=True),
    # paged KV (page 16, permuted pool, chunk grid longer than the live sequence), decode
    "paged_decode_fp16": dict(B=2, TQ=1, T=1024, H=4, HKV=2, D=64, dtype="fp16", sink=32, sw=128,
                              second_k=128, stages=[(64, 4, 32, None), (64, 1, 8, 256)], seed=16,
                              page=16, ext=1536),
    # paged KV, ragged prefill
    "paged_prefill_fp16": dict(B=1, TQ=100, T=1024, H=4, HKV=2, D=64, dtype="fp16", sink=32, sw=128,
                               second_k=128, stages=[(64, 4, 32, None), (64, 1, 8, 256)], seed=17,
                               page=16, ext=1024),
    # no sink and no window (a non-owning sequence shard); prefill back end forced
    "shard_nosink_fp16": dict(B=1, TQ=1, T=1024, H=4, HKV=2, D=64, dtype="fp16", sink=0, sw=0,
                              second_k=128, stages=[(64, 2, 32, None), (64, 1, 8, 256)], seed=18,
                              disable_flashdecode=True),
    # sink not a multiple of the last chunk size: per-head narrowing becomes visible
    "oddsink_fp16": dict(B=1, TQ=128, T=1024, H=4, HKV=2, D=64, dtype="fp16", sink=20, sw=96,
                         second_k=64, stages=[(64, 4, 32, None), (64, 1, 8, 128)], seed=19),
    # window shorter than the first chunk size: right bounds are clamped
    "shortwin_fp16": dict(B=1, TQ=128, T=1000, H=2, HKV=2, D=64, dtype="fp16", sink=8, sw=16,
                          second_k=64, stages=[(64, 4, 32, None), (64, 1, 8, 128)], seed=20),
    # per-batch positions given explicitly
    "positions_fp16": dict(B=2, TQ=64, T=1024, H=4, HKV=2, D=64, dtype="fp16", sink=32, sw=128,
                           second_k=128, stages=[(64, 4, 32, None), (64, 1, 8, 256)], seed=21,
                           pos_offsets=[700, 959]),
    # soft-capped logits (Gemma-2 style): tanh(x / cap) * cap inside the attention kernels only
    "softcap_fp16": dict(B=1, TQ=100, T=1024, H=4, HKV=2, D=64, dtype="fp16", sink=32, sw=128,
                         second_k=128, stages=[(64, 4, 32, None), (64, 1, 8, 256)], seed=22, softcap=1.5),
    "softcap_decode_fp16": dict(B=2, TQ=1, T=1024, H=4, HKV=2, D=64, dtype="fp16", sink=32, sw=128,
                                second_k=128, stages=[(64, 4, 32, None), (64, 1, 8, 256)], seed=23, softcap=1.5),
    # head dim 128, three stages with 16 and 64 pooled query rows: the tcgen05 scan and attention kernels
    "d128_fp16": dict(B=1, TQ=192, T=2048, H=4, HKV=2, D=128, dtype="fp16", sink=32, sw=128,
                      second_k=256, stages=[(64, 4, 64, None), (64, 4, 16, 512), (64, 1, 8, 256)], seed=24),
    # query blocks of 128 rows, eight query heads on one KV head, head dim 128 (the large-GQA prefill shape)
    "bq128_fp16": dict(B=1, TQ=256, T=2048, H=8, HKV=1, D=128, dtype="fp16", sink=32, sw=128,
                       second_k=256, stages=[(128, 4, 64, None), (128, 4, 16, 512), (128, 1, 8, 256)], seed=25),
    # attention blocks of 16 rows under estimator blocks of 64, ragged last block: the returned mask is
    # broken down to the attention block size (repeat-interleave)
    "bsa16_fp16": dict(B=1, TQ=100, T=1024, H=4, HKV=2, D=64, dtype="fp16", sink=32, sw=128,
                       second_k=128, stages=[(64, 2, 32, None), (64, 1, 8, 256)], seed=26, bsa_bq=16),
    # in-kernel RoPE (using_extend + need_apply_rope): q and k arrive un-rotated with cos / sin tables; scan backend
    # "relative" (keys at position 0 / 1, queries at 1 + window) and "streaming" (keys at their chunk's ordinal),
    # attention backend "streaming"
    "rope_rel_fp16": dict(B=1, TQ=128, T=1024, H=4, HKV=2, D=64, dtype="fp16", sink=32, sw=128, second_k=128,
                          stages=[(64, 4, 32, None), (64, 1, 8, 256)], seed=27, rope_in_kernel="relative", rope_theta=10000.0),
    "rope_str_fp16": dict(B=1, TQ=100, T=1024, H=4, HKV=2, D=64, dtype="fp16", sink=32, sw=128, second_k=128,
                          stages=[(64, 4, 32, None), (64, 1, 8, 256)], seed=28, rope_in_kernel="streaming", rope_theta=10000.0),
    "rope_decode_fp16": dict(B=2, TQ=1, T=1024, H=4, HKV=2, D=64, dtype="fp16", sink=32, sw=128, second_k=128,
                             stages=[(64, 4, 32, None), (64, 1, 8, 256)], seed=29, rope_in_kernel="relative", rope_theta=10000.0),
    "rope_mixed_fp32": dict(B=1, TQ=192, T=2048, H=4, HKV=2, D=64, dtype="fp32", sink=32, sw=128, second_k=128,
                            stages=[(64, 4, 64, None), (64, 2, 16, 512), (64, 1, 4, 256)], seed=30, rope_in_kernel="relative",
                            stage_backends=[None, "streaming", None], rope_theta=500000.0),
    # head dim 128: the tcgen05 scan (two rotated key copies) and the tcgen05 attention kernel with rotation in the tile
    "rope_d128_fp16": dict(B=1, TQ=192, T=2048, H=4, HKV=2, D=128, dtype="fp16", sink=32, sw=128, second_k=256,
                           stages=[(64, 4, 64, None), (64, 4, 16, 512), (64, 1, 8, 256)], seed=41, rope_in_kernel="relative",
                           rope_theta=10000.0),
    "rope_d128_str_fp16": dict(B=1, TQ=200, T=2048, H=4, HKV=2, D=128, dtype="fp16", sink=32, sw=128, second_k=256,
                               stages=[(64, 4, 64, None), (64, 1, 8, 256)], seed=42, rope_in_kernel="streaming",
                               rope_theta=500000.0),
    "rope_str_decode_fp16": dict(B=2, TQ=1, T=1024, H=4, HKV=2, D=128, dtype="fp16", sink=32, sw=128, second_k=128,
                                 stages=[(64, 4, 32, None), (64, 1, 8, 256)], seed=31, rope_in_kernel="streaming",
                                 rope_theta=10000.0),
    # fp8 KV: k and v are e5m2 values, handed to the operator as 1-byte tensors (make_inputs returns them widened to
    # the case dtype, which is exact; the generator and the GPU tests pass the 1-byte form)
    "fp8_prefill_fp16": dict(B=2, TQ=100, T=1024, H=4, HKV=2, D=64, dtype="fp16", sink=32, sw=128, second_k=128,
                             stages=[(64, 2, 32, None), (64, 1, 8, 256)], seed=32, kv_fp8=True),
    "fp8_decode_fp16": dict(B=2, TQ=1, T=2048, H=8, HKV=2, D=64, dtype="fp16", sink=32, sw=128, second_k=128,
                            stages=[(64, 4, 64, None), (64, 4, 16, 512), (64, 1, 4, 256)], seed=33, kv_fp8=True),
    # access statistics (require_cache_statistics): which tokens / pages the estimator and the attention kernels loaded
    "stats_prefill_fp16": dict(B=2, TQ=100, T=1024, H=4, HKV=2, D=64, dtype="fp16", sink=32, sw=128, second_k=128,
                               stages=[(64, 2, 32, None), (64, 1, 8, 256)], seed=34, stats=True),
    "stats_decode_fp16": dict(B=2, TQ=1, T=2048, H=8, HKV=2, D=64, dtype="fp16", sink=32, sw=128, second_k=128,
                              stages=[(64, 4, 64, None), (64, 4, 16, 512), (64, 1, 4, 256)], seed=35, stats=True),
    "stats_paged_fp16": dict(B=2, TQ=70, T=1024, H=4, HKV=2, D=64, dtype="fp16", sink=32, sw=128, second_k=128,
                             stages=[(64, 4, 32, None), (64, 1, 8, 256)], seed=36, page=16, ext=1536, stats=True),
    "stats_paged_decode_fp16": dict(B=2, TQ=1, T=1024, H=4, HKV=2, D=64, dtype="fp16", sink=32, sw=128, second_k=128,
                                    stages=[(64, 4, 32, None), (64, 1, 8, 256)], seed=37, page=16, ext=1536, stats=True),
    # benchmark configuration 1 shape (fp32, 4096 x 4096, 8/2 heads, D 64)
    "config1_fp32": dict(B=1, TQ=4096, T=4096, H=8, HKV=2, D=64, dtype="fp32", sink=64, sw=256,
                         second_k=512, stages=[(64, 4, 32, None), (64, 1, 8, 1024)], seed=101,
                         rope_theta=10000.0, out_row_stride=16),
}


def torch_dtype(name: str) -> torch.dtype:
    return _DT[name]


def rope_tables(T: int, D: int, theta: float):
    """cos/sin tables [T, D] with the half-dimension frequencies repeated (rotate-half convention)."""
    inv = 1.0 / (theta ** (np.arange(0, D, 2, dtype=np.float64) / D))
    ang = np.arange(T, dtype=np.float64)[:, None] * inv[None, :]
    ang = np.concatenate([ang, ang], axis=-1)
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def apply_rope(x: np.ndarray, pos: np.ndarray, theta: float) -> np.ndarray:
    """x [B, T, H, D] fp32, pos [B, T] -> rotated x (rotate-half)."""
    D = x.shape[-1]
    cos, sin = rope_tables(int(pos.max()) + 1, D, theta)
    c = cos[pos][:, :, None, :]
    s = sin[pos][:, :, None, :]
    xr = np.concatenate([-x[..., D // 2:], x[..., : D // 2]], axis=-1)
    return (x * c + xr * s).astype(np.float32)


def default_positions(c) -> np.ndarray:
    B, TQ, T = c["B"], c["TQ"], c["T"]
    if "pos_offsets" in c:
        return np.stack([np.arange(TQ) + o for o in c["pos_offsets"]]).astype(np.int64)
    return np.broadcast_to(np.arange(TQ) + (T - TQ), (B, TQ)).astype(np.int64).copy()


def make_inputs(name: str):
    """Return (q, k, v, position_ids, case) as torch CPU tensors in the case dtype.

    q is already multiplied by D**-0.5 (the operator applies no softmax scale itself).
    """
    c = CASES[name]
    B, TQ, T, H, HKV, D = c["B"], c["TQ"], c["T"], c["H"], c["HKV"], c["D"]
    rs = np.random.RandomState(c["seed"])
    q = rs.standard_normal((B, TQ, H, D)).astype(np.float32)
    k = rs.standard_normal((B, T, HKV, D)).astype(np.float32)
    v = rs.standard_normal((B, T, HKV, D)).astype(np.float32)
    pos = default_positions(c)
    if c.get("quant"):
        q = np.clip(np.round(q * 4) / 4, -2, 2)
        k = np.clip(np.round(k * 4) / 4, -2, 2)
        v = np.clip(np.round(v * 4) / 4, -2, 2)
    if "rope_theta" in c and "rope_in_kernel" not in c:
        q = apply_rope(q, pos, c["rope_theta"])
        kpos = np.broadcast_to(np.arange(T), (B, T))
        k = apply_rope(k, kpos, c["rope_theta"])
    q = q * np.float32(D ** -0.5)
    dt = torch_dtype(c["dtype"])
    kt, vt = torch.from_numpy(k), torch.from_numpy(v)
    if c.get("kv_fp8"):
        kt, vt = kt.to(torch.float8_e5m2).float(), vt.to(torch.float8_e5m2).float()
    return (torch.from_numpy(q).to(dt), kt.to(dt), vt.to(dt), torch.from_numpy(pos), c)


def make_paged(k: torch.Tensor, v: torch.Tensor, page: int, seed: int, extra_pages: int = 7):
    """Scatter dense k, v [B, T, HKV, D] into a randomly permuted page pool.

    Returns (k_cache, v_cache [n_pages, page, HKV, D], block_table [B, T // page] int64).
    Pages not referenced by the table hold unrelated random values.
    """
    B, T, HKV, D = k.shape
    assert T % page == 0
    n_used = B * T // page
    n_pages = n_used + extra_pages
    rs = np.random.RandomState(seed + 1000)
    perm = torch.from_numpy(rs.permutation(n_pages)[:n_used].astype(np.int64)).view(B, T // page)
    kc = torch.from_numpy(rs.standard_normal((n_pages, page, HKV, D)).astype(np.float32)).to(k.dtype)
    vc = torch.from_numpy(rs.standard_normal((n_pages, page, HKV, D)).astype(np.float32)).to(v.dtype)
    kc[perm] = k.view(B, T // page, page, HKV, D)
    vc[perm] = v.view(B, T // page, page, HKV, D)
    return kc, vc, perm
