"""Multi-GPU forms of the operator (one process per GPU, ``torch.distributed``).

Two partitionings, both absent from the reference (it runs on one GPU; tensor parallelism is left to
the serving framework, ``src/hip_attn/v1_2/paged_hip.py:14-22``):

* KV-head parallel prefill / decode: a rank owns ``HKV / world`` KV heads and their query heads.
  The only coupling between heads is the head max-reduce of the chunk scores
  (``attention_extend.py:2566-2570``), so every scan stage is followed by one MAX all-reduce of the
  int32 score images and the result is bit-identical to the single-GPU mask.
* Sequence-sharded decode: the key sequence is cut into equal logical shards; each shard is an
  ordinary operator call on its slice (sink only in the first shard, sliding window only in the last)
  that also returns its base-2 log-sum-exp; the partial outputs are all-gathered and merged
  (``attention_decode_bsa.py:1192-1225``).  The number of logical shards is fixed by the caller, so the
  result does not depend on how many GPUs execute them.
"""
from __future__ import annotations

import copy
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
from torch import Tensor

from .metadata import HiPAttentionArgs, HiPAttentionOutputMetadata


def kv_head_slice(rank: int, world: int, H: int, HKV: int) -> Tuple[slice, slice]:
    """Query-head and KV-head slices owned by ``rank``."""
    if HKV % world:
        raise ValueError(f"{HKV} KV heads cannot be split over {world} ranks")
    per = HKV // world
    g = H // HKV
    return slice(rank * per * g, (rank + 1) * per * g), slice(rank * per, (rank + 1) * per)


def make_score_reduce(group=None):
    """MAX all-reduce of the head-reduced score images; a no-op for a single rank."""
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return None

    def reduce(score: Tensor) -> None:
        dist.all_reduce(score, op=dist.ReduceOp.MAX, group=group)

    return reduce


def hip_attention_12_kv_head_parallel(q_local: Tensor, k_local: Optional[Tensor], v_local: Optional[Tensor],
                                      args: HiPAttentionArgs,
                                      cached_metadata: Optional[HiPAttentionOutputMetadata] = None, group=None,
                                      timer=None):
    """Operator call on this rank's heads; masks agree with a single-GPU call over all heads.

    ``q_local`` [B, TQ, H / world, D], ``k_local`` / ``v_local`` [B, TK, HKV / world, D] (or a paged
    cache holding this rank's KV heads in ``args``).  Returns this rank's ``(context, metadata)``.
    """
    from .operator import hip_attention_impl
    return hip_attention_impl(q_local, k_local, v_local, args, cached_metadata, score_reduce=make_score_reduce(group),
                              timer=timer)


def sequence_shard_args(args: HiPAttentionArgs, shard: int, n_shards: int, shard_len: int, per_shard_k: int,
                        device, owns_window: Optional[bool] = None) -> HiPAttentionArgs:
    """Arguments of the operator call that covers logical shard ``shard`` of a decode step.  The sink belongs to
    shard 0, the sliding window to the last shard (``owns_window`` overrides that: with a partly filled sequence
    it is the last shard that holds keys)."""
    a = copy.copy(args)
    a.second_stage_k = per_shard_k
    a.sink_token_size = args.sink_token_size if shard == 0 else 0
    if owns_window is None:
        owns_window = shard == n_shards - 1
    a.sliding_window_size = args.sliding_window_size if owns_window else 0
    a.position_ids = None
    a.extend_context_length = shard_len
    # the flash-decode path of the reference cannot run without a sink (it divides by the number of
    # sink splits, attention_decode_bsa.py:1076, 513); this build has no such limit and keeps decode on
    a.update_flags()
    return a


def merge_shard_partials(outs: Tensor, lses: Tensor, dtype: torch.dtype) -> Tensor:
    """outs [S, B, 1, H, D] fp32 normalised partials, lses [S, B, 1, H] base-2 -> merged [B, 1, H, D]."""
    import ctypes as C
    from . import _lib as L
    from .operator import _DT, _stream
    lib = L.load()
    S, B, TQ, H, D = outs.shape
    po = outs.permute(1, 2, 3, 0, 4).contiguous()  # [B, 1, H, S, D]
    pl = lses.permute(1, 2, 3, 0).contiguous()     # [B, 1, H, S]
    out = torch.empty((B, TQ, H, D), dtype=dtype, device=outs.device)
    L.check(lib.hipattn_merge_partials(po.data_ptr(), pl.data_ptr(), B * TQ * H, S, D, _DT[dtype], out.data_ptr(), D,
                                       None, _stream(outs.device)), "merge_partials")
    return out


def hip_attention_12_sequence_sharded(q: Tensor, shard_kv: Sequence[Tuple], args: HiPAttentionArgs, *, n_shards: int,
                                      shard_len: int, per_shard_k: int, first_shard: int = 0,
                                      cached: Optional[List] = None, group=None, seq_len: Optional[int] = None):
    """Decode step over a key sequence cut into ``n_shards`` logical shards.

    ``shard_kv`` lists this rank's shards in order, each ``(k, v)`` dense slices [B, live length, HKV, D]
    or ``(k_cache, v_cache, block_table, cache_seq_lens)``; ``first_shard`` is the global index of the
    first one.  Ranks hold ``n_shards / world`` consecutive shards.  ``seq_len`` is the live length of the whole
    sequence (default ``n_shards * shard_len``): the last live shard may be partly filled -- its query position
    and chunk grid follow its live length -- and shards beyond it hold no keys.  The sliding window belongs to
    the last live shard.  Neighbouring full shards without sink and window that address the same page pool run
    as ONE batched operator call (they are independent sequences with identical arguments).  Returns
    ``(context [B, 1, H, D], list of metadata, one entry per operator call)``; passing that list back as
    ``cached`` reuses the masks.
    """
    from .operator import hip_attention_impl
    if q.shape[1] != 1:
        raise ValueError("sequence sharding is a decode path (one query row)")
    B = q.shape[0]
    total = n_shards * shard_len if seq_len is None else int(seq_len)
    if not 0 < total <= n_shards * shard_len:
        raise ValueError(f"seq_len {total} outside (0, {n_shards * shard_len}]")
    last_live = (total - 1) // shard_len
    live = [max(0, min(shard_len, total - (first_shard + j) * shard_len)) for j in range(len(shard_kv))]
    for j, kv in enumerate(shard_kv):
        if len(kv) == 2 and live[j] > 0 and kv[0].shape[1] != live[j]:
            raise ValueError(f"shard {first_shard + j}: dense slice of {kv[0].shape[1]} keys, live length {live[j]}")

    def plain(j):   # a full shard without sink and window on a page pool: can share a call with its neighbours
        s = first_shard + j
        return (len(shard_kv[j]) == 4 and live[j] == shard_len and s != last_live
                and (s != 0 or args.sink_token_size == 0))

    groups, j = [], 0
    while j < len(shard_kv):
        e = j + 1
        if plain(j):
            while e < len(shard_kv) and plain(e) and shard_kv[e][0] is shard_kv[j][0] and shard_kv[e][1] is shard_kv[j][1] \
                    and shard_kv[e][2].shape == shard_kv[j][2].shape:
                e += 1
        groups.append((j, e))
        j = e
    outs, lses, mds = [], [], []
    for gi, (j0, j1) in enumerate(groups):
        m = j1 - j0
        if live[j0] == 0:   # beyond the live sequence: an empty partial
            outs.append(torch.zeros((1,) + tuple(q.shape), dtype=torch.float32, device=q.device))
            lses.append(torch.full((1, B, 1, q.shape[2]), float("-inf"), dtype=torch.float32, device=q.device))
            mds.append(None)
            continue
        s = first_shard + j0
        a = sequence_shard_args(args, s, n_shards, live[j0], per_shard_k, q.device, owns_window=s == last_live)
        a.position_ids = torch.full((m * B, 1), live[j0] - 1, dtype=torch.int64, device=q.device)
        kv = shard_kv[j0]
        if len(kv) == 2:
            k, v = kv
            qq = q
        else:
            k = v = None
            a.k_cache, a.v_cache = kv[0], kv[1]
            if m == 1:
                a.block_table, a.cache_seq_lens, qq = kv[2], kv[3], q
            else:
                a.block_table = torch.cat([shard_kv[j][2] for j in range(j0, j1)], 0)
                a.cache_seq_lens = torch.cat([shard_kv[j][3] for j in range(j0, j1)], 0)
                qq = q.repeat(m, 1, 1, 1)
            a.update_flags()
        o, md, lse = hip_attention_impl(qq, k, v, a, None if cached is None else cached[gi], return_lse=True)
        outs.append(o.float().view(m, B, 1, q.shape[2], q.shape[3]))
        lses.append(lse.view(m, B, 1, q.shape[2]))
        mds.append(md)
    po = torch.cat(outs)   # [S_local, B, 1, H, D]
    pl = torch.cat(lses)   # [S_local, B, 1, H]
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        world = dist.get_world_size(group)
        go = torch.empty((world,) + tuple(po.shape), dtype=po.dtype, device=po.device)
        gl = torch.empty((world,) + tuple(pl.shape), dtype=pl.dtype, device=pl.device)
        dist.all_gather_into_tensor(go, po, group=group)
        dist.all_gather_into_tensor(gl, pl, group=group)
        po, pl = go.flatten(0, 1), gl.flatten(0, 1)
    return merge_shard_partials(po, pl, q.dtype), mds
