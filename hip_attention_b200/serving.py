"""Serving-side boundary of the operator: layer configuration, the per-stage mask refresh schedule, the
metadata a decode loop keeps between steps (as plain tensors, or in the preallocated compressed buffers
of ``HiPMetadataCachePool``), and ``forward_paged_hip`` -- the call an inference server makes per attention
layer with its token-granular KV pool.

Mirrors the reference's adapter (``hip_attn/v1_2/hip_config.py``, ``mask_refresh_interval.py``,
``hip_memory_pool.py`` and ``paged_hip.py:327-500``): same class and field names, same JSON keys, same
schedule, same split of a prefill chunk into a sparse part and its last 64 queries, in-kernel RoPE
(``using_extend``, the serving default) included.  Not covered: the host-offload cache.
"""
from __future__ import annotations

import json
import os
from dataclasses import InitVar, dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Union

import torch
from torch import Tensor

from .metadata import (HiPAttentionArgs, HiPAttentionOutputMetadata, HiPAttentionStageInputCache, ScanStage)
from .operator import hip_attention_12


def _default_stages() -> List[ScanStage]:
    """Three stages, chunk 256 / 32 / 8, query block 64 (hip_config.py:7-29)."""
    return [
        ScanStage(stage_block_size_q=64, stage_block_stride_q=4, stage_chunk_size=256, stage_k=None, stage_stride=1),
        ScanStage(stage_block_size_q=64, stage_block_stride_q=4, stage_chunk_size=32, stage_k=32768, stage_stride=1),
        ScanStage(stage_block_size_q=64, stage_block_stride_q=1, stage_chunk_size=8, stage_k=8192, stage_stride=1),
    ]


@dataclass
class HiPAttentionPerLayerConfig:
    """Mask-estimator settings of one kind of layer (hip_config.py:32-63)."""
    second_stage_k: int = 2048
    sliding_window_size: int = 1024
    sink_token_size: int = 256
    sa_extend_backend: str = "streaming"
    scan_extend_backend: Optional[str] = None
    stages: List[ScanStage] = field(default_factory=_default_stages)

    parsed_json: InitVar[Optional[dict]] = None

    def __post_init__(self, parsed_json: Optional[dict]):
        if parsed_json is None:
            return
        rest = dict(parsed_json)
        for key in ("second_stage_k", "sliding_window_size", "sink_token_size", "sa_extend_backend", "scan_extend_backend"):
            if key in rest:
                setattr(self, key, rest.pop(key))
        if "stages" in rest:
            self.stages = [ScanStage(**stage) for stage in rest.pop("stages")]
        if rest:
            raise ValueError(f"Unknown keys in json: {rest.keys()}")


def _default_layers() -> List[HiPAttentionPerLayerConfig]:
    """Entry 0: dense layers (larger k), entry 1: all other layers (hip_config.py:66-81)."""
    return [
        HiPAttentionPerLayerConfig(second_stage_k=4096, sa_extend_backend="streaming", scan_extend_backend="streaming"),
        HiPAttentionPerLayerConfig(second_stage_k=2048, sa_extend_backend="streaming", scan_extend_backend="relative"),
    ]


@dataclass
class HiPAttentionConfig:
    """Model-level configuration, optionally from a JSON string or file (hip_config.py:84-180)."""
    dense_layers: List[int] = field(default_factory=lambda: [0, 1, 2, 3, 31])
    block_sparse_block_size_q: int = 64
    metadata_cache_max_batch_size: int = 32
    mask_refresh_interval: Union[int, List[int]] = field(default_factory=lambda: [32, 16, 8])
    using_extend: bool = True
    layers: List[HiPAttentionPerLayerConfig] = field(default_factory=_default_layers)
    prefill_layers: List[HiPAttentionPerLayerConfig] = field(default_factory=_default_layers)

    # deprecated switches, kept so that existing configuration files load
    apply_v_dot: bool = False
    prefill_always_dense: bool = False
    decode_always_dense: bool = False
    force_dense: bool = False
    prefill_dense_threshold: int = 8192

    json_or_path: InitVar[Optional[str]] = None

    def __post_init__(self, json_or_path: Optional[str]):
        if json_or_path is None:
            parsed = {}
        elif json_or_path.startswith("{"):
            parsed = json.loads(json_or_path)
        else:
            with open(json_or_path, "r") as f:
                parsed = json.load(f)
        for key in ("apply_v_dot", "dense_layers", "prefill_always_dense", "decode_always_dense", "force_dense",
                    "prefill_dense_threshold", "block_sparse_block_size_q", "metadata_cache_max_batch_size", "using_extend"):
            if key in parsed:
                setattr(self, key, parsed.pop(key))
        if "mask_refresh_interval" in parsed:
            if not isinstance(parsed["mask_refresh_interval"], (int, list)):
                raise AssertionError("mask_refresh_interval must be an int or a list of ints")
            self.mask_refresh_interval = parsed.pop("mask_refresh_interval")
        if "layers" in parsed:
            self.layers = [HiPAttentionPerLayerConfig(parsed_json=layer) for layer in parsed.pop("layers")]
        if self.prefill_layers is None:
            self.prefill_layers = self.layers
        if "prefill_layers" in parsed:
            self.prefill_layers = [HiPAttentionPerLayerConfig(parsed_json=layer) for layer in parsed.pop("prefill_layers")]
        if parsed:
            raise ValueError(f"Unknown keys in json: {parsed.keys()}")
        num_stages = len(self.layers[0].stages)
        for layer_config in self.layers:
            if len(layer_config.stages) != num_stages:
                raise AssertionError("all layers must have the same number of stages")
        if isinstance(self.mask_refresh_interval, int):
            self.mask_refresh_interval = [self.mask_refresh_interval] * num_stages

    def layer_config(self, layer_id: int, is_decode: bool) -> HiPAttentionPerLayerConfig:
        """Two entries mean (dense layers, other layers); otherwise one entry per layer (paged_hip.py:358-370)."""
        table = self.layers if is_decode else self.prefill_layers
        if len(table) == 2:
            return table[0 if layer_id in self.dense_layers else 1]
        return table[layer_id]


class HiPMaskRefreshState:
    """Which part of the mask a decode step re-estimates (mask_refresh_interval.py:4-30).

    ``update()`` returns -1 on the first step (estimate everything, nothing cached yet), the index i of the first
    stage whose interval divides the step counter (stages before i keep their cached inputs, the estimator restarts
    at stage i; 0 means from scratch), or None (reuse the cached mask)."""

    def __init__(self, hip_config: HiPAttentionConfig):
        self.hip_config = hip_config
        self.decode_index = 0

    def update(self) -> Optional[int]:
        cached_stages = None
        intervals = self.hip_config.mask_refresh_interval
        if intervals is not None:
            for i_stage, interval in enumerate(intervals):
                if self.decode_index % interval == 0:
                    cached_stages = i_stage
                    break
        if self.decode_index == 0:
            cached_stages = -1
        self.decode_index += 1
        return cached_stages


class HiPMetadataCache:
    """The metadata of the last estimate of one layer and the view of it a step may reuse
    (the selection rules of hip_memory_pool.py:239-300, without the pool's preallocated compressed buffers)."""

    def __init__(self, n_stages: int):
        self.n_stages = n_stages
        self.metadata: Optional[HiPAttentionOutputMetadata] = None

    def set(self, metadata: HiPAttentionOutputMetadata) -> None:
        """Store the metadata a call returned.  A call on a cached mask returns no stage inputs: the ones already
        stored stay (the reference's pool keeps one buffer per stage and only overwrites what was recomputed)."""
        if metadata.stage_caches is None and self.metadata is not None:
            metadata = HiPAttentionOutputMetadata(
                indices=metadata.indices, ks=metadata.ks, ks_count=metadata.ks_count, ks_start_end=metadata.ks_start_end,
                mask_cache_statistics=metadata.mask_cache_statistics, sa_cache_statistics=metadata.sa_cache_statistics,
                stage_caches=self.metadata.stage_caches)
        self.metadata = metadata

    def get(self, cached_stages: Optional[int]) -> Optional[HiPAttentionOutputMetadata]:
        md = self.metadata
        if cached_stages == -1 or md is None:
            return None
        if cached_stages is None or cached_stages == self.n_stages:
            return HiPAttentionOutputMetadata(indices=md.indices, ks=md.ks, ks_count=md.ks_count, ks_start_end=md.ks_start_end,
                                              mask_cache_statistics=None, sa_cache_statistics=None, stage_caches=None)
        if cached_stages == 0:
            return None     # re-estimate from scratch
        caches = [HiPAttentionStageInputCache(indices_left=None, indices_right=None, out_scores=None)]
        caches += list(md.stage_caches[1:cached_stages + 1])
        return HiPAttentionOutputMetadata(indices=None, ks=None, ks_count=None, ks_start_end=None,
                                          mask_cache_statistics=None, sa_cache_statistics=None, stage_caches=caches)


class _PoolBuffer:
    """One preallocated buffer of the metadata pool (hip_memory_pool.py:20-53): ``per_head`` buffers are
    [max_batch * heads, ...] and sliced by batch * heads rows, the others are [max_batch, 1, heads, ...]; values are
    stored in ``store`` and handed back as fresh tensors of ``dtype``."""

    def __init__(self, max_batch: int, heads: int, tail: Sequence[int], dtype: torch.dtype, per_head: bool, store: Optional[torch.dtype],
                 device) -> None:
        lead = (max_batch * heads,) if per_head else (max_batch, 1, heads)
        self.buffer = torch.zeros((*lead, *tail), dtype=store or dtype, device=device)
        self.dtype, self.per_head = dtype, per_head

    def _check(self, rows: int, what: str) -> None:
        if self.buffer.shape[0] < rows:
            raise ValueError(f"the metadata pool holds {self.buffer.shape[0]} rows, {what} needs {rows}: lower the CUDA-graph batch size or "
                             'raise "metadata_cache_max_batch_size" in the attention configuration')

    def get(self, batch_size: int, heads: int) -> Tensor:
        # (the reference compares the batch size with the row count even where rows are batch x head, and then hands
        # back a silently truncated slice; here a batch beyond the configured maximum is an error in both layouts)
        self._check(batch_size * heads if self.per_head else batch_size, "the requested batch")
        view = self.buffer[:batch_size * heads] if self.per_head else self.buffer[:batch_size, :, :heads]
        return view.to(self.dtype, copy=True)

    def set(self, value: Tensor) -> None:
        self._check(value.shape[0], "the stored value")
        dst = self.buffer[:value.shape[0]] if self.per_head else self.buffer[:value.shape[0], :, :value.shape[2]]
        dst.copy_(value.to(self.buffer.dtype))


class HiPMetadataCachePool:
    """Preallocated per-layer buffers that carry the mask and the stage inputs of decode steps from one step to the
    next at fixed addresses, so that a captured CUDA graph can replay them (hip_memory_pool.py:55-433).

    Block indices and chunk bounds are stored as uint32 and the stage scores as bfloat16, as the reference stores
    them: a mask that went through the pool has its INT64_MAX padding replaced by 2^32 - 1 (still beyond every
    token, and ``ks`` bounds the entries that count), and an estimator restart sees scores rounded to bfloat16.
    ``set_hip_metadata_cache`` / ``get_hip_metadata_cache`` take the same arguments as the reference's.  The
    research switches that enlarge or delay the buffers (HIP_DEBUG_UNION_HEAD, HIP_DIAG_INFO,
    HIP_DEBUG_ADD_DELAY_WINDOW, HIP_DEBUG_DELAYED_STAGE0) are not built."""

    _COUNTERS = ("access_count", "unique_access_count", "cache_miss_count")

    def __init__(self, max_total_num_tokens: int, query_head_num: int, layer_num: int, context_length: int, device,
                 hip_config: HiPAttentionConfig) -> None:
        self.hip_config, self.layer_num, self.head_num, self.device = hip_config, layer_num, query_head_num, device
        self.max_batch_size = hip_config.metadata_cache_max_batch_size
        self.layer_configs = {i: hip_config.layer_config(i, is_decode=True) for i in range(layer_num)}
        self.cache: List[Dict[str, _PoolBuffer]] = []
        for i in range(layer_num):
            layer = self.layer_configs[i]

            def buf(tail, dtype, per_head=True, store=None):
                return _PoolBuffer(self.max_batch_size, self.head_num, tail, dtype, per_head, store, device)

            n_blocks = -(-layer.second_stage_k // layer.stages[-1].stage_chunk_size)
            bufs = {"indices": buf([1, n_blocks], torch.int64, store=torch.uint32), "ks": buf([1], torch.int64),
                    "ks_count": buf([1, 1], torch.int64), "ks_start_end": buf([1, 2], torch.int64)}
            for prefix in ("mask", "sa"):
                for c in self._COUNTERS:
                    bufs[f"{prefix}_{c}"] = buf([1], torch.int64)
            reach = context_length - layer.sliding_window_size - layer.sink_token_size
            for i_stage, stage in enumerate(layer.stages):
                if i_stage == 0:
                    continue
                n = min(stage.stage_k, reach) // stage.stage_chunk_size
                bufs[f"stage_{i_stage}_indices_left"] = buf([n], torch.int64, per_head=False, store=torch.uint32)
                bufs[f"stage_{i_stage}_indices_right"] = buf([n], torch.int64, per_head=False, store=torch.uint32)
                bufs[f"stage_{i_stage}_out_scores"] = buf([n], torch.float32, per_head=False, store=torch.bfloat16)
            self.cache.append(bufs)
        self.allocated_gpu_bytes = self.compute_allocated_bytes()

    def reset_decode_phase(self) -> None:
        """Called by the server when a decode phase starts; only the delayed-stage research mode keeps state there."""

    def compute_allocated_bytes(self) -> int:
        return sum(b.buffer.numel() * b.buffer.element_size() for layer in self.cache for b in layer.values())

    def _buffer(self, layer_idx: int, name: str) -> _PoolBuffer:
        if layer_idx not in range(len(self.cache)):
            raise IndexError(f"layer {layer_idx} is not in range({len(self.cache)})")
        if name not in self.cache[layer_idx]:
            raise KeyError(f"{name} is not one of {sorted(self.cache[layer_idx])}")
        return self.cache[layer_idx][name]

    def get_buffer(self, layer_idx: int, name: str, batch_size: int) -> Tensor:
        return self._buffer(layer_idx, name).get(batch_size, self.head_num)

    def set_buffer(self, layer_idx: int, name: str, value: Tensor) -> None:
        self._buffer(layer_idx, name).set(value)

    def get_hip_metadata_cache(self, layer_id: int, size: int, batch_size: int,
                               cached_stages: Optional[int]) -> Optional[HiPAttentionOutputMetadata]:
        """What a step may reuse: the mask (``cached_stages`` None or the number of stages), nothing (0, or -1 for the
        first step), or the inputs of stages 1 .. cached_stages, from which the estimator restarts."""
        if size != batch_size:
            raise ValueError("the pool serves decode steps: one query token per request")
        n_stages = len(self.layer_configs[layer_id].stages)
        if cached_stages is None or cached_stages == n_stages:
            return HiPAttentionOutputMetadata(
                indices=self.get_buffer(layer_id, "indices", batch_size), ks=self.get_buffer(layer_id, "ks", batch_size),
                ks_count=self.get_buffer(layer_id, "ks_count", batch_size), ks_start_end=self.get_buffer(layer_id, "ks_start_end", batch_size),
                mask_cache_statistics=None, sa_cache_statistics=None, stage_caches=None)
        if cached_stages <= 0:
            return None
        caches = [HiPAttentionStageInputCache(indices_left=None, indices_right=None, out_scores=None)]
        for i_stage in range(1, cached_stages + 1):
            caches.append(HiPAttentionStageInputCache(
                indices_left=self.get_buffer(layer_id, f"stage_{i_stage}_indices_left", batch_size),
                indices_right=self.get_buffer(layer_id, f"stage_{i_stage}_indices_right", batch_size),
                out_scores=self.get_buffer(layer_id, f"stage_{i_stage}_out_scores", batch_size)))
        return HiPAttentionOutputMetadata(indices=None, ks=None, ks_count=None, ks_start_end=None, mask_cache_statistics=None,
                                          sa_cache_statistics=None, stage_caches=caches)

    def set_hip_metadata_cache(self, layer_id: int, size: int, batch_size: int, metadata: HiPAttentionOutputMetadata) -> None:
        """Store what a step returned.  Stage inputs are only overwritten when the step recomputed them."""
        if size != batch_size:
            raise ValueError("the pool serves decode steps: one query token per request")
        for name in ("indices", "ks", "ks_count", "ks_start_end"):
            self.set_buffer(layer_id, name, getattr(metadata, name))
        for prefix, stats in (("sa", metadata.sa_cache_statistics), ("mask", metadata.mask_cache_statistics)):
            counts = stats.compute_statistics() if stats is not None else {}
            for c in self._COUNTERS:
                v = counts.get(c)
                v = torch.zeros((1,), dtype=torch.int64, device=self.device) if v is None else v
                self.set_buffer(layer_id, f"{prefix}_{c}", v.view(1, 1).expand(self.max_batch_size, 1))
        for i_stage, cache in enumerate(metadata.stage_caches or []):
            if i_stage == 0:
                continue
            self.set_buffer(layer_id, f"stage_{i_stage}_indices_left", cache.indices_left)
            self.set_buffer(layer_id, f"stage_{i_stage}_indices_right", cache.indices_right)
            self.set_buffer(layer_id, f"stage_{i_stage}_out_scores", cache.out_scores)

    def compute_cache_statistics(self, batch_size: int) -> dict:
        """Access / miss totals over all layers and the hit ratio (0 / 0 when the steps gathered no statistics)."""
        result = {}
        for prefix in ("sa", "mask"):
            access = sum(self.get_buffer(i, f"{prefix}_access_count", batch_size).sum() for i in range(self.layer_num))
            miss = sum(self.get_buffer(i, f"{prefix}_cache_miss_count", batch_size).sum() for i in range(self.layer_num))
            result.update({f"{prefix}_access": access, f"{prefix}_miss": miss, f"{prefix}_hit_ratio": 1 - (miss / access)})
        return result


LAST_DENSE = 64   # queries at the end of a prefill chunk that attend a near-full window (paged_hip.py:462)


def cuda_graph_capture_configs(hip_config: HiPAttentionConfig):
    """The ``(num_stage_cached,)`` variants of a decode step a server captures as CUDA graphs
    (``paged_hip.py:27-32``): the whole mask cached (``None``) and one entry per stage the estimator may
    restart from."""
    configs = [(None,)]
    for i_stage in range(len(hip_config.layers[0].stages)):
        configs.append((i_stage,))
    return configs


def forward_paged_hip(query: Tensor, sm_scale: float, batch_size: int, k_cache: Optional[Tensor], v_cache: Optional[Tensor],
                      offload_cache: Any, positions: Tensor, seq_lens: Tensor, req_to_tokens: Tensor,
                      req_pool_indices: Tensor, rope_cos: Optional[Tensor], rope_sin: Optional[Tensor], layer_id: int,
                      logit_cap: float, orig_context_len: int, max_context_len: int, is_prefill: bool,
                      hip_config: HiPAttentionConfig, cached_metadata: Optional[HiPAttentionOutputMetadata] = None,
                      k: Optional[Tensor] = None, v: Optional[Tensor] = None, online_update_cache: bool = False,
                      offloading_metadata: Any = None, is_decode: bool = False, query_for_mask: Optional[Tensor] = None,
                      diag_sliding_window_indices: Optional[Tensor] = None):
    """One attention layer of a serving step; parameter list and order of the reference's
    ``forward_paged_hip`` (``paged_hip.py:35-62``, body ``:327-500``), so positional callers keep working.

    ``query`` [N, H, D] holds ``batch_size`` requests of N / batch_size tokens each; ``k_cache`` / ``v_cache``
    [tokens, HKV, D] are the server's token-granular pools (page size 1; a ``float8_e5m2`` pool is read as such)
    and ``req_to_tokens[req_pool_indices]`` the per-request token tables; ``k`` / ``v`` [B, T, HKV, D] may be given
    instead (padded to ``max_context_len``).  ``rope_cos`` / ``rope_sin`` are used when the configuration has
    ``using_extend`` set.  Decode steps and short chunks are one operator call.  A prefill chunk of 128 tokens or
    more is split: all but the last 64 queries run with the layer's window, the last 64 with the window sentinel
    777, which the operator turns into (model context - sink - second_stage_k - query block) so that they see
    nearly everything.  ``is_prefill`` only selects what the reference validates against its offload cache and is
    otherwise unused, as there.  Not built (rejected): ``offload_cache``, ``online_update_cache``,
    ``offloading_metadata``, ``diag_sliding_window_indices``.
    Returns (context [B, tokens, H, D], metadata of the last call)."""
    if offload_cache is not None or online_update_cache or offloading_metadata is not None:
        raise NotImplementedError("the host-offload cache (offload_cache / online_update_cache / offloading_metadata) is not built")
    if diag_sliding_window_indices is not None:
        raise NotImplementedError("diag_sliding_window_indices is not built")
    N, num_heads, hidden = query.shape
    if N % batch_size:
        raise ValueError(f"{N} query tokens are not a multiple of the batch size {batch_size}")
    dst_len = N // batch_size
    if is_decode and dst_len != 1:
        raise ValueError("a decode step has one query token per request")
    layer = hip_config.layer_config(layer_id, is_decode)
    is_dense = layer_id in hip_config.dense_layers
    query = query.view(batch_size, dst_len, num_heads, hidden)
    if query_for_mask is not None:
        query_for_mask = query_for_mask.view(batch_size, -1, num_heads, hidden)
    if k is not None and k.shape[1] != max_context_len:
        pad_k = torch.zeros((k.shape[0], max_context_len, k.shape[2], k.shape[3]), dtype=k.dtype, device=k.device)
        pad_v = torch.zeros_like(pad_k)
        pad_k[:, :k.shape[1]] = k
        pad_v[:, :v.shape[1]] = v
        k, v = pad_k, pad_v
    if k_cache is not None:
        if v_cache.shape != k_cache.shape or k_cache.shape[-1] != hidden:
            raise ValueError("k_cache and v_cache must be [tokens, kv_heads, head_dim] pools of q's head_dim")
        k_cache = k_cache.view(k_cache.shape[0], 1, k_cache.shape[1], hidden)
        v_cache = v_cache.view(v_cache.shape[0], 1, v_cache.shape[1], hidden)
    elif k is None:
        raise ValueError("neither k_cache nor k was given")
    block_table = req_to_tokens.index_select(0, req_pool_indices)
    if block_table.shape[0] != batch_size:
        raise ValueError("req_pool_indices must name one request per batch entry")
    head_dim = k_cache.shape[-1] if k_cache is not None else k.shape[-1]
    # statistics are gathered whenever the mask is (re)estimated (paged_hip.py:399-405)
    require_stats = (cached_metadata is None or cached_metadata.indices is None
                     or os.getenv("HIP_DISABLE_COMPUTE_STATISTICS", "1") == "0")
    scan_backend = layer.scan_extend_backend
    if scan_backend is None:   # paged_hip.py:433-441
        scan_backend = "relative" if hip_config.apply_v_dot else ("streaming" if is_dense else "relative")

    def make_args(position_ids: Tensor, window: int) -> HiPAttentionArgs:
        return HiPAttentionArgs(
            k_cache=k_cache, v_cache=v_cache, block_table=block_table, cache_seq_lens=seq_lens, position_ids=position_ids,
            block_size_k=32 if head_dim > 128 else 64, sliding_window_size=window, sink_token_size=layer.sink_token_size,
            using_extend=hip_config.using_extend, need_apply_rope=hip_config.using_extend, rope_cos=rope_cos, rope_sin=rope_sin,
            logit_softcap=logit_cap if logit_cap != 0.0 else None,
            second_stage_k=layer.second_stage_k, stages=layer.stages, model_context_length=orig_context_len,
            extend_context_length=max_context_len, block_sparse_block_size_q=hip_config.block_sparse_block_size_q,
            scan_extend_backend=scan_backend, sa_extend_backend=layer.sa_extend_backend,
            require_cache_statistics=require_stats, disable_flashdecode=not is_decode,
            q_mask=(query_for_mask * sm_scale).to(query.dtype) if query_for_mask is not None else None, layer_id=layer_id)

    pos = positions.view(batch_size, dst_len)
    if is_decode or dst_len < 2 * LAST_DENSE:
        context, metadata = hip_attention_12((query * sm_scale).to(query.dtype), k, v, args=make_args(pos, layer.sliding_window_size),
                                             cached_metadata=cached_metadata)
        return context.to(query.dtype), metadata
    if query_for_mask is not None:
        raise ValueError("query_for_mask cannot be combined with the split of a prefill chunk")
    sparse, _ = hip_attention_12((query[:, :-LAST_DENSE] * sm_scale).to(query.dtype), k, v,
                                 args=make_args(pos[:, :-LAST_DENSE], layer.sliding_window_size), cached_metadata=cached_metadata)
    dense, metadata = hip_attention_12((query[:, -LAST_DENSE:] * sm_scale).to(query.dtype), k, v,
                                       args=make_args(pos[:, -LAST_DENSE:], 777), cached_metadata=cached_metadata)
    return torch.cat([sparse.to(query.dtype), dense.to(query.dtype)], dim=1), metadata
