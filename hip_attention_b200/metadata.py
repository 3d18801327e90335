"""Argument and result types of ``hip_attention_12``.

Field names, defaults and meanings follow the reference's ``src/hip_attn/v1_2/attention_metadata.py``
(``Stage`` :27-37, ``ScanStage`` :55-60, ``HiPAttentionCacheAccessStatistics`` :77-108,
``HiPAttentionStageInputCache`` :110-115, ``HiPAttentionOutputMetadata`` :117-130, ``HiPAttentionArgs``
:133-260) so that code written against the reference keeps working.  Differences: any positive page
size is accepted (the reference asserts 1..32, :239), and options that belong to the host-offload
cache are rejected by the operator instead of being silently carried.
"""
from __future__ import annotations

import copy
import os
from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Literal, Optional

import torch
from torch import Tensor


@dataclass
class Stage:
    stage_block_size_q: int
    stage_block_stride_q: int
    stage_chunk_size: int
    stage_k: Optional[int]
    stage_stride: int
    require_realign_index: bool = False
    require_reset_score: bool = False
    require_post_sort: bool = False


@dataclass
class ScanStage(Stage):
    stage_extend_backend: Optional[str] = None
    require_realign_index: bool = True
    require_reset_score: bool = True
    require_post_sort: bool = True


@dataclass
class NopStage(Stage):
    require_realign_index: bool = True
    require_reset_score: bool = False
    require_post_sort: bool = True


@dataclass
class EvalScoreStage(Stage):
    block_chunk: int = 64
    stage_extend_backend: Optional[str] = None
    require_reset_score: bool = True
    require_post_sort: bool = True


@dataclass
class EnsembleScoreStage(Stage):
    reduce_method: str = "sum"
    require_reset_score: bool = True
    require_post_sort: bool = True


def _default_stages() -> List[Stage]:
    spec = ((4, 256, None), (4, 32, 32768), (1, 8, 8192))
    return [ScanStage(stage_block_size_q=64, stage_block_stride_q=sq, stage_chunk_size=c, stage_k=k, stage_stride=1)
            for sq, c, k in spec]


@dataclass
class HiPAttentionCacheAccessStatistics:
    access_counter: Optional[Tensor]      # [B, HKV, pages]
    cache_miss_counter: Optional[Tensor]  # [B, HKV, pages]

    def compute_statistics(self) -> Dict[str, Optional[Tensor]]:
        keys = ("unique_access_count", "access_count", "cache_miss_count", "cache_hit_ratio")
        enabled = os.getenv("HIP_DISABLE_COMPUTE_STATISTICS", "1") == "0"
        if not enabled or self.access_counter is None:
            return dict.fromkeys(keys)
        total = self.access_counter.sum()
        miss = self.cache_miss_counter.sum()
        return {
            "unique_access_count": self.access_counter.clamp(0, 1).sum(),
            "access_count": total,
            "cache_miss_count": miss,
            "cache_hit_ratio": 1 - (miss / total),
        }


@dataclass
class HiPAttentionStageInputCache:
    indices_left: Optional[Tensor]   # [B, BDST, H, n] int64
    indices_right: Optional[Tensor]  # [B, BDST, H, n] int64
    out_scores: Optional[Tensor]     # [B, BDST, H, n] fp32


@dataclass
class HiPAttentionOutputMetadata:
    indices: Optional[Tensor]        # [B * H, BDST, K] int64, ascending, padded with INT64_MAX
    ks: Optional[Tensor]             # [B * H, BDST] int64
    ks_count: Optional[Tensor]       # [B * H, BDST, 1] int64
    ks_start_end: Optional[Tensor]   # [B * H, BDST, 2] int32
    mask_cache_statistics: Optional[HiPAttentionCacheAccessStatistics]
    sa_cache_statistics: Optional[HiPAttentionCacheAccessStatistics]
    stage_caches: Optional[List[HiPAttentionStageInputCache]]


@dataclass
class HiPAttentionArgs:
    position_ids: Optional[Tensor] = None

    sink_token_size: int = 256
    sliding_window_size: int = 512
    block_size_k: int = 64   # chunks per scan group
    block_size_q: int = 64   # overwritten by the operator
    mask_k: int = 512        # overwritten by the operator

    second_stage_k: int = 2048
    stages: List[Stage] = field(default_factory=_default_stages)
    model_context_length: int = 131072
    extend_context_length: int = 512 * 1024

    mask_only: bool = False
    block_sparse_block_size_q: Optional[int] = 64

    scan_early_terminate: int = 1
    stage_early_terminate: int = 1
    scan_extend_backend: str = "relative"
    sa_extend_backend: str = "streaming"
    low_percent: float = 0.0
    low_k_ratio: float = 1.0
    dim_to_lower: Literal["head", "seq"] = "head"
    q_mask: Optional[Tensor] = None
    k_mask: Optional[Tensor] = None
    idx_pca_hid_q: Optional[Tensor] = None
    idx_pca_hid_k: Optional[Tensor] = None

    is_causal: bool = True

    using_extend: bool = False
    need_apply_rope: bool = False
    rope_cos: Optional[Tensor] = None
    rope_sin: Optional[Tensor] = None

    offload_cache: Any = None
    k_cache: Optional[Tensor] = None
    v_cache: Optional[Tensor] = None
    cache_seq_lens: Optional[Tensor] = None
    block_table: Optional[Tensor] = None

    logit_softcap: Optional[float] = None
    online_update_cache: bool = False

    require_cache_statistics: bool = True
    require_stage_caches: bool = True
    disable_flashdecode: bool = False
    sliding_window_indices: Optional[Tensor] = None
    layer_id: int = 31

    def __post_init__(self):
        if self.rope_cos is not None and self.rope_cos.ndim == 3:
            self.rope_cos = self.rope_cos.reshape(-1, self.rope_cos.shape[-1])
            self.rope_sin = self.rope_sin.reshape(-1, self.rope_sin.shape[-1])
        self.update_flags()

    def update_flags(self) -> None:
        if self.logit_softcap == 0:
            self.logit_softcap = None
        self.using_paged_cache = self.k_cache is not None or self.offload_cache is not None
        if self.k_cache is not None:
            self.paged_cache_page_count = int(self.k_cache.shape[0])
            self.paged_cache_page_size = int(self.k_cache.shape[1])
            if self.paged_cache_page_size <= 0:
                raise ValueError("k_cache must be [n_pages, page_size, kv_heads, head_dim] with page_size > 0")

    def clone(self) -> "HiPAttentionArgs":
        self.update_flags()
        return copy.copy(self)

    def json(self, convert_tensor_to_meta: bool = True) -> Dict[str, Any]:
        out = {f.name: getattr(self, f.name) for f in fields(self)}
        if convert_tensor_to_meta:
            for key, val in out.items():
                if isinstance(val, Tensor):
                    out[key] = f"{val.dtype}{list(val.shape)}@{val.device}.{val.data_ptr():02X}"
        return out
