"""HiP / InfiniteHiP attention for NVIDIA B200 (sm_100a).

Drop-in for the ``hip_attention_12`` operator of DeepAuto-AI/hip-attention (``src/hip_attn/__init__.py:28-38``):
same call, same argument and metadata types, CUDA kernels behind a C ABI (``include/hipattn.h``).
"""
from .metadata import (EnsembleScoreStage, EvalScoreStage, HiPAttentionArgs, HiPAttentionCacheAccessStatistics,
                       HiPAttentionOutputMetadata, HiPAttentionStageInputCache, NopStage, ScanStage, Stage)
from .operator import PhaseTimer, hip_attention_12, hip_attention_impl, read_status
from .serving import (HiPAttentionConfig, HiPAttentionPerLayerConfig, HiPMaskRefreshState, HiPMetadataCache,
                      HiPMetadataCachePool, cuda_graph_capture_configs, forward_paged_hip)

# the names the reference exports for this generation of the operator
HiPAttentionArgs12 = HiPAttentionArgs
HiPAttentionOutputMetadata12 = HiPAttentionOutputMetadata
HiPAttentionCacheAccessStatistics12 = HiPAttentionCacheAccessStatistics
ScanStage12 = ScanStage
dual_stage_quadratic_hip_attention = hip_attention_12

__all__ = [
    "hip_attention_12", "dual_stage_quadratic_hip_attention", "hip_attention_impl", "read_status", "PhaseTimer",
    "HiPAttentionArgs", "HiPAttentionArgs12", "HiPAttentionOutputMetadata", "HiPAttentionOutputMetadata12",
    "HiPAttentionCacheAccessStatistics", "HiPAttentionCacheAccessStatistics12", "HiPAttentionStageInputCache",
    "Stage", "ScanStage", "ScanStage12", "NopStage", "EvalScoreStage", "EnsembleScoreStage",
    "HiPAttentionConfig", "HiPAttentionPerLayerConfig", "HiPMaskRefreshState", "HiPMetadataCache", "HiPMetadataCachePool",
    "forward_paged_hip", "cuda_graph_capture_configs",
]
