"""Serving-side adapter: configuration, refresh schedule and metadata-cache rules against fixtures recorded from the
reference's own modules (tests/golden/gen_serving.py); the paged forward call against the reference's outputs on a B200."""
import json
import os

import numpy as np
import pytest
import torch

GOLD = os.path.join(os.path.dirname(__file__), "golden")
import sys
sys.path.insert(0, GOLD)
import gen_serving as G  # noqa: E402  (inputs and JSON strings of the fixtures; imports nothing of the reference at import time)


def _record():
    with open(os.path.join(GOLD, "serving_config.json")) as f:
        return json.load(f)


def _as_record(cfg):
    return json.loads(json.dumps(G.config_record(cfg)))


@pytest.mark.parametrize("name", list(G.CONFIG_JSONS))
def test_config_parses_like_the_reference(name):
    from hip_attention_b200 import HiPAttentionConfig
    assert _as_record(HiPAttentionConfig(json_or_path=G.CONFIG_JSONS[name])) == _record()["configs"][name]


@pytest.mark.parametrize("name", list(G.BAD_JSONS))
def test_config_rejects_what_the_reference_rejects(name):
    from hip_attention_b200 import HiPAttentionConfig
    expected = _record()["bad"][name]
    assert expected is not None
    with pytest.raises(Exception) as e:
        HiPAttentionConfig(json_or_path=G.BAD_JSONS[name])
    assert type(e.value).__name__ == expected


def test_config_from_file(tmp_path):
    from hip_attention_b200 import HiPAttentionConfig
    p = tmp_path / "hip.json"
    p.write_text(G.CONFIG_JSONS["custom_layers"])
    assert _as_record(HiPAttentionConfig(json_or_path=str(p))) == _record()["configs"]["custom_layers"]


@pytest.mark.parametrize("name", list(G.SCHEDULES))
def test_refresh_schedule(name):
    from hip_attention_b200 import HiPAttentionConfig, HiPMaskRefreshState
    st = HiPMaskRefreshState(HiPAttentionConfig(json_or_path=G.CONFIG_JSONS[name]))
    assert [st.update() for _ in range(70)] == _record()["schedules"][name]


def test_layer_selection():
    from hip_attention_b200 import HiPAttentionConfig
    cfg = HiPAttentionConfig(json_or_path=G.CONFIG_JSONS["custom_layers"])
    cfg.dense_layers = [0, 3]
    assert cfg.layer_config(3, True) is cfg.layers[0] and cfg.layer_config(7, True) is cfg.layers[1]
    assert cfg.layer_config(7, False) is cfg.prefill_layers[1]


def test_metadata_cache_rules():
    """What a step may reuse for each value of the schedule (hip_memory_pool.py:239-300)."""
    from hip_attention_b200 import (HiPAttentionOutputMetadata, HiPAttentionStageInputCache, HiPMetadataCache)
    t = lambda v: torch.tensor([v])   # noqa: E731
    caches = [HiPAttentionStageInputCache(None, None, None)] + [HiPAttentionStageInputCache(t(i), t(10 + i), t(20 + i)) for i in (1, 2)]
    md = HiPAttentionOutputMetadata(indices=t(1), ks=t(2), ks_count=t(3), ks_start_end=t(4), mask_cache_statistics=None,
                                    sa_cache_statistics=None, stage_caches=caches)
    c = HiPMetadataCache(n_stages=3)
    assert c.get(None) is None                       # nothing stored yet
    c.set(md)
    assert c.get(-1) is None and c.get(0) is None    # first step / restart from scratch
    full = c.get(None)
    assert full.indices is md.indices and full.stage_caches is None
    assert c.get(3).indices is md.indices             # "all stages cached" = the whole mask
    part = c.get(1)
    assert part.indices is None and len(part.stage_caches) == 2
    assert part.stage_caches[0].indices_left is None and part.stage_caches[1] is caches[1]
    assert len(c.get(2).stage_caches) == 3
    # a call on the cached mask returns no stage inputs: the stored ones stay usable
    c.set(HiPAttentionOutputMetadata(indices=t(7), ks=t(2), ks_count=t(3), ks_start_end=t(4), mask_cache_statistics=None,
                                     sa_cache_statistics=None, stage_caches=None))
    assert c.get(None).indices.item() == 7 and c.get(1).stage_caches[1] is caches[1]


@pytest.mark.gpu
def test_forward_paged_hip_matches_the_reference():
    """Prefill chunk (split into a sparse part and its last 64 queries, window sentinel 777), a decode step from
    scratch, one restarting at stage 1 from cached stage inputs and one on the cached mask: masks identical to the
    reference's, outputs within fp16 tolerance."""
    from hip_attention_b200 import HiPAttentionConfig, HiPMetadataCache, forward_paged_hip
    g = np.load(os.path.join(GOLD, "serving_paged.npz"))
    c = G.PAGED
    x = {k_: v_.cuda() for k_, v_ in G.paged_inputs().items()}
    cfg = HiPAttentionConfig(json_or_path=G.CONFIG_JSONS["custom_layers"])
    T = c["T"]

    def call(q, positions, seq_len, is_decode, cached):
        return forward_paged_hip(q, c["sm_scale"], 1, x["k_pool"], x["v_pool"], positions.cuda(), torch.tensor([seq_len], device="cuda"),
                                 x["req_to_tokens"], x["req_pool_indices"], c["layer_id"], 0.0, c["model_context"], T, cfg,
                                 cached_metadata=cached, is_decode=is_decode)

    tol = 3e-3
    p0 = T - 3 - c["chunk"]
    out, md = call(x["q_prefill"], torch.arange(p0, p0 + c["chunk"]), T - 3, False, None)
    assert np.array_equal(md.indices.cpu().numpy(), g["prefill_indices"]) and np.array_equal(md.ks.cpu().numpy(), g["prefill_ks"])
    assert np.abs(out.float().cpu().numpy() - g["prefill_out"]).max() < tol
    cache = HiPMetadataCache(n_stages=2)
    out0, md0 = call(x["q_decode"][0], torch.tensor([T - 3]), T - 2, True, cache.get(-1))
    cache.set(md0)
    assert np.array_equal(md0.indices.cpu().numpy(), g["decode0_indices"]) and np.array_equal(md0.ks.cpu().numpy(), g["decode0_ks"])
    assert np.abs(out0.float().cpu().numpy() - g["decode0_out"]).max() < tol
    out1, md1 = call(x["q_decode"][1], torch.tensor([T - 2]), T - 1, True, cache.get(1))
    cache.set(md1)
    assert np.array_equal(md1.indices.cpu().numpy(), g["decode1_indices"]) and np.array_equal(md1.ks.cpu().numpy(), g["decode1_ks"])
    assert np.abs(out1.float().cpu().numpy() - g["decode1_out"]).max() < tol
    out2, _ = call(x["q_decode"][2], torch.tensor([T - 1]), T, True, cache.get(None))
    assert np.abs(out2.float().cpu().numpy() - g["decode2_out"]).max() < tol
