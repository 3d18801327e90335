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
        # positional, in the reference's order (paged_hip.py:35-62)
        return forward_paged_hip(q, c["sm_scale"], 1, x["k_pool"], x["v_pool"], None, positions.cuda(),
                                 torch.tensor([seq_len], device="cuda"), x["req_to_tokens"], x["req_pool_indices"], None, None,
                                 c["layer_id"], 0.0, c["model_context"], T, not is_decode, cfg, cached, None, None, False, None,
                                 is_decode)

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


def _pool(device):
    from hip_attention_b200 import HiPAttentionConfig, HiPMetadataCachePool
    c = G.PAGED
    cfg = HiPAttentionConfig(json_or_path=G.CONFIG_JSONS["custom_layers"])
    return HiPMetadataCachePool(max_total_num_tokens=c["T"] + 77, query_head_num=c["H"], layer_num=c["layer_id"] + 1,
                                context_length=c["T"], device=device, hip_config=cfg), cfg


def test_metadata_pool_stores_and_returns_like_the_reference():
    """The metadata of a decode step goes into the preallocated buffers and comes back as the reference's pool
    returns it: block indices through uint32 (the INT64_MAX padding becomes 2^32 - 1), stage scores through
    bfloat16, fresh tensors on every read, the same buffer sizes."""
    from hip_attention_b200 import HiPAttentionOutputMetadata, HiPAttentionStageInputCache
    g = np.load(os.path.join(GOLD, "serving_pool.npz"))
    pool, cfg = _pool("cpu")
    lid = G.PAGED["layer_id"]
    assert pool.compute_allocated_bytes() == int(g["allocated_bytes"]) == pool.allocated_gpu_bytes
    t = torch.from_numpy
    md = HiPAttentionOutputMetadata(
        indices=t(g["in_indices"]), ks=t(g["in_ks"]), ks_count=t(g["in_ks_count"]), ks_start_end=t(g["in_ks_start_end"]),
        mask_cache_statistics=None, sa_cache_statistics=None,
        stage_caches=[HiPAttentionStageInputCache(None, None, None),
                      HiPAttentionStageInputCache(t(g["in_stage1_left"]), t(g["in_stage1_right"]), t(g["in_stage1_scores"]))])
    assert pool.get_hip_metadata_cache(lid, 1, 1, -1) is None
    pool.set_hip_metadata_cache(lid, 1, 1, md)
    for cached in (None, 2):
        got = pool.get_hip_metadata_cache(lid, 1, 1, cached)
        assert got.stage_caches is None
        for name in ("indices", "ks", "ks_count", "ks_start_end"):
            v = getattr(got, name)
            assert v.dtype == torch.int64 and np.array_equal(v.numpy(), g["mask_" + name]), name
    # padding entries (INT64_MAX) come back as 2^32 - 1
    padded = md.indices.clone()
    padded[:, :, -3:] = torch.iinfo(torch.int64).max
    pool.set_buffer(lid, "indices", padded)
    back = pool.get_buffer(lid, "indices", 1)
    assert torch.equal(back[:, :, :-3], padded[:, :, :-3]) and bool((back[:, :, -3:] == 2 ** 32 - 1).all())
    pool.set_buffer(lid, "indices", md.indices)
    assert pool.get_hip_metadata_cache(lid, 1, 1, 0) is None
    part = pool.get_hip_metadata_cache(lid, 1, 1, 1)
    assert part.indices is None and part.ks is None and len(part.stage_caches) == 2 and part.stage_caches[0].indices_left is None
    s1 = part.stage_caches[1]
    assert np.array_equal(s1.indices_left.numpy(), g["stage1_left"]) and np.array_equal(s1.indices_right.numpy(), g["stage1_right"])
    assert s1.out_scores.dtype == torch.float32 and np.array_equal(s1.out_scores.numpy(), g["stage1_scores"])
    # reads are copies: writing into one does not change the pool
    s1.out_scores.zero_()
    assert np.array_equal(pool.get_hip_metadata_cache(lid, 1, 1, 1).stage_caches[1].out_scores.numpy(), g["stage1_scores"])
    # a step on the cached mask returns no stage inputs: the stored ones stay
    pool.set_hip_metadata_cache(lid, 1, 1, HiPAttentionOutputMetadata(md.indices, md.ks, md.ks_count, md.ks_start_end, None, None, None))
    assert np.array_equal(pool.get_hip_metadata_cache(lid, 1, 1, 1).stage_caches[1].indices_left.numpy(), g["stage1_left"])


def test_metadata_pool_limits_and_errors():
    pool, cfg = _pool("cpu")
    lid = G.PAGED["layer_id"]
    g = np.load(os.path.join(GOLD, "serving_pool.npz"))
    # the reference returns a truncated slice for a per-head buffer read beyond the configured batch (recorded as
    # "none"); the pool here refuses it, as both do for the per-batch buffers
    assert str(g["too_large"]) == "none"
    with pytest.raises(ValueError):
        pool.get_buffer(lid, "ks", cfg.metadata_cache_max_batch_size + 1)
    with pytest.raises(ValueError):
        pool.get_buffer(lid, "stage_1_out_scores", cfg.metadata_cache_max_batch_size + 1)
    assert pool.get_buffer(lid, "ks", cfg.metadata_cache_max_batch_size).shape[0] == cfg.metadata_cache_max_batch_size * G.PAGED["H"]
    with pytest.raises(ValueError):
        pool.set_buffer(lid, "ks", torch.zeros((cfg.metadata_cache_max_batch_size * G.PAGED["H"] + 1, 1), dtype=torch.int64))
    with pytest.raises(KeyError):
        pool.get_buffer(lid, "stage_0_indices_left", 1)
    with pytest.raises(IndexError):
        pool.get_buffer(lid + 1, "ks", 1)
    with pytest.raises(ValueError):
        pool.get_hip_metadata_cache(lid, 2, 1, None)
    # dense layers size their buffers from their own configuration (entry 0 of a two-entry layer table)
    assert pool.cache[0]["indices"].buffer.shape[-1] == 256 // 8 and pool.cache[lid]["indices"].buffer.shape[-1] == 128 // 8
    stats = pool.compute_cache_statistics(1)
    assert int(stats["sa_access"]) == 0 and int(stats["mask_miss"]) == 0
    pool.reset_decode_phase()


@pytest.mark.gpu
def test_decode_steps_through_the_metadata_pool_match_the_reference():
    """Decode steps whose cached metadata travels through the pool's compressed buffers: the restart at stage 1 sees
    bfloat16-rounded scores and uint32 bounds, the step after it reads the pooled mask; masks identical to the
    reference run through its own pool, outputs within fp16 tolerance."""
    from hip_attention_b200 import forward_paged_hip
    g = np.load(os.path.join(GOLD, "serving_pool.npz"))
    c = G.PAGED
    x = {k_: v_.cuda() for k_, v_ in G.paged_inputs().items()}
    pool, cfg = _pool("cuda")
    T, lid = c["T"], c["layer_id"]

    def call(q, position, seq_len, cached):
        # by keyword, exactly as the fixture generator calls the reference
        return forward_paged_hip(
            query=q, sm_scale=c["sm_scale"], batch_size=1, k_cache=x["k_pool"], v_cache=x["v_pool"], offload_cache=None,
            positions=torch.tensor([position], device="cuda"), seq_lens=torch.tensor([seq_len], device="cuda"),
            req_to_tokens=x["req_to_tokens"], req_pool_indices=x["req_pool_indices"], rope_cos=None, rope_sin=None, layer_id=lid,
            logit_cap=0.0, orig_context_len=c["model_context"], max_context_len=T, is_prefill=False, hip_config=cfg,
            cached_metadata=cached, is_decode=True)

    tol = 3e-3
    out0, md0 = call(x["q_decode"][0], T - 3, T - 2, pool.get_hip_metadata_cache(lid, 1, 1, -1))
    pool.set_hip_metadata_cache(lid, 1, 1, md0)
    assert np.array_equal(pool.get_hip_metadata_cache(lid, 1, 1, None).indices.cpu().numpy(), g["mask_indices"])
    assert np.array_equal(pool.get_hip_metadata_cache(lid, 1, 1, 1).stage_caches[1].out_scores.cpu().numpy(), g["stage1_scores"])
    out1, md1 = call(x["q_decode"][1], T - 2, T - 1, pool.get_hip_metadata_cache(lid, 1, 1, 1))
    pool.set_hip_metadata_cache(lid, 1, 1, md1)
    assert np.array_equal(md1.indices.cpu().numpy(), g["decode1_indices"]) and np.array_equal(md1.ks.cpu().numpy(), g["decode1_ks"])
    assert np.abs(out1.float().cpu().numpy() - g["decode1_out"]).max() < tol
    out2, _ = call(x["q_decode"][2], T - 1, T, pool.get_hip_metadata_cache(lid, 1, 1, None))
    assert np.abs(out2.float().cpu().numpy() - g["decode2_out"]).max() < tol


def test_forward_paged_hip_has_the_reference_parameter_list():
    """A caller written against the reference passes positionally: the names and their order must be the
    reference's (paged_hip.py:35-62), and the unbuilt options must be refused, not silently dropped."""
    import inspect
    from hip_attention_b200 import HiPAttentionConfig, cuda_graph_capture_configs, forward_paged_hip
    names = list(inspect.signature(forward_paged_hip).parameters)
    assert names == ["query", "sm_scale", "batch_size", "k_cache", "v_cache", "offload_cache", "positions", "seq_lens",
                     "req_to_tokens", "req_pool_indices", "rope_cos", "rope_sin", "layer_id", "logit_cap", "orig_context_len",
                     "max_context_len", "is_prefill", "hip_config", "cached_metadata", "k", "v", "online_update_cache",
                     "offloading_metadata", "is_decode", "query_for_mask", "diag_sliding_window_indices"]
    params = inspect.signature(forward_paged_hip).parameters
    assert all(params[n].default is inspect.Parameter.empty for n in names[:18])
    assert params["cached_metadata"].default is None and params["is_decode"].default is False
    cfg = HiPAttentionConfig()
    assert cuda_graph_capture_configs(cfg) == [(None,), (0,), (1,), (2,)]
    q = torch.zeros(2, 4, 64)
    tbl = torch.zeros(1, 8, dtype=torch.int64)
    common = (q, 1.0, 1, None, None)
    rest = (torch.zeros(2, dtype=torch.int64), torch.tensor([8]), tbl, torch.tensor([0]), None, None, 0, 0.0, 64, 64, True, cfg)
    with pytest.raises(NotImplementedError):
        forward_paged_hip(*common, object(), *rest)
    with pytest.raises(NotImplementedError):
        forward_paged_hip(*common, None, *rest, online_update_cache=True)
    with pytest.raises(NotImplementedError):
        forward_paged_hip(*common, None, *rest, diag_sliding_window_indices=torch.zeros(1))


@pytest.mark.gpu
def test_forward_paged_hip_with_in_kernel_rope_matches_the_reference():
    """The serving default ``using_extend``: un-rotated keys in the pool and cos / sin tables handed to the call.  A
    dense layer (scan backend streaming) and a sparse one, each a split prefill chunk and a decode step: masks
    identical to the reference's, outputs within fp16 tolerance."""
    from cases import rope_tables
    from hip_attention_b200 import HiPAttentionConfig, forward_paged_hip
    g = np.load(os.path.join(GOLD, "serving_paged_extend.npz"))
    c = G.PAGED
    x = {k_: v_.cuda() for k_, v_ in G.paged_inputs().items()}
    cfg = HiPAttentionConfig(json_or_path=G.EXTEND_JSON)
    assert cfg.using_extend
    T = c["T"]
    cos, sin = rope_tables(T + 8, c["D"], G.EXTEND_THETA)
    cos, sin = torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda()
    for layer_id in (0, c["layer_id"]):
        def call(q, positions, seq_len, is_decode):
            return forward_paged_hip(q, c["sm_scale"], 1, x["k_pool"], x["v_pool"], None, positions.cuda(),
                                     torch.tensor([seq_len], device="cuda"), x["req_to_tokens"], x["req_pool_indices"], cos, sin,
                                     layer_id, 0.0, c["model_context"], T, not is_decode, cfg, None, None, None, False, None,
                                     is_decode)
        p0 = T - 3 - c["chunk"]
        out, md = call(x["q_prefill"], torch.arange(p0, p0 + c["chunk"]), T - 3, False)
        assert np.array_equal(md.indices.cpu().numpy(), g[f"l{layer_id}_prefill_indices"])
        assert np.array_equal(md.ks.cpu().numpy(), g[f"l{layer_id}_prefill_ks"])
        assert np.abs(out.float().cpu().numpy() - g[f"l{layer_id}_prefill_out"]).max() < 3e-3
        out0, md0 = call(x["q_decode"][0], torch.tensor([T - 3]), T - 2, True)
        assert np.array_equal(md0.indices.cpu().numpy(), g[f"l{layer_id}_decode_indices"])
        assert np.array_equal(md0.ks.cpu().numpy(), g[f"l{layer_id}_decode_ks"])
        assert np.abs(out0.float().cpu().numpy() - g[f"l{layer_id}_decode_out"]).max() < 3e-3
