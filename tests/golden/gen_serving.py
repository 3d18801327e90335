"""Generate the fixtures of the serving-side adapter by running the reference's own modules.

Usage (only where the reference checkout is available; it is not needed to run the tests):

    python tests/golden/gen_serving.py --reference /path/to/hip-attention

Writes ``serving_config.json`` (parsed configurations and mask-refresh schedules from
``hip_attn/v1_2/hip_config.py`` and ``mask_refresh_interval.py``) and ``serving_paged.npz`` (outputs of
``hip_attn/v1_2/paged_hip.py::forward_paged_hip`` on a small token-granular KV pool: a prefill chunk long enough
to be split into a sparse part and its last 64 queries, a decode step that estimates everything, one that restarts
at stage 1 from the cached stage inputs and one that reuses the cached mask) and ``serving_pool.npz`` (the metadata
of the first decode step stored into and read back from ``hip_memory_pool.py::HiPMetadataCachePool``, and two decode
steps fed from the pool's compressed buffers).  The reference runs on the CPU
through ``TRITON_INTERPRET=1`` with the same shims and tie rule as ``gen_golden.py``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

_SMALL_LAYERS = [
    {"second_stage_k": 256, "sliding_window_size": 64, "sink_token_size": 16,
     "stages": [dict(stage_block_size_q=32, stage_block_stride_q=2, stage_chunk_size=32, stage_k=None, stage_stride=1),
                dict(stage_block_size_q=32, stage_block_stride_q=1, stage_chunk_size=8, stage_k=512, stage_stride=1)]},
    {"second_stage_k": 128, "sliding_window_size": 128, "sink_token_size": 32, "scan_extend_backend": "streaming",
     "stages": [dict(stage_block_size_q=32, stage_block_stride_q=2, stage_chunk_size=32, stage_k=None, stage_stride=1),
                dict(stage_block_size_q=32, stage_block_stride_q=1, stage_chunk_size=8, stage_k=256, stage_stride=1)]}]
CONFIG_JSONS = {
    "default": None,
    "no_extend": '{"using_extend": false}',
    "int_interval": '{"mask_refresh_interval": 8, "dense_layers": [0, 5], "block_sparse_block_size_q": 32}',
    # decode and prefill layers are separate keys: a file that sets only "layers" keeps the default prefill layers
    "decode_layers_only": json.dumps({"using_extend": False, "layers": _SMALL_LAYERS}),
    "custom_layers": json.dumps({"using_extend": False, "mask_refresh_interval": [4, 2, 1], "metadata_cache_max_batch_size": 8,
                                 "block_sparse_block_size_q": 32, "layers": _SMALL_LAYERS, "prefill_layers": _SMALL_LAYERS}),
}
BAD_JSONS = {"unknown_key": '{"not_a_key": 1}', "unknown_layer_key": '{"layers": [{"foo": 1}, {"foo": 2}]}'}
SCHEDULES = {"default": None, "int_interval": None, "custom_layers": None}   # by configuration name, 70 steps each

# the paged case: one request, context 1024, two-stage layers from "custom_layers" (layer 7 is not dense -> entry 1)
PAGED = dict(T=1024, H=4, HKV=2, D=64, chunk=160, layer_id=7, seed=4242, sm_scale=0.125, model_context=1024)


def paged_inputs():
    import numpy as np
    import torch
    c = PAGED
    rs = np.random.RandomState(c["seed"])
    T, H, HKV, D = c["T"], c["H"], c["HKV"], c["D"]
    k = torch.from_numpy(rs.standard_normal((T, HKV, D)).astype(np.float32)).to(torch.float16)
    v = torch.from_numpy(rs.standard_normal((T, HKV, D)).astype(np.float32)).to(torch.float16)
    q_prefill = torch.from_numpy(rs.standard_normal((c["chunk"], H, D)).astype(np.float32)).to(torch.float16)
    q_decode = torch.from_numpy(rs.standard_normal((3, 1, H, D)).astype(np.float32)).to(torch.float16)
    # token-granular pool: the request's tokens sit at permuted slots, the rest of the pool holds noise
    n_slots = T + 77
    perm = torch.from_numpy(rs.permutation(n_slots)[:T].astype(np.int64))
    k_pool = torch.from_numpy(rs.standard_normal((n_slots, HKV, D)).astype(np.float32)).to(torch.float16)
    v_pool = torch.from_numpy(rs.standard_normal((n_slots, HKV, D)).astype(np.float32)).to(torch.float16)
    k_pool[perm] = k
    v_pool[perm] = v
    req_to_tokens = torch.zeros((3, T), dtype=torch.int64)
    req_to_tokens[1] = perm
    return dict(k=k, v=v, q_prefill=q_prefill, q_decode=q_decode, k_pool=k_pool, v_pool=v_pool, req_to_tokens=req_to_tokens,
                req_pool_indices=torch.tensor([1], dtype=torch.int64))


def config_record(cfg):
    def layer(l):
        return dict(second_stage_k=l.second_stage_k, sliding_window_size=l.sliding_window_size, sink_token_size=l.sink_token_size,
                    sa_extend_backend=l.sa_extend_backend, scan_extend_backend=l.scan_extend_backend,
                    stages=[dict(stage_block_size_q=s.stage_block_size_q, stage_block_stride_q=s.stage_block_stride_q,
                                 stage_chunk_size=s.stage_chunk_size, stage_k=s.stage_k, stage_stride=s.stage_stride) for s in l.stages])
    return dict(dense_layers=cfg.dense_layers, block_sparse_block_size_q=cfg.block_sparse_block_size_q,
                metadata_cache_max_batch_size=cfg.metadata_cache_max_batch_size, mask_refresh_interval=cfg.mask_refresh_interval,
                using_extend=cfg.using_extend, layers=[layer(l) for l in cfg.layers], prefill_layers=[layer(l) for l in cfg.prefill_layers])


# The dense-layer entry uses window 128 here: with second_stage_k 256, sink 16 and window 64 the reference's flash-decode
# kernel cuts the 32 selected blocks into 7 ranges of 5 blocks and walks each range two blocks at a time without stopping at
# the range's end (attention_decode_bsa.py:235-249), so the block at every seam enters the softmax twice; with window 128
# the ranges hold 6 blocks and nothing is counted twice.
_EXTEND_LAYERS = [dict(_SMALL_LAYERS[0], sliding_window_size=128), _SMALL_LAYERS[1]]
EXTEND_JSON = json.dumps({"using_extend": True, "mask_refresh_interval": [4, 2, 1], "metadata_cache_max_batch_size": 8,
                          "block_sparse_block_size_q": 32, "layers": _EXTEND_LAYERS, "prefill_layers": _EXTEND_LAYERS})
EXTEND_THETA = 10000.0


def paged_extend(a, ph, cfgm):
    """The paged forward call with the serving default ``using_extend``: un-rotated keys in the pool, cos / sin
    tables handed in, scan backends relative (layer 7 overrides to streaming through its layer entry) and streaming
    (layer 0, a dense layer), attention backend streaming.  A split prefill chunk and one decode step per layer."""
    import numpy as np
    import torch
    from cases import rope_tables
    _sort = torch.Tensor.sort

    def stable_sort(self, *args, **kw):
        kw["stable"] = True
        return _sort(self, *args, **kw)

    def stable_topk(self, k, dim=-1, largest=True, sorted=True):
        r = _sort(self, dim=dim, descending=largest, stable=True)
        return torch.return_types.topk((r.values.narrow(dim, 0, k), r.indices.narrow(dim, 0, k)))

    torch.Tensor.sort = stable_sort
    torch.Tensor.topk = stable_topk
    c = PAGED
    x = paged_inputs()
    cfg = cfgm.HiPAttentionConfig(json_or_path=EXTEND_JSON)
    T = c["T"]
    cos, sin = rope_tables(T + 8, c["D"], EXTEND_THETA)
    cos, sin = torch.from_numpy(cos), torch.from_numpy(sin)
    save = {}
    for layer_id in (0, c["layer_id"]):
        def call(q, positions, seq_len, is_decode):
            return ph.forward_paged_hip(
                query=q, sm_scale=c["sm_scale"], batch_size=1, k_cache=x["k_pool"], v_cache=x["v_pool"], offload_cache=None,
                positions=positions, seq_lens=torch.tensor([seq_len], dtype=torch.int64), req_to_tokens=x["req_to_tokens"],
                req_pool_indices=x["req_pool_indices"], rope_cos=cos, rope_sin=sin, layer_id=layer_id, logit_cap=0.0,
                orig_context_len=c["model_context"], max_context_len=T, is_prefill=not is_decode, hip_config=cfg,
                cached_metadata=None, is_decode=is_decode)
        p0 = T - 3 - c["chunk"]
        out, md = call(x["q_prefill"], torch.arange(p0, p0 + c["chunk"], dtype=torch.int64), T - 3, False)
        save[f"l{layer_id}_prefill_out"], save[f"l{layer_id}_prefill_indices"] = out.float().numpy(), md.indices.numpy()
        save[f"l{layer_id}_prefill_ks"] = md.ks.numpy()
        out0, md0 = call(x["q_decode"][0], torch.tensor([T - 3], dtype=torch.int64), T - 2, True)
        save[f"l{layer_id}_decode_out"], save[f"l{layer_id}_decode_indices"] = out0.float().numpy(), md0.indices.numpy()
        save[f"l{layer_id}_decode_ks"] = md0.ks.numpy()
    np.savez_compressed(os.path.join(a.out, "serving_paged_extend.npz"), **save)
    print("wrote serving_paged_extend.npz")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of DeepAuto-AI/hip-attention")
    ap.add_argument("--out", default=HERE)
    ap.add_argument("--skip-paged", action="store_true")
    ap.add_argument("--only-extend", action="store_true", help="only the in-kernel RoPE run (serving_paged_extend.npz)")
    a = ap.parse_args()
    import gen_golden
    gen_golden._import_reference(a.reference)
    import importlib

    import numpy as np
    import torch
    cfgm = importlib.import_module("hip_attn.v1_2.hip_config")
    mrm = importlib.import_module("hip_attn.v1_2.mask_refresh_interval")
    md_mod = importlib.import_module("hip_attn.v1_2.attention_metadata")

    if a.only_extend:
        return paged_extend(a, importlib.import_module("hip_attn.v1_2.paged_hip"), cfgm)
    record = {"configs": {}, "bad": {}, "schedules": {}}
    for name, js in CONFIG_JSONS.items():
        record["configs"][name] = config_record(cfgm.HiPAttentionConfig(json_or_path=js))
    for name, js in BAD_JSONS.items():
        try:
            cfgm.HiPAttentionConfig(json_or_path=js)
            record["bad"][name] = None
        except Exception as e:      # noqa: BLE001 - the exception type is what is recorded
            record["bad"][name] = type(e).__name__
    for name in SCHEDULES:
        st = mrm.HiPMaskRefreshState(cfgm.HiPAttentionConfig(json_or_path=CONFIG_JSONS[name]))
        record["schedules"][name] = [st.update() for _ in range(70)]
    with open(os.path.join(a.out, "serving_config.json"), "w") as f:
        json.dump(record, f, indent=1, sort_keys=True)
    print("wrote serving_config.json")
    if a.skip_paged:
        return

    # ---- forward_paged_hip on the reference ----
    _sort, _topk = torch.Tensor.sort, torch.Tensor.topk

    def stable_sort(self, *args, **kw):
        kw["stable"] = True
        return _sort(self, *args, **kw)

    def stable_topk(self, k, dim=-1, largest=True, sorted=True):
        r = _sort(self, dim=dim, descending=largest, stable=True)
        return torch.return_types.topk((r.values.narrow(dim, 0, k), r.indices.narrow(dim, 0, k)))

    torch.Tensor.sort = stable_sort
    torch.Tensor.topk = stable_topk
    ph = importlib.import_module("hip_attn.v1_2.paged_hip")
    c = PAGED
    x = paged_inputs()
    cfg = cfgm.HiPAttentionConfig(json_or_path=CONFIG_JSONS["custom_layers"])
    T = c["T"]

    def call(q, positions, seq_len, is_decode, cached):
        return ph.forward_paged_hip(
            query=q, sm_scale=c["sm_scale"], batch_size=1, k_cache=x["k_pool"], v_cache=x["v_pool"], offload_cache=None,
            positions=positions, seq_lens=torch.tensor([seq_len], dtype=torch.int64), req_to_tokens=x["req_to_tokens"],
            req_pool_indices=x["req_pool_indices"], rope_cos=None, rope_sin=None, layer_id=c["layer_id"], logit_cap=0.0,
            orig_context_len=c["model_context"], max_context_len=T, is_prefill=not is_decode, hip_config=cfg,
            cached_metadata=cached, is_decode=is_decode)

    save = {}
    # prefill: the chunk covers positions [T - 3 - chunk, T - 3)
    p0 = T - 3 - c["chunk"]
    out, md = call(x["q_prefill"], torch.arange(p0, p0 + c["chunk"], dtype=torch.int64), T - 3, False, None)
    save["prefill_out"] = out.float().numpy()
    save["prefill_indices"] = md.indices.numpy()
    save["prefill_ks"] = md.ks.numpy()
    # decode step 0: estimate everything
    Cache = md_mod.HiPAttentionStageInputCache
    Meta = md_mod.HiPAttentionOutputMetadata
    out0, md0 = call(x["q_decode"][0], torch.tensor([T - 3], dtype=torch.int64), T - 2, True, None)
    save["decode0_out"], save["decode0_indices"], save["decode0_ks"] = out0.float().numpy(), md0.indices.numpy(), md0.ks.numpy()
    # decode step 1: restart at stage 1 from the cached stage inputs (what the metadata pool hands out for cached_stages = 1)
    cached1 = Meta(indices=None, ks=None, ks_count=None, ks_start_end=None, mask_cache_statistics=None, sa_cache_statistics=None,
                   stage_caches=[Cache(indices_left=None, indices_right=None, out_scores=None), md0.stage_caches[1]])
    out1, md1 = call(x["q_decode"][1], torch.tensor([T - 2], dtype=torch.int64), T - 1, True, cached1)
    save["decode1_out"], save["decode1_indices"], save["decode1_ks"] = out1.float().numpy(), md1.indices.numpy(), md1.ks.numpy()
    # decode step 2: reuse the mask of step 1
    cached2 = Meta(indices=md1.indices, ks=md1.ks, ks_count=md1.ks_count, ks_start_end=md1.ks_start_end, mask_cache_statistics=None,
                   sa_cache_statistics=None, stage_caches=None)
    out2, md2 = call(x["q_decode"][2], torch.tensor([T - 1], dtype=torch.int64), T, True, cached2)
    save["decode2_out"] = out2.float().numpy()
    np.savez_compressed(os.path.join(a.out, "serving_paged.npz"), **save)
    print("wrote serving_paged.npz")

    # ---- the metadata pool: store the first decode step, read it back in the three ways a step can ask for it ----
    pm = importlib.import_module("hip_attn.v1_2.hip_memory_pool")
    pool = pm.HiPMetadataCachePool(max_total_num_tokens=T + 77, query_head_num=c["H"], layer_num=c["layer_id"] + 1, context_length=T,
                                   device="cpu", hip_config=cfg)
    ps = {"allocated_bytes": np.int64(pool.compute_allocated_bytes())}
    ps["in_indices"], ps["in_ks"], ps["in_ks_count"], ps["in_ks_start_end"] = (md0.indices.numpy(), md0.ks.numpy(), md0.ks_count.numpy(),
                                                                               md0.ks_start_end.numpy())
    ps["in_stage1_left"], ps["in_stage1_right"], ps["in_stage1_scores"] = (md0.stage_caches[1].indices_left.numpy(),
                                                                           md0.stage_caches[1].indices_right.numpy(),
                                                                           md0.stage_caches[1].out_scores.float().numpy())
    pool.set_hip_metadata_cache(c["layer_id"], 1, 1, md0)
    got = pool.get_hip_metadata_cache(c["layer_id"], 1, 1, None)
    ps["mask_indices"], ps["mask_ks"], ps["mask_ks_count"], ps["mask_ks_start_end"] = (got.indices.numpy(), got.ks.numpy(), got.ks_count.numpy(),
                                                                                       got.ks_start_end.numpy())
    assert pool.get_hip_metadata_cache(c["layer_id"], 1, 1, 0) is None
    got1 = pool.get_hip_metadata_cache(c["layer_id"], 1, 1, 1)
    assert got1.indices is None and len(got1.stage_caches) == 2 and got1.stage_caches[0].indices_left is None
    ps["stage1_left"], ps["stage1_right"], ps["stage1_scores"] = (got1.stage_caches[1].indices_left.numpy(), got1.stage_caches[1].indices_right.numpy(),
                                                                  got1.stage_caches[1].out_scores.numpy())
    # decode step 1 restarted from the pool's stage inputs (scores rounded to bfloat16), then step 2 on the pooled mask
    outp1, mdp1 = call(x["q_decode"][1], torch.tensor([T - 2], dtype=torch.int64), T - 1, True, got1)
    ps["decode1_out"], ps["decode1_indices"], ps["decode1_ks"] = outp1.float().numpy(), mdp1.indices.numpy(), mdp1.ks.numpy()
    pool.set_hip_metadata_cache(c["layer_id"], 1, 1, mdp1)
    outp2, _ = call(x["q_decode"][2], torch.tensor([T - 1], dtype=torch.int64), T, True, pool.get_hip_metadata_cache(c["layer_id"], 1, 1, None))
    ps["decode2_out"] = outp2.float().numpy()
    try:
        pool.get_buffer(c["layer_id"], "ks", cfg.metadata_cache_max_batch_size + 1)
        ps["too_large"] = np.array("none")
    except Exception as e:      # noqa: BLE001 - the exception type is what is recorded
        ps["too_large"] = np.array(type(e).__name__)
    np.savez_compressed(os.path.join(a.out, "serving_pool.npz"), **ps)
    print("wrote serving_pool.npz")


if __name__ == "__main__":
    main()
