"""Host-side logic of the two multi-GPU partitionings, rehearsed with 2 gloo ranks on the CPU.

The CPU oracle stands in for the device kernels; what is exercised is the partitioning itself:
which heads / key shards a rank owns, the MAX all-reduce of head-reduced scores after every scan
stage, and the all-gather + log-sum-exp merge of per-shard decode partials.
"""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _setup(rank, world, port):
    for p in (ROOT, os.path.join(ROOT, "tests"), os.path.join(ROOT, "tests", "golden")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)


def _kv_head_worker(rank, world, port, name, out):
    _setup(rank, world, port)
    from oracle import hip_oracle as O
    from hip_attention_b200.sharded import kv_head_slice, make_score_reduce
    from util import case_inputs
    q, k, v, pos, c, cfg, _ = case_inputs(name)
    hs, ks = kv_head_slice(rank, world, c["H"], c["HKV"])
    reduce = make_score_reduce()
    assert reduce is not None
    m = O.estimate_mask(q[:, :, hs].contiguous(), O.DenseKV(k[:, :, ks].contiguous()), pos, cfg, score_reduce=reduce)
    out[rank] = (m.indices, m.ks)
    dist.destroy_process_group()


@pytest.mark.parametrize("name", ["prefill_fp32", "decode_fp16"])
def test_kv_head_parallel_masks_equal_single_process(name):
    from oracle import hip_oracle as O
    from util import case_inputs
    world = 2
    out = mp.Manager().dict()
    mp.spawn(_kv_head_worker, args=(world, 29611 + hash(name) % 200, name, out), nprocs=world, join=True)
    q, k, v, pos, c, cfg, _ = case_inputs(name)
    ref = O.estimate_mask(q, O.DenseKV(k), pos, cfg)
    B, H = c["B"], c["H"]
    per = H // world
    full = ref.indices.view(B, H, *ref.indices.shape[1:])
    for r in range(world):
        idx, ks = out[r]
        assert torch.equal(idx.view(B, per, *idx.shape[1:]), full[:, r * per:(r + 1) * per])
        assert torch.equal(ks.view(B, per, -1), ref.ks.view(B, H, -1)[:, r * per:(r + 1) * per])


def _shard_worker(rank, world, port, out):
    _setup(rank, world, port)
    from oracle import hip_oracle as O
    from hip_attention_b200 import HiPAttentionArgs
    from hip_attention_b200.sharded import sequence_shard_args
    S, L = 4, 512
    q, k, v, cfg_stages = _shard_problem(S * L)
    per = S // world
    parts_o, parts_l = [], []
    for j in range(per):
        s = rank * per + j
        a = sequence_shard_args(HiPAttentionArgs(sink_token_size=32, sliding_window_size=64), s, S, L, 64, "cpu")
        cfg = O.OracleConfig(stages=cfg_stages, sink=a.sink_token_size, sw=a.sliding_window_size, second_stage_k=a.second_stage_k)
        pos = torch.full((1, 1), L - 1, dtype=torch.int64)
        ks, vs = O.DenseKV(k[:, s * L:(s + 1) * L]), O.DenseKV(v[:, s * L:(s + 1) * L])
        m = O.estimate_mask(q, ks, pos, cfg)
        o, lse = O.attention_on_mask(q, ks, vs, pos, m, sink=cfg.sink, sw=max(cfg.sw, cfg_stages[0].chunk_size), return_lse=True)
        parts_o.append(o)
        parts_l.append(lse)
    po, pl = torch.stack(parts_o), torch.stack(parts_l)
    go = [torch.empty_like(po) for _ in range(world)]
    gl = [torch.empty_like(pl) for _ in range(world)]
    dist.all_gather(go, po)
    dist.all_gather(gl, pl)
    merged, _ = O.merge_partials(torch.cat(go), torch.cat(gl))
    out[rank] = merged
    dist.destroy_process_group()


def _shard_problem(T):
    from oracle import hip_oracle as O
    import numpy as np
    rs = np.random.RandomState(5)
    D = 64
    q = torch.from_numpy(rs.standard_normal((1, 1, 4, D)).astype("float32") * D ** -0.5)
    k = torch.from_numpy(rs.standard_normal((1, T, 2, D)).astype("float32"))
    v = torch.from_numpy(rs.standard_normal((1, T, 2, D)).astype("float32"))
    stages = [O.OracleStage(64, 4, 32, None), O.OracleStage(64, 1, 8, 128)]
    return q, k, v, stages


def test_sequence_sharded_decode_is_independent_of_rank_count():
    """4 logical shards on 2 ranks give the result of 4 shards on 1 rank; shard 0 alone owns the sink and
    the last shard alone owns the sliding window."""
    from oracle import hip_oracle as O
    from hip_attention_b200 import HiPAttentionArgs
    from hip_attention_b200.sharded import sequence_shard_args
    out = mp.Manager().dict()
    mp.spawn(_shard_worker, args=(2, 29877, out), nprocs=2, join=True)
    assert torch.equal(out[0], out[1])
    S, L = 4, 512
    q, k, v, stages = _shard_problem(S * L)
    os_, ls_ = [], []
    for s in range(S):
        a = sequence_shard_args(HiPAttentionArgs(sink_token_size=32, sliding_window_size=64), s, S, L, 64, "cpu")
        assert a.sink_token_size == (32 if s == 0 else 0) and a.sliding_window_size == (64 if s == S - 1 else 0)
        assert a.second_stage_k == 64 and a.extend_context_length == L
        cfg = O.OracleConfig(stages=stages, sink=a.sink_token_size, sw=a.sliding_window_size, second_stage_k=64)
        pos = torch.full((1, 1), L - 1, dtype=torch.int64)
        ks, vs = O.DenseKV(k[:, s * L:(s + 1) * L]), O.DenseKV(v[:, s * L:(s + 1) * L])
        m = O.estimate_mask(q, ks, pos, cfg)
        o, lse = O.attention_on_mask(q, ks, vs, pos, m, sink=cfg.sink, sw=max(cfg.sw, 32), return_lse=True)
        os_.append(o)
        ls_.append(lse)
    ref, _ = O.merge_partials(torch.stack(os_), torch.stack(ls_))
    assert (out[0] - ref).abs().max().item() < 1e-12


def test_kv_head_slice_partitions_heads():
    from hip_attention_b200.sharded import kv_head_slice
    seen_q, seen_kv = [], []
    for r in range(4):
        hs, ks = kv_head_slice(r, 4, 32, 8)
        seen_q += list(range(32))[hs]
        seen_kv += list(range(8))[ks]
        assert (hs.stop - hs.start) == 4 * (ks.stop - ks.start)
    assert seen_q == list(range(32)) and seen_kv == list(range(8))
    with pytest.raises(ValueError):
        kv_head_slice(0, 3, 32, 8)
