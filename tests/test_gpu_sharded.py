"""Sequence-sharded decode on one GPU: shards batched into one operator call, and a partly filled sequence."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _problem(S=8, L=4096, page=64):
    import bench
    from cases import make_paged
    w = dict(bench.WORKLOADS["decode_1m"], T=S * L, keep=[2048, 1024, 256])
    q, k, v = bench.make_qkv(w, "cuda")
    kc, vc, table = make_paged(k.cpu(), v.cpu(), page, 9)
    kc, vc, table = kc.cuda(), vc.cuda(), table.cuda().to(torch.int32)
    pps = L // page
    paged = [(kc, vc, table[:, s * pps:(s + 1) * pps].contiguous(), torch.full((1,), L, dtype=torch.int32, device="cuda"))
             for s in range(S)]
    dense = [(k[:, s * L:(s + 1) * L].contiguous(), v[:, s * L:(s + 1) * L].contiguous()) for s in range(S)]
    return w, q, paged, dense, bench.make_args(w)


def test_batched_shards_equal_shards_one_by_one():
    """Six of eight shards (no sink, no window, one page pool) run as one batched call: the masks are those of the
    one-by-one calls and the merged output agrees within the output tolerance (the batched call may cut its key
    ranges differently, which reorders fp32 sums)."""
    from hip_attention_b200 import read_status
    from hip_attention_b200.sharded import hip_attention_12_sequence_sharded
    S, L = 8, 4096
    w, q, paged, dense, args = _problem(S, L)
    read_status("cuda")
    one, mds1 = hip_attention_12_sequence_sharded(q, dense, args, n_shards=S, shard_len=L, per_shard_k=256)
    bat, mdsb = hip_attention_12_sequence_sharded(q, paged, args, n_shards=S, shard_len=L, per_shard_k=256)
    torch.cuda.synchronize()
    assert read_status("cuda") == 0
    assert len(mds1) == S and len(mdsb) == 3          # [shard 0] [shards 1-6] [shard 7]
    H = q.shape[2]
    assert torch.equal(mdsb[0].indices, mds1[0].indices) and torch.equal(mdsb[2].indices, mds1[7].indices)
    for j in range(6):
        assert torch.equal(mdsb[1].indices[j * H:(j + 1) * H], mds1[1 + j].indices), f"shard {1 + j}"
        assert torch.equal(mdsb[1].ks[j * H:(j + 1) * H], mds1[1 + j].ks)
    assert (bat.float() - one.float()).abs().max().item() < 1e-2
    again, _ = hip_attention_12_sequence_sharded(q, paged, args, n_shards=S, shard_len=L, per_shard_k=256, cached=mdsb)
    assert torch.equal(again, bat)


def test_partly_filled_sequence():
    """A sequence that ends inside shard 5: the window moves to that shard, its position follows its live length,
    shards 6 and 7 contribute nothing; the page-pool form and the form with dense slices of the live lengths agree."""
    from hip_attention_b200 import read_status
    from hip_attention_b200.sharded import hip_attention_12_sequence_sharded
    S, L = 8, 4096
    live = 5 * L + 1000
    w, q, paged, dense, args = _problem(S, L)
    paged = [(kc, vc, tb, torch.full((1,), max(0, min(L, live - s * L)), dtype=torch.int32, device="cuda"))
             for s, (kc, vc, tb, _) in enumerate(paged)]
    dense = [(k[:, :max(0, min(L, live - s * L))], v[:, :max(0, min(L, live - s * L))]) for s, (k, v) in enumerate(dense)]
    read_status("cuda")
    a, _ = hip_attention_12_sequence_sharded(q, paged, args, n_shards=S, shard_len=L, per_shard_k=256, seq_len=live)
    b, mds = hip_attention_12_sequence_sharded(q, dense, args, n_shards=S, shard_len=L, per_shard_k=256, seq_len=live)
    torch.cuda.synchronize()
    assert read_status("cuda") == 0
    assert mds[6] is None and mds[7] is None
    assert torch.isfinite(a.float()).all()
    assert (a.float() - b.float()).abs().max().item() < 1e-2
    full, _ = hip_attention_12_sequence_sharded(q, paged, args, n_shards=S, shard_len=L, per_shard_k=256)
    assert (a.float() - full.float()).abs().max().item() > 0      # the cut sequence is a different problem
    with pytest.raises(ValueError):
        hip_attention_12_sequence_sharded(q, dense, args, n_shards=S, shard_len=L, per_shard_k=256)   # slices too short
