"""GPU parity: the CUDA path (through the C ABI) against the CPU oracle and the reference fixtures."""
import os

import numpy as np
import pytest
import torch

from cases import CASES
from oracle import hip_oracle as O
from util import case_inputs, make_args, output_tolerance, run_gpu

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
SMALL = [n for n in CASES if n != "config1_fp32"]


def _oracle(q, k, v, pos, cfg, paged, **kw):
    return O.hip_attention_oracle(q, k, v, pos, cfg, paged=paged, **kw)


def _check_mask(md, m):
    assert md.indices.dtype == torch.int64 and md.ks.dtype == torch.int64 and md.ks_start_end.dtype == torch.int32
    assert torch.equal(md.indices.cpu(), m.indices), "indices differ from the oracle"
    assert torch.equal(md.ks.cpu(), m.ks)
    assert torch.equal(md.ks_count.cpu(), m.ks_count)
    assert torch.equal(md.ks_start_end.cpu(), m.ks_start_end)


def _check_out(out, ref, dtype):
    mx, mean = output_tolerance(dtype)
    err = (out.float().cpu().double() - ref.double()).abs()
    assert err.max().item() <= mx, f"max-abs {err.max().item()}"
    assert err.mean().item() <= mean, f"mean-abs {err.mean().item()}"


@pytest.mark.parametrize("name", SMALL)
def test_matches_reference_fixture(name):
    """Same inputs as the recorded reference run: masks identical, output within tolerance."""
    g = np.load(os.path.join(GOLD, f"{name}.npz"))
    q, k, v, pos, c, cfg, paged = case_inputs(name)
    out, md = run_gpu(q, k, v, pos, c, paged)
    assert np.array_equal(md.indices.cpu().numpy(), g["indices"])
    assert np.array_equal(md.ks.cpu().numpy(), g["ks"])
    assert np.array_equal(md.ks_count.cpu().numpy(), g["ks_count"])
    assert np.array_equal(md.ks_start_end.cpu().numpy(), g["ks_start_end"])
    for i in range(1, len(cfg.stages)):
        assert np.array_equal(md.stage_caches[i].indices_left.cpu().numpy(), g[f"stage{i}_left"])
        assert np.array_equal(md.stage_caches[i].indices_right.cpu().numpy(), g[f"stage{i}_right"])
        assert np.array_equal(md.stage_caches[i].out_scores.cpu().numpy(), g[f"stage{i}_scores"])
    assert md.stage_caches[0].indices_left is None
    rs = c.get("out_row_stride", 1)
    tol = 2e-5 if c["dtype"] == "fp32" else 3e-3  # the fp16 reference rounds P and the output to fp16
    err = np.abs(out.float().cpu().numpy()[:, ::rs] - g["out"]).max()
    assert err < tol, err


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("name", ["prefill_fp32", "ragged_fp16", "decode_fp16", "square_fp16", "oddsink_fp16",
                                  "shortwin_fp16", "paged_decode_fp16", "shard_nosink_fp16", "positions_fp16",
                                  "softcap_fp16", "softcap_decode_fp16", "rope_rel_fp16", "rope_str_fp16", "rope_decode_fp16",
                                  "rope_mixed_fp32", "rope_str_decode_fp16", "rope_d128_fp16", "rope_d128_str_fp16", "fp8_prefill_fp16",
                                  "fp8_decode_fp16"])
def test_matches_oracle_all_dtypes(name, dtype):
    q, k, v, pos, c, cfg, paged = case_inputs(name, dtype)
    (ref, m) = _oracle(q, k, v, pos, cfg, paged)
    out, md = run_gpu(q, k, v, pos, c, paged)
    _check_mask(md, m)
    _check_out(out, ref, dtype)


@pytest.mark.parametrize("name", ["prefill_fp32", "ragged_fp16", "oddsink_fp16", "shortwin_fp16", "rope_rel_fp16",
                                  "rope_mixed_fp32", "rope_d128_fp16", "rope_d128_str_fp16"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_scan_stage_outputs(name, dtype):
    """Per-head narrowed bounds and scores of every scan stage equal the oracle's, bit for bit."""
    q, k, v, pos, c, cfg, paged = case_inputs(name, dtype)
    ksrc = O.DenseKV(k)
    m = O.estimate_mask(q, ksrc, pos, cfg, keep_stage_outputs=True)
    dbg = {}
    run_gpu(q, k, v, pos, c, paged, debug=dbg)
    B, TQ, H, D = q.shape
    for i, (l, r, s, red) in enumerate(m.stage_outputs):
        st = dbg["stages"][i]
        n = l.shape[-1]
        assert torch.equal(st["left"].cpu().view(B, -1, H, n).long(), l), f"stage {i} left"
        assert torch.equal(st["right"].cpu().view(B, -1, H, n).long(), r), f"stage {i} right"
        assert torch.equal(st["score"].cpu().view(B, -1, H, n), s), f"stage {i} score"


def test_config1_fixture():
    """benchmark configuration 1 (fp32 4096 x 4096, 8/2 heads, D 64) against the recorded reference run."""
    path = os.path.join(GOLD, "config1_fp32.npz")
    if not os.path.exists(path):
        pytest.skip("fixture not generated")
    g = np.load(path)
    q, k, v, pos, c, cfg, paged = case_inputs("config1_fp32")
    out, md = run_gpu(q, k, v, pos, c, paged)
    assert np.array_equal(md.indices.cpu().numpy(), g["indices"])
    assert np.array_equal(md.ks.cpu().numpy(), g["ks"])
    err = np.abs(out.float().cpu().numpy()[:, ::c["out_row_stride"]] - g["out"]).max()
    assert err < 2e-5, err


@pytest.mark.parametrize("page", [1, 16, 64])
@pytest.mark.parametrize("tq,case", [(1, "paged_prefill_fp16"), (100, "paged_prefill_fp16"), (200, "d128_fp16"), (200, "rope_d128_fp16")])
def test_paged_equals_dense(page, tq, case):
    """Paging is pure addressing: a permuted page pool gives the dense result (any page size); head dim 128 takes the
    tcgen05 scan and attention kernels, with and without in-kernel RoPE."""
    import cases as cs
    from cases import make_paged
    base = dict(cs.CASES[case], TQ=tq, dtype="bf16")
    cs.CASES["_tmp_paged"] = {k_: v_ for k_, v_ in base.items() if k_ not in ("page", "ext")}
    try:
        q, k, v, pos, c, cfg, _ = case_inputs("_tmp_paged")
    finally:
        del cs.CASES["_tmp_paged"]
    out_d, md_d = run_gpu(q, k, v, pos, c, None)
    kc, vc, table = make_paged(k, v, page, 5)
    for ext in (c["T"], c["T"] + 512):
        paged = (kc, vc, table.to(torch.int32), torch.full((c["B"],), c["T"], dtype=torch.int32), ext)
        out_p, md_p = run_gpu(q, k, v, pos, c, paged)
        assert torch.equal(md_p.indices, md_d.indices) and torch.equal(md_p.ks, md_d.ks)
        assert torch.equal(out_p, out_d)


@pytest.mark.parametrize("name", ["prefill_fp32", "ragged_fp16", "decode_fp16", "bsa16_fp16", "d128_fp16"])
def test_cached_mask_and_stage_restart(name):
    """Reference invariant (tests/v1_2/test_gen3_stage_caching.py:170-186): replaying any prefix of the
    stage caches, or the whole cached mask, reproduces the output (sum of squared differences < 1e-8)."""
    from hip_attention_b200 import HiPAttentionOutputMetadata, hip_attention_12
    q, k, v, pos, c, cfg, paged = case_inputs(name)
    dev = "cuda"
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    out, md = hip_attention_12(qd, kd, vd, make_args(c, pos.to(dev)))
    out2, md2 = hip_attention_12(qd, kd, vd, make_args(c, pos.to(dev)), cached_metadata=md)
    assert torch.equal(out, out2)
    assert md2.mask_cache_statistics is None and md2.sa_cache_statistics is not None
    assert torch.equal(md2.indices, md.indices) and md2.indices.data_ptr() != md.indices.data_ptr()
    for n in range(1, len(md.stage_caches) + 1):
        part = HiPAttentionOutputMetadata(indices=None, ks=None, ks_count=None, ks_start_end=None,
                                          mask_cache_statistics=None, sa_cache_statistics=None,
                                          stage_caches=list(md.stage_caches[:n]))
        o3, m3 = hip_attention_12(qd, kd, vd, make_args(c, pos.to(dev)), cached_metadata=part)
        assert ((o3.float() - out.float()) ** 2).sum().item() < 1e-8
        assert torch.equal(m3.indices, md.indices)
        assert len(m3.stage_caches) == len(cfg.stages)
    # a foreign cache (plain int64 tensors, as the reference would hand over) restarts the same way
    from hip_attention_b200 import HiPAttentionStageInputCache
    foreign = [HiPAttentionStageInputCache(None, None, None)] + [
        HiPAttentionStageInputCache(s.indices_left.clone(), s.indices_right.clone(), s.out_scores.clone())
        for s in md.stage_caches[1:]]
    part = HiPAttentionOutputMetadata(None, None, None, None, None, None, foreign)
    o4, m4 = hip_attention_12(qd, kd, vd, make_args(c, pos.to(dev)), cached_metadata=part)
    assert torch.equal(m4.indices, md.indices) and torch.equal(o4, out)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_decode_kernel_equals_prefill_kernel(dtype):
    """Reference check (tests/v1_2/test_attention_decode_bsa.py:104-107): split-KV decode and the
    prefill kernel agree on the same mask."""
    from hip_attention_b200 import hip_attention_12
    q, k, v, pos, c, cfg, paged = case_inputs("decode_fp16", dtype)
    dev = "cuda"
    o1, md = hip_attention_12(q.to(dev), k.to(dev), v.to(dev), make_args(c, pos.to(dev)))
    a2 = make_args(c, pos.to(dev))
    a2.disable_flashdecode = True
    o2, _ = hip_attention_12(q.to(dev), k.to(dev), v.to(dev), a2, cached_metadata=md)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert (o1.float() - o2.float()).abs().max().item() < tol


def test_lse_and_merge_match_oracle():
    """Partial outputs with their log-sum-exp merge to the unsplit result (attention_decode_bsa.py:1192-1225)."""
    from hip_attention_b200 import hip_attention_impl
    q, k, v, pos, c, cfg, paged = case_inputs("decode_fp16", torch.float32)
    ksrc, vsrc = O.DenseKV(k), O.DenseKV(v)
    m = O.estimate_mask(q, ksrc, pos, cfg)
    ref, lse_ref = O.attention_on_mask(q, ksrc, vsrc, pos, m, sink=cfg.sink, sw=max(cfg.sw, cfg.stages[0].chunk_size),
                                       return_lse=True)
    out, md, lse = hip_attention_impl(q.cuda(), k.cuda(), v.cuda(), make_args(c, pos.cuda()), return_lse=True)
    assert (lse.cpu().double() - lse_ref).abs().max().item() < 1e-4
    assert (out.cpu().double() - ref).abs().max().item() < 2e-5


def test_short_context_has_empty_selection():
    """K shorter than sink + window: nothing to scan, attention covers sink and window only."""
    from hip_attention_b200 import HiPAttentionArgs, hip_attention_12
    torch.manual_seed(0)
    B, TQ, T, H, HKV, D = 1, 40, 200, 4, 2, 64
    q = (torch.randn(B, TQ, H, D) * D ** -0.5).cuda().bfloat16()
    k = torch.randn(B, T, HKV, D).cuda().bfloat16()
    v = torch.randn(B, T, HKV, D).cuda().bfloat16()
    out, md = hip_attention_12(q, k, v, HiPAttentionArgs())
    assert md.indices.shape == (B * H, 1, 0) and int(md.ks.sum()) == 0
    kk = k.float().repeat_interleave(H // HKV, 2)
    vv = v.float().repeat_interleave(H // HKV, 2)
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), kk)
    causal = (torch.arange(T, device="cuda")[None, :] <= (torch.arange(TQ, device="cuda") + T - TQ)[:, None])
    ref = torch.einsum("bhqk,bkhd->bqhd", s.masked_fill(~causal, float("-inf")).softmax(-1), vv)
    assert (out.float() - ref).abs().max().item() < 2e-2


def test_invalid_arguments_raise_before_launch():
    from hip_attention_b200 import HiPAttentionArgs, ScanStage, hip_attention_12
    q = torch.zeros(1, 8, 4, 64, device="cuda", dtype=torch.bfloat16)
    k = torch.zeros(1, 1024, 2, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        hip_attention_12(q, k, k[:, :512], HiPAttentionArgs())
    with pytest.raises(NotImplementedError):
        hip_attention_12(q, k, k, HiPAttentionArgs(using_extend=True, need_apply_rope=False))
    with pytest.raises(ValueError):
        hip_attention_12(q, k, k, HiPAttentionArgs(using_extend=True, need_apply_rope=True))   # no cos / sin tables
    tab = torch.zeros(2048, 64, device="cuda")
    with pytest.raises(NotImplementedError):
        hip_attention_12(q, k, k, HiPAttentionArgs(using_extend=True, need_apply_rope=True, rope_cos=tab, rope_sin=tab,
                                                   scan_extend_backend="dynamic_extend"))
    with pytest.raises(ValueError):
        hip_attention_12(q, k, k, HiPAttentionArgs(stages=[ScanStage(64, 4, 256, 128, 1)]))
    with pytest.raises(ValueError):
        hip_attention_12(q, k, k, HiPAttentionArgs(position_ids=torch.zeros(1, 7, dtype=torch.int64, device="cuda")))
    with pytest.raises(NotImplementedError):
        hip_attention_12(q[..., :48].contiguous(), k[..., :48].contiguous(), k[..., :48].contiguous(), HiPAttentionArgs())
    with pytest.raises(RuntimeError):
        hip_attention_12(q.cpu(), k.cpu(), k.cpu(), HiPAttentionArgs())


@pytest.mark.parametrize("tq", [1, 70])
def test_query_position_beyond_dense_keys_is_clamped_and_flagged(tq):
    """Dense K / V and a query position at or beyond their length: sink and window entries stop at T (no row past
    the end of the tensors is read -- the rows behind them hold NaN here and would poison the output), the status
    word reports it, and the result is the softmax over the admitted keys below T."""
    from hip_attention_b200 import hip_attention_impl, read_status
    q, k, v, pos, c, cfg, _ = case_inputs("ragged_fp16", torch.bfloat16)
    B, T = k.shape[0], k.shape[1]
    q = q[:, :tq].contiguous()
    big_k = torch.full((B, T + 64) + tuple(k.shape[2:]), float("nan"), dtype=k.dtype, device="cuda")
    big_v = torch.full_like(big_k, float("nan"))
    big_k[:, :T], big_v[:, :T] = k.cuda(), v.cuda()
    kd, vd = big_k[:, :T], big_v[:, :T]          # views: the allocation continues behind them
    pos_far = (torch.arange(tq)[None] + T + 5 - (tq - 1)).expand(B, tq).contiguous()   # last row at T + 5
    read_status("cuda")
    out, md = hip_attention_impl(q.cuda(), kd, vd, make_args(c, pos_far.cuda()))
    torch.cuda.synchronize()
    assert read_status("cuda") & 2
    assert torch.isfinite(out.float()).all()
    m = O.OracleMask(md.indices.cpu(), md.ks.cpu(), md.ks_count.cpu(), md.ks_start_end.cpu())
    m.block_size_k, m.block_size_q = cfg.stages[-1].chunk_size, cfg.stages[-1].block_size_q
    ref = _attention_below_T(q, k, v, pos_far, m, cfg)
    _check_out(out, ref, torch.bfloat16)


def _attention_below_T(q, k, v, pos, m, cfg):
    """fp64 softmax over the attended set of ``oracle.attended_columns`` cut at the number of keys."""
    B, TQ, H, D = q.shape
    T, G = k.shape[1], H // k.shape[2]
    sw = max(cfg.sw, cfg.stages[0].chunk_size)
    bq = m.block_size_q
    out = torch.zeros(B, TQ, H, D, dtype=torch.float64)
    for b in range(B):
        for d in range(-(-TQ // bq)):
            r0, r1 = d * bq, min(TQ, (d + 1) * bq)
            for h in range(H):
                cols, allow = O.attended_columns(m.indices[b * H + h, d], int(m.ks[b * H + h, d]), pos[b, r0:r1], sink=cfg.sink,
                                                 sw=sw, c_last=m.block_size_k, T=T)
                keep = cols < T
                cols, allow = cols[keep], allow[:, keep]
                s = q[b, r0:r1, h].double() @ k[b, cols, h // G].double().T
                s = s.masked_fill(~allow, float("-inf"))
                out[b, r0:r1, h] = torch.nan_to_num(torch.softmax(s, -1)) @ v[b, cols, h // G].double()
    return out


@pytest.mark.parametrize("name", ["fp8_prefill_fp16", "fp8_decode_fp16"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fp8_cache_forms_agree(name, dtype):
    """An fp8 (e5m2) KV cache as a dense 1-byte tensor, as a permuted page pool, and as the uint8 view a serving
    adapter makes of it: identical masks and outputs; float32 queries are refused."""
    from cases import make_paged
    from hip_attention_b200 import hip_attention_impl
    q, k, v, pos, c, cfg, _ = case_inputs(name, dtype)
    out_d, md_d = run_gpu(q, k, v, pos, c, None)
    kc, vc, table = make_paged(k, v, 16, 11)
    for view in (torch.float8_e5m2, torch.uint8):
        k8, v8 = kc.to(torch.float8_e5m2).view(view).cuda(), vc.to(torch.float8_e5m2).view(view).cuda()
        args = make_args(c, pos.cuda(), k_cache=k8, v_cache=v8, block_table=table.cuda(),
                         cache_seq_lens=torch.full((c["B"],), c["T"], dtype=torch.int64, device="cuda"), extend_context_length=c["T"])
        out_p, md_p = hip_attention_impl(q.cuda(), None, None, args)
        assert torch.equal(md_p.indices, md_d.indices) and torch.equal(md_p.ks, md_d.ks)
        assert torch.equal(out_p, out_d)
    with pytest.raises(NotImplementedError):
        hip_attention_impl(q.float().cuda(), k.to(torch.float8_e5m2).cuda(), v.to(torch.float8_e5m2).cuda(), make_args(c, pos.cuda()))


def test_fp8_cache_on_the_benchmark_shape():
    """Head dim 128, bf16 queries, fp8 keys and values (prefill through the prepared 16-bit key copy and the tensor-core
    scan): the mask equals the one of the same call on the widened values, the output stays within tolerance of it."""
    import bench
    from hip_attention_b200 import hip_attention_impl, read_status
    w = dict(bench.WORKLOADS["prefill_128k"], TQ=512, T=8192, keep=[4096, 2048, 1024])
    q, k, v = bench.make_qkv(w, "cuda")
    k8, v8 = k.to(torch.float8_e5m2), v.to(torch.float8_e5m2)
    read_status("cuda")
    out8, md8 = hip_attention_impl(q, k8, v8, bench.make_args(w))
    out16, md16 = hip_attention_impl(q, k8.to(q.dtype), v8.to(q.dtype), bench.make_args(w))
    torch.cuda.synchronize()
    assert read_status("cuda") == 0
    assert torch.equal(md8.indices, md16.indices) and torch.equal(md8.ks, md16.ks)
    d = (out8.float() - out16.float()).abs()
    assert d.max().item() <= 2e-2 and d.mean().item() <= 2e-3


STATS = ["stats_prefill_fp16", "stats_decode_fp16", "stats_paged_fp16", "stats_paged_decode_fp16"]


@pytest.mark.parametrize("name", STATS)
def test_access_statistics_match_the_reference(name):
    """require_cache_statistics: the positions (dense K) or pages (paged K) the estimator and the attention loaded,
    as recorded from the reference; no offload cache exists, so nothing is ever a miss.  A call on the cached mask
    reports the attention's accesses only."""
    from hip_attention_b200 import hip_attention_12
    g = np.load(os.path.join(GOLD, f"{name}.npz"))
    q, k, v, pos, c, cfg, paged = case_inputs(name)
    out, md = run_gpu(q, k, v, pos, c, paged)
    for nm, st in (("mask", md.mask_cache_statistics), ("sa", md.sa_cache_statistics)):
        assert st.access_counter.dtype == torch.int32 and st.cache_miss_counter.dtype == torch.int32
        assert np.array_equal(st.access_counter.cpu().numpy(), g[f"{nm}_access"]), f"{nm} access counter"
        assert int(st.cache_miss_counter.sum()) == 0 and st.cache_miss_counter.shape == st.access_counter.shape
    import os as _os
    _os.environ["HIP_DISABLE_COMPUTE_STATISTICS"] = "0"
    try:
        got = md.sa_cache_statistics.compute_statistics()
        assert int(got["access_count"]) == int(g["sa_access"].sum()) and int(got["cache_miss_count"]) == 0
    finally:
        del _os.environ["HIP_DISABLE_COMPUTE_STATISTICS"]
    if paged is None:
        _, md2 = hip_attention_12(q.cuda(), k.cuda(), v.cuda(), make_args(c, pos.cuda()), cached_metadata=md)
        assert md2.mask_cache_statistics is None
        assert torch.equal(md2.sa_cache_statistics.access_counter, md.sa_cache_statistics.access_counter)
        a2 = make_args(c, pos.cuda())
        a2.require_cache_statistics = False
        _, md3 = hip_attention_12(q.cuda(), k.cuda(), v.cuda(), a2)
        assert md3.mask_cache_statistics.access_counter is None and md3.sa_cache_statistics.access_counter is None


@pytest.mark.parametrize("name", ["stats_prefill_fp16", "stats_decode_fp16", "stats_paged_fp16"])
def test_access_statistics_match_the_oracle_in_bf16(name):
    """The same sets from every scan kernel that can run the case (tensor-core rounds with row skipping, strict rounds,
    whole chunks in decode): a skipped row was marked when it was first fetched, a whole-chunk pass marks the rows the
    rounds would have asked for."""
    q, k, v, pos, c, cfg, paged = case_inputs(name, torch.bfloat16)
    if paged is not None:
        kc, vc, table, seq, ext = paged
        ksrc = O.PagedKV(kc, table, seq, ext)
    else:
        ksrc = O.DenseKV(k)
    m = O.estimate_mask(q, ksrc, pos, cfg, statistics=True)
    sw_attn = max(0, cfg.sw - cfg.stages[0].chunk_size) + cfg.stages[0].chunk_size
    sa = O.attention_access(m, pos, ksrc, c["H"], sink=cfg.sink, sw=sw_attn, decode=c["TQ"] == 1)
    for mode in ("auto", "strict"):
        os.environ["HIPATTN_SCAN_MODE"] = mode
        try:
            out, md = run_gpu(q, k, v, pos, c, paged)
        finally:
            del os.environ["HIPATTN_SCAN_MODE"]
        assert torch.equal(md.mask_cache_statistics.access_counter.cpu(), m.mask_access), mode
        assert torch.equal(md.sa_cache_statistics.access_counter.cpu(), sa), mode


def test_unbuilt_stage_flags_are_refused():
    """A stage that switches off realignment, score reset or the position sort selects a branch the kernels do not
    have: the call must say so instead of returning a different mask."""
    from hip_attention_b200 import HiPAttentionArgs, ScanStage, hip_attention_12
    q = torch.zeros(1, 8, 4, 64, device="cuda", dtype=torch.bfloat16)
    k = torch.zeros(1, 4096, 2, 64, device="cuda", dtype=torch.bfloat16)
    for flag in ("require_realign_index", "require_reset_score", "require_post_sort"):
        stages = [ScanStage(64, 4, 256, None, 1), ScanStage(64, 4, 32, 2048, 1, **{flag: False})]
        with pytest.raises(NotImplementedError):
            hip_attention_12(q, k, k, HiPAttentionArgs(stages=stages, second_stage_k=512))


def test_bad_page_table_is_clamped_and_flagged():
    """Out-of-range block-table entries never fault: they read page 0 and set a status bit."""
    from cases import make_paged
    from hip_attention_b200 import read_status
    q, k, v, pos, c, cfg, _ = case_inputs("paged_decode_fp16", torch.bfloat16)
    kc, vc, table = make_paged(k, v, 16, 3)
    table = table.clone()
    table[0, 5] = 10 ** 6
    table[1, 7] = -3
    read_status("cuda")
    paged = (kc, vc, table, torch.full((c["B"],), c["T"], dtype=torch.int64), c["ext"])
    out, md = run_gpu(q, k, v, pos, c, paged)
    torch.cuda.synchronize()
    assert read_status("cuda") & 1
    assert torch.isfinite(out.float()).all()


def _scan_check_run(dtype, TQ=512, T=16384, rope_backend=None):
    """Run the estimator in check mode on a bench-shaped problem; returns (stats, indices)."""
    import bench
    from hip_attention_b200 import hip_attention_impl
    w = dict(bench.WORKLOADS["prefill_128k"], TQ=TQ, T=T, keep=[4096, 2048, 1024],
             dtype={torch.bfloat16: "bf16", torch.float16: "fp16"}[dtype])
    q, k, v = bench.make_qkv(w, "cuda")
    kw = {}
    if rope_backend is not None:
        from cases import rope_tables
        cos, sin = rope_tables(T + 8, w["D"], w["theta"])
        kw = dict(using_extend=True, need_apply_rope=True, rope_cos=torch.from_numpy(cos).cuda(), rope_sin=torch.from_numpy(sin).cuda(),
                  scan_extend_backend=rope_backend)
    args = bench.make_args(w, **kw)
    stats = torch.zeros(4, dtype=torch.int64, device="cuda")
    out, md = hip_attention_impl(q, k, v, args, debug={"scan_stats": stats})
    torch.cuda.synchronize()
    return stats.cpu(), md, (q, k, v, w)


@pytest.mark.parametrize("scan_kernel", ["auto", "mma"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_scan_tensor_core_path_is_exact(dtype, scan_kernel, monkeypatch):
    """The tensor-core scans (tcgen05, mma.sync) take a shortcut only where rounding is certain.  In
    check mode every key is also scored by the strict definition: no shortcut may be wrong, and the
    observed deviation must stay well inside the assumed error radius.  Strict and automatic modes give
    identical masks."""
    import numpy as np
    monkeypatch.setenv("HIPATTN_SCAN_KERNEL", scan_kernel)
    monkeypatch.setenv("HIPATTN_SCAN_MODE", "check")
    stats, md_check, _ = _scan_check_run(dtype)
    keys, fallbacks, wrong = int(stats[0]), int(stats[1]), int(stats[2])
    ratio = float(np.array([int(stats[3]) & 0xffffffff], dtype=np.uint32).view(np.float32)[0])
    assert keys > 800_000
    assert wrong == 0, f"{wrong} shortcuts disagree with the strict score"
    assert ratio < 0.5, f"deviation reached {ratio:.3f} of the assumed radius"
    assert fallbacks / keys < 0.25
    monkeypatch.setenv("HIPATTN_SCAN_MODE", "auto")
    _, md_auto, _ = _scan_check_run(dtype)
    monkeypatch.setenv("HIPATTN_SCAN_MODE", "strict")
    _, md_strict, _ = _scan_check_run(dtype)
    assert torch.equal(md_auto.indices, md_strict.indices) and torch.equal(md_auto.ks, md_strict.ks)
    assert torch.equal(md_check.indices, md_strict.indices)
    print(f"scan check {scan_kernel} {dtype}: keys {keys} fallbacks {fallbacks} ({100 * fallbacks / keys:.2f} %) max ratio {ratio:.4f}")


@pytest.mark.parametrize("backend", ["relative", "streaming"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_scan_tensor_core_path_is_exact_with_rope(dtype, backend, monkeypatch):
    """The same with in-kernel RoPE: "relative" (two rotated key copies) and "streaming" (keys rotated and scaled inside
    the operand tile, their magnitudes summed there) on the tcgen05 scan against the strict kernel."""
    import numpy as np
    monkeypatch.setenv("HIPATTN_SCAN_MODE", "check")
    stats, md_check, _ = _scan_check_run(dtype, rope_backend=backend)
    keys, fallbacks, wrong = int(stats[0]), int(stats[1]), int(stats[2])
    ratio = float(np.array([int(stats[3]) & 0xffffffff], dtype=np.uint32).view(np.float32)[0])
    assert keys > 800_000
    assert wrong == 0, f"{wrong} shortcuts disagree with the strict score"
    assert ratio < 0.5, f"deviation reached {ratio:.3f} of the assumed radius"
    assert fallbacks / keys < 0.25
    monkeypatch.setenv("HIPATTN_SCAN_MODE", "strict")
    _, md_strict, _ = _scan_check_run(dtype, rope_backend=backend)
    monkeypatch.setenv("HIPATTN_SCAN_MODE", "auto")
    _, md_auto, _ = _scan_check_run(dtype, rope_backend=backend)
    assert torch.equal(md_auto.indices, md_strict.indices) and torch.equal(md_auto.ks, md_strict.ks)
    assert torch.equal(md_check.indices, md_strict.indices)
    print(f"scan check rope {backend} {dtype}: keys {keys} fallbacks {fallbacks} ({100 * fallbacks / keys:.2f} %) max ratio {ratio:.4f}")


@pytest.mark.parametrize("shape", [
    dict(D=128, H=8, HKV=2, TQ=300, T=8192, strides=[4, 4, 1]),                       # 16 / 16 / 64 pooled rows, ragged block
    dict(D=64, H=4, HKV=4, TQ=256, T=4096, strides=[2, 2, 1], keep=[2048, 1024, 512]),  # 32 / 32 / 64 rows, head dim 64
    dict(D=128, H=4, HKV=1, TQ=128, T=1504, strides=[4, 2, 4], keep=[1024, 512, 256]),   # few chunks: groups of 16 and 32
    dict(D=128, H=4, HKV=2, B=2, TQ=192, T=6000, strides=[1, 4, 2], keep=[4096, 1024, 512], bq=64),
])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_scan_kernels_agree(shape, dtype, monkeypatch):
    """The scan kernels (tcgen05, mma.sync, strict) give
    identical per-head bounds and scores at every stage, dense and through a permuted page pool."""
    import bench
    from cases import make_paged
    from hip_attention_b200 import hip_attention_impl, read_status
    w = dict(bench.WORKLOADS["prefill_128k"], keep=[4096, 2048, 1024], **{k_: v_ for k_, v_ in shape.items() if k_ != "keep"})
    if "keep" in shape:
        w["keep"] = shape["keep"]
    w["dtype"] = {torch.bfloat16: "bf16", torch.float16: "fp16"}[dtype]
    q, k, v = bench.make_qkv(w, "cuda")
    results = {}
    for name, env in (("auto", {"HIPATTN_SCAN_KERNEL": "auto", "HIPATTN_SCAN_MODE": "auto"}),
                      ("mma", {"HIPATTN_SCAN_KERNEL": "mma", "HIPATTN_SCAN_MODE": "auto"}),
                      ("strict", {"HIPATTN_SCAN_KERNEL": "auto", "HIPATTN_SCAN_MODE": "strict"})):
        for k_, v_ in env.items():
            monkeypatch.setenv(k_, v_)
        dbg = {}
        read_status("cuda")
        out, md = hip_attention_impl(q, k, v, bench.make_args(w), debug=dbg)
        torch.cuda.synchronize()
        assert read_status("cuda") == 0
        results[name] = (dbg["stages"], md)
    # the same problem through a paged cache, default kernel
    monkeypatch.setenv("HIPATTN_SCAN_MODE", "auto")
    monkeypatch.setenv("HIPATTN_SCAN_KERNEL", "auto")
    kc, vc, table = make_paged(k.cpu(), v.cpu(), 16, 7)
    args = bench.make_args(w, k_cache=kc.cuda(), v_cache=vc.cuda(), block_table=table.cuda().to(torch.int32),
                           cache_seq_lens=torch.full((w["B"],), w["T"], dtype=torch.int32, device="cuda"),
                           extend_context_length=w["T"])
    out_p, md_p = hip_attention_impl(q, None, None, args)
    ref_st, ref_md = results["strict"]
    for name in ("auto", "mma"):
        st, md = results[name]
        assert len(st) == len(ref_st)
        for i, (a, b_) in enumerate(zip(st, ref_st)):
            for key in ("left", "right", "score", "score_max"):
                assert torch.equal(a[key], b_[key]), f"{name}: stage {i} {key} differs from the strict kernel"
        assert torch.equal(md.indices, ref_md.indices) and torch.equal(md.ks, ref_md.ks)
    assert torch.equal(md_p.indices, ref_md.indices) and torch.equal(md_p.ks, ref_md.ks)


@pytest.mark.parametrize("kernel", ["tcgen05", "mma"])
@pytest.mark.parametrize("bq,tq,hkv", [(64, 300, 2), (128, 300, 2), (64, 64, 4), (64, 1024, 1)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_prefill_head_dim_128_matches_oracle(kernel, bq, tq, hkv, dtype, monkeypatch):
    """Head dim 128 (the shape of the benchmark configs): both tensor-core prefill kernels against the
    fp64 recompute on the oracle's mask, ragged last block included."""
    import bench
    from hip_attention_b200 import hip_attention_impl, read_status
    monkeypatch.setenv("HIPATTN_PREFILL_KERNEL", kernel)
    w = dict(bench.WORKLOADS["prefill_128k"], TQ=tq, T=4096, H=8, HKV=hkv, bq=bq, keep=[2048, 1024, 512], sink=64, sw=256,
             dtype={torch.bfloat16: "bf16", torch.float16: "fp16"}[dtype])
    q, k, v = bench.make_qkv(w, "cuda")
    read_status("cuda")
    out, md, lse = hip_attention_impl(q, k, v, bench.make_args(w), return_lse=True)
    torch.cuda.synchronize()
    assert read_status("cuda") == 0
    cfg = bench.oracle_config(w)
    pos = (torch.arange(tq) + w["T"] - tq)[None]
    qc, kc, vc = q.cpu(), k.cpu(), v.cpu()
    m = O.estimate_mask(qc, O.DenseKV(kc), pos, cfg)
    assert torch.equal(md.indices.cpu(), m.indices) and torch.equal(md.ks.cpu(), m.ks)
    ref, lse_ref = O.attention_on_mask(qc, O.DenseKV(kc), O.DenseKV(vc), pos, m, sink=cfg.sink,
                                       sw=max(cfg.sw, cfg.stages[0].chunk_size), return_lse=True)
    _check_out(out, ref, dtype)
    assert (lse.cpu().double() - lse_ref).abs().max().item() < 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [
    dict(B=3, H=8, HKV=2, D=128, T=8192),                                  # four heads per KV head: chunk 32 and chunk 8
    dict(B=2, H=4, HKV=2, D=64, T=4096, keep=[2048, 1024, 512]),           # two heads per KV head: only chunk 8 qualifies
    dict(B=2, H=3, HKV=3, D=128, T=5000, keep=[4096, 1024, 512]),          # one head per KV head, ragged last chunk
])
@pytest.mark.parametrize("rope", [False, True])
def test_decode_scan_whole_chunks_equals_rounds(shape, dtype, rope, monkeypatch):
    """Decode: scoring whole small chunks once per KV head and replaying the search gives the per-head bounds
    and scores of the round-by-round strict kernel at every stage, dense and paged; also with in-kernel RoPE, scan
    backend "streaming" (every token of a chunk rotated to the chunk's index)."""
    import bench
    from cases import make_paged, rope_tables
    from hip_attention_b200 import hip_attention_impl, read_status
    w = dict(bench.WORKLOADS["decode_128k"], keep=[4096, 2048, 1024], **{k_: v_ for k_, v_ in shape.items() if k_ != "keep"})
    if "keep" in shape:
        w["keep"] = shape["keep"]
    w["dtype"] = {torch.bfloat16: "bf16", torch.float16: "fp16", torch.float32: "fp32"}[dtype]
    w["kind"] = "prefill"          # dense q / k / v tensors from the generator
    q, k, v = bench.make_qkv(w, "cuda")
    kw = {}
    if rope:
        cos, sin = rope_tables(w["T"] + 8, w["D"], w["theta"])
        kw = dict(using_extend=True, need_apply_rope=True, rope_cos=torch.from_numpy(cos).cuda(), rope_sin=torch.from_numpy(sin).cuda(),
                  scan_extend_backend="streaming")
    results = {}
    for name in ("chunks", "rounds"):
        monkeypatch.setenv("HIPATTN_DECODE_SCAN", name)
        dbg = {}
        read_status("cuda")
        out, md = hip_attention_impl(q, k, v, bench.make_args(w, **kw), debug=dbg)
        torch.cuda.synchronize()
        assert read_status("cuda") == 0
        results[name] = (dbg["stages"], md, out)
    for i, (a, b_) in enumerate(zip(results["chunks"][0], results["rounds"][0])):
        for key in ("left", "right", "score", "score_max"):
            assert torch.equal(a[key], b_[key]), f"stage {i} {key}"
    assert torch.equal(results["chunks"][1].indices, results["rounds"][1].indices)
    assert torch.equal(results["chunks"][2], results["rounds"][2])
    if w["T"] % 16 == 0:
        monkeypatch.setenv("HIPATTN_DECODE_SCAN", "chunks")
        kc, vc, table = make_paged(k.cpu(), v.cpu(), 16, 11)
        args = bench.make_args(w, k_cache=kc.cuda(), v_cache=vc.cuda(), block_table=table.cuda().to(torch.int32),
                               cache_seq_lens=torch.full((w["B"],), w["T"], dtype=torch.int32, device="cuda"),
                               extend_context_length=w["T"], **kw)
        out_p, md_p = hip_attention_impl(q, None, None, args)
        assert torch.equal(md_p.indices, results["rounds"][1].indices)
        assert torch.equal(out_p, results["rounds"][2])


def test_values_may_arrive_after_the_call_is_issued():
    """The estimator reads q and k only: with ``v_ready`` the call is issued before v has been copied in on
    another stream, and gives the result of the plain call."""
    import bench
    from hip_attention_b200 import hip_attention_impl
    w = dict(bench.WORKLOADS["prefill_128k"], TQ=256, T=8192, H=8, HKV=2, keep=[4096, 2048, 1024])
    q, k, v = bench.make_qkv(w, "cuda")
    args = bench.make_args(w)
    ref, _ = hip_attention_impl(q, k, v, args)
    torch.cuda.synchronize()
    hv = v.cpu().pin_memory()
    dv = torch.zeros_like(v)
    side = torch.cuda.Stream()
    ev = torch.cuda.Event()
    with torch.cuda.stream(side):
        torch.cuda._sleep(20_000_000)            # the copy starts well after the call below has been issued
        dv.copy_(hv, non_blocking=True)
        ev.record(side)
    out, _ = hip_attention_impl(q, k, dv, args, v_ready=ev)
    torch.cuda.synchronize()
    assert torch.equal(out, ref)


def test_decode_under_cuda_graph_capture():
    """With position_ids given the operator makes no host synchronisation, so a decode step (mask
    refresh or cached mask) can be captured in a CUDA graph and replayed on new queries
    (reference: attention_extend.py:1980-1982, tests/v1_2/test_attention_decode_bsa.py:66-101)."""
    from hip_attention_b200 import hip_attention_12, read_status
    q, k, v, pos, c, cfg, _ = case_inputs("decode_fp16", torch.bfloat16)
    dev = "cuda"
    k, v, pos = k.to(dev), v.to(dev), pos.to(dev)
    q_static = q.to(dev).clone()
    read_status(dev)
    args = make_args(c, pos)
    eager_out, eager_md = hip_attention_12(q_static, k, v, args)          # also warms allocations
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        hip_attention_12(q_static, k, v, args)
        hip_attention_12(q_static, k, v, args, cached_metadata=eager_md)
    torch.cuda.current_stream().wait_stream(side)
    g_refresh, g_cached = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
    with torch.cuda.graph(g_refresh):
        out_r, md_r = hip_attention_12(q_static, k, v, args)
    with torch.cuda.graph(g_cached):
        out_c, _ = hip_attention_12(q_static, k, v, args, cached_metadata=md_r)
    q2 = torch.roll(q.to(dev), 5, dims=-1).contiguous()
    q_static.copy_(q2)
    g_refresh.replay()
    g_cached.replay()
    torch.cuda.synchronize()
    ref_out, ref_md = hip_attention_12(q2, k, v, args)
    assert torch.equal(md_r.indices, ref_md.indices)
    assert torch.equal(out_r, ref_out) and torch.equal(out_c, ref_out)
    assert read_status(dev) == 0


@pytest.mark.parametrize("kernel", ["tcgen05_ws", "tcgen05", "mma"])
def test_prefill_head_dim_128_softcap(kernel, monkeypatch):
    """Soft-capped logits on the tensor-core prefill kernels (the capped path also applies the admission
    rule per element)."""
    import bench
    from hip_attention_b200 import hip_attention_impl
    monkeypatch.setenv("HIPATTN_PREFILL_KERNEL", kernel)
    w = dict(bench.WORKLOADS["prefill_128k"], TQ=200, T=4096, H=8, HKV=2, keep=[2048, 1024, 512], sink=64, sw=256)
    q, k, v = bench.make_qkv(w, "cuda")
    args = bench.make_args(w, logit_softcap=1.5)
    out, md = hip_attention_impl(q, k, v, args)
    cfg = bench.oracle_config(w)
    cfg.softcap = 1.5
    pos = (torch.arange(200) + w["T"] - 200)[None]
    ref, m = O.hip_attention_oracle(q.cpu(), k.cpu(), v.cpu(), pos, cfg)
    assert torch.equal(md.indices.cpu(), m.indices)
    _check_out(out, ref, torch.bfloat16)


def test_bounded_wait_times_out_and_reports():
    """A wait nothing satisfies ends by itself: the kernel returns, the status word carries the time-out
    bit, and the device keeps working."""
    import time
    from hip_attention_b200 import _lib as L, read_status
    from hip_attention_b200.operator import status_word
    lib = L.load()
    read_status("cuda")
    t0 = time.perf_counter()
    L.check(lib.hipattn_debug_bounded_wait(status_word("cuda").data_ptr(), torch.cuda.current_stream().cuda_stream), "probe")
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert read_status("cuda") & L.STATUS_TIMEOUT
    assert dt < 2.0
    x = torch.ones(1024, device="cuda")
    assert float(x.sum()) == 1024.0
    assert read_status("cuda") == 0


@pytest.mark.parametrize("cfg", [
    dict(H=8, HKV=2, bq=64, T=8192, TQ=300, sink=64, sw=1024, dt="bf16", rope=None),
    dict(H=16, HKV=2, bq=128, T=12000, TQ=192, sink=256, sw=512, dt="fp16", rope="streaming"),
    dict(H=8, HKV=1, bq=64, T=8192, TQ=64, sink=16, sw=1024, dt="bf16", rope="streaming"),
    dict(H=4, HKV=4, bq=128, T=4096, TQ=100, sink=0, sw=1024, dt="fp16", rope="relative"),
    dict(H=8, HKV=2, bq=64, T=4096, TQ=2048, sink=256, sw=128, dt="bf16", rope="relative"),
    dict(H=16, HKV=2, bq=128, T=16384, TQ=192, sink=0, sw=128, dt="fp16", rope=None),
    dict(H=8, HKV=2, bq=128, T=2048, TQ=512, sink=16, sw=1024, dt="bf16", rope=None),
    dict(H=8, HKV=2, bq=64, T=2048, TQ=64, sink=16, sw=64, dt="fp16", rope=None),
])
def test_prefill_attention_kernels_agree_and_repeat(cfg, monkeypatch):
    """The warp-specialised tcgen05 attention kernel against the mma.sync one on assorted shapes (one / two heads per
    CTA, 64- and 128-row blocks, ragged blocks, sink-less, with and without in-kernel RoPE): outputs within two
    element-type roundings, the status word clean, and every repeat of the call bit-identical (the kernel's roles meet
    on mbarriers only; a missed hand-off would show as a difference between repeats)."""
    import bench
    from cases import rope_tables
    from hip_attention_b200 import hip_attention_impl, read_status
    T = cfg["T"]
    w = dict(bench.WORKLOADS["prefill_128k"], TQ=cfg["TQ"], T=T, H=cfg["H"], HKV=cfg["HKV"], bq=cfg["bq"], sink=cfg["sink"],
             sw=cfg["sw"], dtype=cfg["dt"], keep=[min(4096, T // 2), min(2048, T // 4), min(1024, T // 8)], seed=77,
             strides=[4, 4, 1] if cfg["bq"] == 64 else [4, 4, 2])
    q, k, v = bench.make_qkv(w, "cuda")
    kw = {}
    if cfg["rope"]:
        cos, sin = rope_tables(T + 8, w["D"], w["theta"])
        kw = dict(using_extend=True, need_apply_rope=True, rope_cos=torch.from_numpy(cos).cuda(), rope_sin=torch.from_numpy(sin).cuda(),
                  scan_extend_backend=cfg["rope"])
    args = bench.make_args(w, **kw)
    monkeypatch.setenv("HIPATTN_PREFILL_KERNEL", "tcgen05")
    read_status("cuda")
    out, md = hip_attention_impl(q, k, v, args)
    for _ in range(3):
        again, _ = hip_attention_impl(q, k, v, args, md)
        assert torch.equal(again, out)
    assert read_status("cuda") == 0
    monkeypatch.setenv("HIPATTN_PREFILL_KERNEL", "mma")
    ref, _ = hip_attention_impl(q, k, v, args, md)
    assert torch.isfinite(out.float()).all()
    assert (out.float() - ref.float()).abs().max().item() <= (4e-2 if cfg["dt"] == "bf16" else 5e-3)
