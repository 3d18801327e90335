"""Helpers shared by the parity tests."""
import torch

from cases import CASES, make_inputs, make_paged
from oracle import hip_oracle as O


def make_args(c, pos=None, **kw):
    from hip_attention_b200 import HiPAttentionArgs, ScanStage
    sb = c.get("stage_backends") or [None] * len(c["stages"])
    if "rope_in_kernel" in c:
        from cases import rope_tables
        dev = pos.device if pos is not None else "cpu"
        cos, sin = rope_tables(max(c.get("ext", c["T"]), c["T"]) + 8, c["D"], c.get("rope_theta", 10000.0))
        kw = dict(rope_cos=torch.from_numpy(cos).to(dev), rope_sin=torch.from_numpy(sin).to(dev),
                  scan_extend_backend=c["rope_in_kernel"], sa_extend_backend="streaming", **kw)
    return HiPAttentionArgs(
        position_ids=pos, sliding_window_size=c["sw"], sink_token_size=c["sink"], block_size_k=64,
        second_stage_k=c["second_k"],
        stages=[ScanStage(stage_block_size_q=bq, stage_block_stride_q=sq, stage_chunk_size=cs, stage_k=sk, stage_stride=1,
                          stage_extend_backend=sb[i]) for i, (bq, sq, cs, sk) in enumerate(c["stages"])],
        block_sparse_block_size_q=c.get("bsa_bq", c["stages"][-1][0]), using_extend="rope_in_kernel" in c,
        need_apply_rope="rope_in_kernel" in c,
        disable_flashdecode=c.get("disable_flashdecode", False), logit_softcap=c.get("softcap"), **kw)


def case_inputs(name, dtype=None):
    """(q, k, v, pos, case, cfg, paged) on the CPU; ``dtype`` overrides the case's element type."""
    q, k, v, pos, c = make_inputs(name)
    if dtype is not None and dtype != q.dtype:
        # re-round from the fp32 draw so that the new type is not a double rounding of the old one
        c = dict(c)
        dn = {torch.float32: "fp32", torch.float16: "fp16", torch.bfloat16: "bf16"}[dtype]
        import cases as cs
        saved = cs.CASES[name]
        cs.CASES[name] = dict(saved, dtype=dn)
        try:
            q, k, v, pos, c = make_inputs(name)
        finally:
            cs.CASES[name] = saved
    cfg = O.config_from_case(c)
    paged = None
    if "page" in c:
        kc, vc, table = make_paged(k, v, c["page"], c["seed"])
        paged = (kc, vc, table, torch.full((c["B"],), c["T"], dtype=torch.int64), c["ext"])
    return q, k, v, pos, c, cfg, paged


def run_gpu(q, k, v, pos, c, paged, dev="cuda", **kw):
    from hip_attention_b200 import hip_attention_impl
    if paged is not None:
        kc, vc, table, seq, ext = paged
        args = make_args(c, pos.to(dev), k_cache=kc.to(dev), v_cache=vc.to(dev), block_table=table.to(dev),
                         cache_seq_lens=seq.to(dev), extend_context_length=ext)
        return hip_attention_impl(q.to(dev), None, None, args, **kw)
    if c.get("kv_fp8") and q.dtype != torch.float32:
        k, v = k.to(torch.float8_e5m2), v.to(torch.float8_e5m2)
    return hip_attention_impl(q.to(dev), k.to(dev), v.to(dev), make_args(c, pos.to(dev)), **kw)


def output_tolerance(dtype):
    """(max-abs, mean-abs) bound of the attention output against a high-precision recompute on the
    same mask: the bf16 contract is max-abs <= 2e-2 and mean-abs <= 2e-3; fp32 must be near exact."""
    if dtype == torch.float32:
        return 2e-5, 2e-6
    return 2e-2, 2e-3
