"""Generate the golden fixtures in this directory by running the reference operator.

Usage (only where the reference checkout is available; it is not needed to run the tests):

    python tests/golden/gen_golden.py --reference /path/to/hip-attention [case ...]

The reference is imported unmodified through a namespace shim (its package ``__init__``
pulls in GPU-only dependencies) and executed on the CPU with ``TRITON_INTERPRET=1``.
The interpreter has no bf16, so the cases use fp32 and fp16.

The reference orders equal scores with ``topk(sorted=False)`` / ``sort(stable=False)``, which is
implementation-defined.  Unless ``--native-ties`` is given, ``torch.Tensor.topk`` and
``torch.Tensor.sort`` are wrapped for the duration of the call so that equal scores keep their
positional order (lower chunk position first) -- the tie rule this project fixes.  Cases without
tied scores give byte-identical fixtures either way.  For every case the script
stores ``indices``, ``ks``, ``ks_count``, ``ks_start_end``, the stage-input caches and the
attention output (optionally a strided subset of query rows) in ``<case>.npz``.
"""
from __future__ import annotations

import argparse
import os
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))


def _import_reference(ref_root: str):
    os.environ["TRITON_INTERPRET"] = "1"
    os.environ["HIP_DISABLE_AUTOTUNE"] = "1"
    os.environ["HIP_DISABLE_AUTOTUNE_WARNINGS"] = "1"
    tmp = tempfile.mkdtemp(prefix="hipref_shim_")
    os.makedirs(f"{tmp}/shim/hip_attn")
    with open(f"{tmp}/shim/hip_attn/__init__.py", "w") as f:
        f.write(f"__path__ = [{os.path.join(ref_root, 'src', 'hip_attn')!r}]\n")
    for mod in ("matplotlib/__init__.py", "matplotlib/pyplot.py", "cupy/__init__.py", "nvtx.py"):
        p = f"{tmp}/stubs/{mod}"
        os.makedirs(os.path.dirname(p), exist_ok=True)
        open(p, "w").close()
    sys.path[:0] = [f"{tmp}/shim", f"{tmp}/stubs"]
    import torch

    torch.cuda.is_current_stream_capturing = lambda: False
    torch.cuda.current_device = lambda: 0
    torch.cuda.set_device = lambda d: None
    torch.cuda.get_device_name = lambda *a: "cpu"
    # the interpreter cannot run libdevice intrinsics: give it tanh (used by the logit soft-cap) in
    # terms of operations it can run; on a GPU the reference calls the libdevice function
    import triton.language as tl

    def _tanh(x, _semantic=None):
        e = tl.exp(2.0 * x)
        return (e - 1.0) / (e + 1.0)

    tl.extra.cuda.libdevice.tanh = _tanh
    import hip_attn.v1_2.attention_extend as ext
    from hip_attn.v1_2.attention_metadata import HiPAttentionArgs, ScanStage

    return ext.dual_stage_quadratic_hip_attention, HiPAttentionArgs, ScanStage


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of DeepAuto-AI/hip-attention")
    ap.add_argument("--native-ties", action="store_true", help="keep torch's own order among equal scores")
    ap.add_argument("--out", default=HERE)
    ap.add_argument("cases", nargs="*")
    a = ap.parse_args()
    op, Args, ScanStage = _import_reference(a.reference)
    sys.path.insert(0, HERE)
    import numpy as np
    import torch
    from cases import CASES, make_inputs, make_paged

    if not a.native_ties:
        _sort = torch.Tensor.sort
        _topk = torch.Tensor.topk

        def stable_sort(self, *args, **kw):
            kw["stable"] = True
            return _sort(self, *args, **kw)

        def stable_topk(self, k, dim=-1, largest=True, sorted=True):
            r = _sort(self, dim=dim, descending=largest, stable=True)
            return torch.return_types.topk((r.values.narrow(dim, 0, k), r.indices.narrow(dim, 0, k)))

        torch.Tensor.sort = stable_sort
        torch.Tensor.topk = stable_topk

    names = a.cases or list(CASES)
    for name in names:
        q, k, v, pos, c = make_inputs(name)

        rope_kw = {}
        if "rope_in_kernel" in c:
            from cases import rope_tables
            cos, sin = rope_tables(max(c.get("ext", c["T"]), c["T"]) + 8, c["D"], c.get("rope_theta", 10000.0))
            rope_kw = dict(rope_cos=torch.from_numpy(cos), rope_sin=torch.from_numpy(sin), scan_extend_backend=c["rope_in_kernel"],
                           sa_extend_backend="streaming")
        sb = c.get("stage_backends") or [None] * len(c["stages"])

        def mk(**kw):
            kw = {**rope_kw, **kw}
            return Args(
                position_ids=pos, sliding_window_size=c["sw"], sink_token_size=c["sink"], block_size_k=64,
                second_stage_k=c["second_k"],
                stages=[ScanStage(stage_block_size_q=bq, stage_block_stride_q=sq, stage_chunk_size=cs,
                                  stage_k=sk, stage_stride=1, stage_extend_backend=sb[i])
                        for i, (bq, sq, cs, sk) in enumerate(c["stages"])],
                block_sparse_block_size_q=c.get("bsa_bq", c["stages"][-1][0]), using_extend="rope_in_kernel" in c,
                need_apply_rope="rope_in_kernel" in c,
                disable_flashdecode=c.get("disable_flashdecode", False), logit_softcap=c.get("softcap"), **kw)

        t0 = time.time()
        if "page" in c:
            kc, vc, table = make_paged(k, v, c["page"], c["seed"])
            args = mk(k_cache=kc, v_cache=vc, block_table=table,
                      cache_seq_lens=torch.full((c["B"],), c["T"], dtype=torch.int64),
                      extend_context_length=c["ext"])
            out, md = op(q, None, None, args=args)
        else:
            args = mk()
            if c.get("kv_fp8"):   # the 1-byte form the serving adapter hands over (paged_hip.py:409-418)
                k, v = k.to(torch.float8_e5m2).view(torch.uint8), v.to(torch.float8_e5m2).view(torch.uint8)
            out, md = op(q, k, v, args=args)
        el = time.time() - t0
        rs = c.get("out_row_stride", 1)
        save = dict(
            indices=md.indices.numpy(), ks=md.ks.numpy(), ks_count=md.ks_count.numpy(),
            ks_start_end=md.ks_start_end.numpy(), out=out.float().numpy()[:, ::rs],
            n_stage_caches=np.int64(len(md.stage_caches)),
        )
        for nm, st in (("mask", md.mask_cache_statistics), ("sa", md.sa_cache_statistics)):
            if c.get("stats") and st is not None and st.access_counter is not None:
                save[f"{nm}_access"] = st.access_counter.numpy()
                save[f"{nm}_miss"] = st.cache_miss_counter.numpy()
        for i, sc in enumerate(md.stage_caches):
            if sc.indices_left is not None:
                save[f"stage{i}_left"] = sc.indices_left.numpy()
                save[f"stage{i}_right"] = sc.indices_right.numpy()
                save[f"stage{i}_scores"] = sc.out_scores.numpy()
        # cached-mask replay: full reuse, and restart from every stage-cache prefix
        if "page" not in c and c["T"] <= 2048:
            o2, m2 = op(q, k, v, args=mk(), cached_metadata=md)
            save["out_cached_full"] = o2.float().numpy()[:, ::rs]
            for n in range(2, len(md.stage_caches) + 1):  # n == 1 crashes in the reference (stage 0 caches None)
                from hip_attn.v1_2.attention_metadata import HiPAttentionOutputMetadata
                part = HiPAttentionOutputMetadata(
                    indices=None, ks=None, ks_count=None, ks_start_end=None, mask_cache_statistics=None,
                    sa_cache_statistics=None, stage_caches=list(md.stage_caches[:n]))
                o3, m3 = op(q, k, v, args=mk(), cached_metadata=part)
                save[f"out_restart{n}"] = o3.float().numpy()[:, ::rs]
                save[f"indices_restart{n}"] = m3.indices.numpy()
        np.savez_compressed(os.path.join(a.out, f"{name}.npz"), **save)
        print(f"{name}: {el:.1f}s  indices {tuple(md.indices.shape)}  ks[0] {md.ks[0].tolist()[:8]}", flush=True)


if __name__ == "__main__":
    main()
