"""The CUDA path against the reference's own Triton kernels on the same GPU, in bf16 and head dim 128.

The reference (an unmodified copy under ``baseline/_ref``, see ``baseline/reference_loader.py``) orders equal scores
arbitrarily and accumulates its dot products in tensor-core order, while this project fixes both (lower position
first; sequential fp32).  The masks therefore need not be bit-identical: decisions whose scores differ by less than
a rounding step of the element type may fall either way.  What is required: nearly all (head, query block) rows
carry the identical block set, the sets overlap almost completely over all rows, and the outputs agree within the
bf16 output tolerance.  Skipped where no copy of the reference is present.
"""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "baseline"))
import reference_loader as R  # noqa: E402

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not R.available(), reason="no copy of the reference under baseline/_ref")]


@pytest.fixture(scope="module")
def reference():
    return R.load_reference()


@pytest.mark.parametrize("shape", [dict(TQ=1024, T=16384), dict(TQ=1, T=16384, B=4)])
def test_bf16_head_dim_128_against_the_triton_reference(reference, shape):
    import bench
    from hip_attention_b200 import hip_attention_impl, read_status
    op, Args, ScanStage = reference
    w = dict(bench.WORKLOADS["prefill_128k"], keep=[4096, 2048, 1024], **shape)
    q, k, v = bench.make_qkv(w, "cuda")
    ra = R.reference_args(Args, ScanStage, bq=w["bq"], strides=w["strides"], chunks=w["chunks"], keep=w["keep"],
                          sink=w["sink"], sw=w["sw"])
    o_ref, md_ref = op(q, k, v, args=ra)
    read_status("cuda")
    o, md = hip_attention_impl(q, k, v, bench.make_args(w))
    torch.cuda.synchronize()
    assert read_status("cuda") == 0
    assert md.indices.shape == md_ref.indices.shape and md.indices.dtype == md_ref.indices.dtype
    assert md.ks.shape == md_ref.ks.shape and md.ks_start_end.dtype == md_ref.ks_start_end.dtype
    ag = bench.mask_agreement(md, md_ref, o, o_ref)
    print("agreement with the Triton reference:", shape, ag)
    assert ag["block_overlap"] >= 0.97, ag
    # Two bf16 results are compared here, and the reference multiplies q by D^(1/4) and k by D^(-1/4) and rounds both
    # to bf16 before the dot product (attention_extend_bsa.py:497-509), which moves its logits by up to 2^-8 of their
    # size; this project's output is held to max-abs 2e-2 / mean-abs 2e-3 against the fp64 recompute in the parity
    # tests.  Between the two implementations the bounds are therefore wider.
    assert ag["out_mean_abs"] <= 4e-3, ag
    assert ag["out_max_abs"] <= 1e-1, ag
    # the reference accepts this project's metadata and reproduces this project's output on it
    o2, _ = op(q, k, v, args=ra, cached_metadata=md)
    d = (o2.float() - o.float()).abs()
    assert d.max().item() <= 1e-1 and d.mean().item() <= 4e-3
