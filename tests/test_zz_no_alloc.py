"""The allocation-free decode entry point against the regular one.

``hipattn_bsa_decode_noalloc`` exists for hosts that must not allocate device memory while they run
(a server that gave all of it to its KV-cache pool, a plugin that only ever receives pointers).  It
keeps the per-split partial results in an array inside the library instead of caller-provided
buffers.  Here it is called through the C ABI twice in a row -- the second call finds the first
call's leftovers in that array -- and each result must equal what ``hipattn_bsa_attention`` +
``hipattn_merge_partials`` produce with ordinary torch-allocated buffers.  Both paths launch the same
kernels on the same data, so the outputs are compared exactly.

This file sorts last on purpose: a run that stops at the first failure has then already run every
other test.
"""
import ctypes as C

import pytest
import torch

from util import case_inputs, make_args

pytestmark = pytest.mark.gpu


def _decode_problem(dtype, seed_shift=0):
    """Mask + tensors of a small decode step, produced by the regular operator."""
    from hip_attention_b200 import hip_attention_12
    q, k, v, pos, c, cfg, _ = case_inputs("decode_fp16", dtype)
    if seed_shift:
        q = torch.roll(q, seed_shift, dims=-1).contiguous()
    dev = "cuda"
    q, k, v, pos = q.to(dev), k.to(dev), v.to(dev), pos.to(dev)
    _, md = hip_attention_12(q, k, v, make_args(c, pos))
    return q, k, v, pos, c, md


def _params(q, k, v, pos, c, md, out, n_splits):
    from hip_attention_b200 import _lib as L
    from hip_attention_b200.operator import _DT, _tokens, status_word
    B, TQ, H, D = q.shape
    bp = L.BsaParams()
    bp.q, bp.q_stride_b, bp.q_stride_t, bp.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1), q.stride(2)
    bp.out, bp.o_stride_b, bp.o_stride_t, bp.o_stride_h = out.data_ptr(), out.stride(0), out.stride(1), out.stride(2)
    bp.pos, bp.pos_stride_b, bp.pos_stride_t = pos.data_ptr(), pos.stride(0), pos.stride(1)
    bp.k, bp.v = _tokens(k, None, None, None, "k"), _tokens(v, None, None, None, "v")
    bp.indices, bp.idx_stride_n, bp.idx_stride_d = md.indices.data_ptr(), md.indices.stride(0), md.indices.stride(1)
    bp.ks, bp.ks_stride_n, bp.ks_stride_d = md.ks.data_ptr(), md.ks.stride(0), md.ks.stride(1)
    bp.status = status_word(q.device).data_ptr()
    bp.dtype, bp.D, bp.B, bp.TQ, bp.H, bp.HKV, bp.T = _DT[q.dtype], D, B, TQ, H, k.shape[2], k.shape[1]
    bp.block_size_q, bp.index_block_q = 1, c["stages"][-1][0]
    bp.block_size_k, bp.K = c["stages"][-1][2], md.indices.shape[-1]
    bp.sink, bp.window = c["sink"], max(c["sw"], c["stages"][0][2])
    bp.n_splits, bp.heads_share_mask, bp.logit_softcap = n_splits, 1, 0.0
    return bp


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_noalloc_decode_equals_regular_entry_point_twice(dtype):
    from hip_attention_b200 import _lib as L
    lib = L.load()
    n_splits = 4
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):  # the second call reuses the array the first one filled
        q, k, v, pos, c, md = _decode_problem(dtype, seed_shift=call * 3)
        B, TQ, H, D = q.shape
        # regular path: caller-provided scratch
        ref = torch.empty_like(q)
        part_o = torch.empty((B, H, n_splits, D), dtype=torch.float32, device=q.device)
        part_lse = torch.empty((B, H, n_splits), dtype=torch.float32, device=q.device)
        bp = _params(q, k, v, pos, c, md, ref, n_splits)
        bp.part_o, bp.part_lse = part_o.data_ptr(), part_lse.data_ptr()
        L.check(lib.hipattn_bsa_attention(C.byref(bp), stream), "bsa_attention")
        ref_lse = torch.empty((B, TQ, H), dtype=torch.float32, device=q.device)
        L.check(lib.hipattn_merge_partials(part_o.data_ptr(), part_lse.data_ptr(), B * H, n_splits, D, bp.dtype,
                                           ref.data_ptr(), D, ref_lse.data_ptr(), stream), "merge_partials")
        # allocation-free path: outputs only
        out = torch.empty_like(q)
        lse = torch.empty((B, TQ, H), dtype=torch.float32, device=q.device)
        bp2 = _params(q, k, v, pos, c, md, out, n_splits)
        bp2.lse_out = lse.data_ptr()
        before = torch.cuda.memory_allocated()
        L.check(lib.hipattn_bsa_decode_noalloc(C.byref(bp2), stream), "bsa_decode_noalloc")
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        assert torch.equal(out, ref), f"call {call}: max diff {(out.float() - ref.float()).abs().max().item()}"
        assert torch.isfinite(lse).all() and torch.equal(lse, ref_lse)
        assert out.float().abs().max().item() > 0


def test_noalloc_decode_single_range_bypasses_the_array():
    """With one key range there are no partial results: the call goes straight to the regular kernel and must
    give what ``hipattn_bsa_attention`` gives, log-sum-exp included."""
    from hip_attention_b200 import _lib as L
    lib = L.load()
    stream = torch.cuda.current_stream().cuda_stream
    q, k, v, pos, c, md = _decode_problem(torch.bfloat16)
    B, TQ, H, D = q.shape
    ref, out = torch.empty_like(q), torch.empty_like(q)
    ref_lse = torch.empty((B, TQ, H), dtype=torch.float32, device=q.device)
    lse = torch.empty_like(ref_lse)
    bp = _params(q, k, v, pos, c, md, ref, 1)
    bp.lse_out = ref_lse.data_ptr()
    L.check(lib.hipattn_bsa_attention(C.byref(bp), stream), "bsa_attention")
    bp2 = _params(q, k, v, pos, c, md, out, 1)
    bp2.lse_out = lse.data_ptr()
    L.check(lib.hipattn_bsa_decode_noalloc(C.byref(bp2), stream), "bsa_decode_noalloc")
    torch.cuda.synchronize()
    assert torch.equal(out, ref) and torch.equal(lse, ref_lse)


def test_noalloc_decode_rejects_oversized_requests():
    from hip_attention_b200 import _lib as L
    lib = L.load()
    q, k, v, pos, c, md = _decode_problem(torch.bfloat16)
    out = torch.empty_like(q)
    bp = _params(q, k, v, pos, c, md, out, 4)
    bp.B = 1 << 20  # B * H * n_splits * (D + 1) floats is far beyond the built-in array
    rc = lib.hipattn_bsa_decode_noalloc(C.byref(bp), torch.cuda.current_stream().cuda_stream)
    assert rc == 2
    assert b"exceeds the built-in scratch" in lib.hipattn_error_string()
    bp = _params(q, k, v, pos, c, md, out, 4)
    bp.TQ = 2
    assert lib.hipattn_bsa_decode_noalloc(C.byref(bp), None) == 1
    # the other refusals: more key ranges than the merge supports, no output, an output that is not contiguous
    bp = _params(q, k, v, pos, c, md, out, 65)
    assert lib.hipattn_bsa_decode_noalloc(C.byref(bp), None) == 1
    bp = _params(q, k, v, pos, c, md, out, 4)
    bp.out = None
    assert lib.hipattn_bsa_decode_noalloc(C.byref(bp), None) == 1
    wide = torch.empty(q.shape[:-1] + (2 * q.shape[-1],), dtype=q.dtype, device=q.device)
    bp = _params(q, k, v, pos, c, md, wide[..., : q.shape[-1]], 4)
    assert bp.o_stride_h != q.shape[-1]
    assert lib.hipattn_bsa_decode_noalloc(C.byref(bp), None) == 1
