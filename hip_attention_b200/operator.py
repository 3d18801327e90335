"""``hip_attention_12``: hierarchical mask estimation + block-sparse attention on B200.

Host-side driver with the call signature, argument semantics, returned metadata and cached-mask
behaviour of the reference's ``dual_stage_quadratic_hip_attention``
(``src/hip_attn/v1_2/attention_extend.py:1918-3133``).  All device work goes through the C ABI of
``libhipattn_sm100.so`` (``include/hipattn.h``); torch is used for device memory and streams only.

What differs from the reference by design:

* chunk lists are kept once per (batch, query block) as int32 -- with the head max-reduce every head
  selects the same chunks -- and widened / expanded to the reference's per-head int64 layout only in
  the returned metadata;
* equal scores are ordered by chunk position (lower first), where the reference leaves it open;
* pages of any positive size are accepted;
* K smaller than ``sink + window`` (no chunk to scan) yields an empty selection instead of failing.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional, Tuple

import numpy as np
import torch
from torch import Tensor

from . import _lib as L
from .metadata import (HiPAttentionArgs, HiPAttentionCacheAccessStatistics, HiPAttentionOutputMetadata,
                       HiPAttentionStageInputCache, ScanStage)

_DT = {torch.float32: L.F32, torch.float16: L.F16, torch.bfloat16: L.BF16}
INT64_MAX = torch.iinfo(torch.int64).max
SCORE_INIT = -32000.0
_status_words = {}
# an fp8 KV cache: e5m2 values, handed over as float8_e5m2 or as the uint8 view the serving adapter makes of it
# (paged_hip.py:409-418); every value is read as the 16-bit number it converts to exactly
_FP8 = (torch.float8_e5m2, torch.uint8)
_ROPE_MODES = {"relative": L.ROPE_RELATIVE, "streaming": L.ROPE_STREAMING}


def _cdiv(a: int, b: int) -> int:
    return -(-a // b)


def _next_pow2(x: int) -> int:
    return 1 if x <= 1 else 1 << (x - 1).bit_length()


def _ptr(t: Optional[Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def status_word(device) -> Tensor:
    """Device status word (one int32 per device) the kernels OR their HIPATTN_STATUS_* bits into."""
    dev = torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    w = _status_words.get(key)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
        _status_words[key] = w
    return w


def read_status(device, reset: bool = True) -> int:
    """Synchronising read of the status word (0 = clean)."""
    w = status_word(device)
    v = int(w.item())
    if reset and v:
        w.zero_()
    return v


def scan_scales(D: int, dtype: torch.dtype) -> Tuple[float, float]:
    """Query / key scales of the scan (``attention_extend.py:924-940``), rounded to the element type."""
    s = np.sqrt(np.float32(D)).astype(np.float32)
    ss = np.sqrt(s).astype(np.float32)
    qs = torch.tensor(float(np.float32(s / ss)), dtype=torch.float32).to(dtype).float().item()
    ks = torch.tensor(float(np.float32(np.float32(1.0) / ss)), dtype=torch.float32).to(dtype).float().item()
    return qs, ks


def _tokens(dense: Optional[Tensor], cache: Optional[Tensor], table: Optional[Tensor], seq_lens: Optional[Tensor],
            what: str) -> L.Tokens:
    t = L.Tokens()
    if cache is not None:
        if cache.ndim != 4 or cache.stride(-1) != 1:
            raise ValueError(f"{what}_cache must be [n_pages, page_size, kv_heads, head_dim] with a contiguous last dim")
        if table is None or table.ndim != 2 or seq_lens is None or seq_lens.ndim != 1:
            raise ValueError("paged KV needs block_table [B, pages] and cache_seq_lens [B]")
        if table.dtype not in (torch.int32, torch.int64) or seq_lens.dtype not in (torch.int32, torch.int64):
            raise ValueError("block_table and cache_seq_lens must be int32 or int64")
        if table.stride(1) != 1:
            raise ValueError("block_table rows must be contiguous")
        if not seq_lens.is_contiguous():
            raise ValueError("cache_seq_lens must be contiguous")
        t.cache = cache.data_ptr()
        t.fp8_e5m2 = int(cache.dtype in _FP8)
        t.stride_page, t.stride_off, t.stride_ch = cache.stride(0), cache.stride(1), cache.stride(2)
        t.block_table = table.data_ptr()
        t.table_stride_b = table.stride(0)
        t.cache_seq_lens = seq_lens.data_ptr()
        t.n_pages = cache.shape[0]
        t.table_width = table.shape[1]
        t.table_is_i64 = int(table.dtype == torch.int64)
        t.seq_lens_is_i64 = int(seq_lens.dtype == torch.int64)
        t.page_size = cache.shape[1]
    else:
        if dense is None:
            raise ValueError(f"{what} is None and no {what}_cache was given")
        if dense.ndim != 4 or dense.stride(-1) != 1:
            raise ValueError(f"{what} must be [B, T, kv_heads, head_dim] with a contiguous last dim")
        t.dense = dense.data_ptr()
        t.fp8_e5m2 = int(dense.dtype in _FP8)
        t.stride_b, t.stride_t, t.stride_h = dense.stride(0), dense.stride(1), dense.stride(2)
    return t


def _rope_tables(args: HiPAttentionArgs, q: Tensor) -> Optional[Tuple[Tensor, Tensor]]:
    """cos / sin [rows, D] in q's element type, contiguous (the kernels cast the tables to the element type before
    use, ``attention_extend.py:308-321``; doing it once here is the same arithmetic)."""
    if not args.using_extend:
        return None
    D = q.shape[-1]
    out = []
    for t in (args.rope_cos, args.rope_sin):
        if t.ndim != 2 or t.shape[-1] < D // 2:
            raise ValueError(f"rope tables must be [positions, >= head_dim / 2], got {tuple(t.shape)}")
        if t.device != q.device:
            raise ValueError(f"rope table on {t.device}, q on {q.device}")
        t = t.to(q.dtype)
        if t.stride(-1) != 1 or t.stride(0) % 8 or t.data_ptr() % 16:
            t = t.contiguous()
            if t.shape[-1] % 8:
                pad = torch.zeros((t.shape[0], -(-t.shape[-1] // 8) * 8), dtype=t.dtype, device=t.device)
                pad[:, :t.shape[-1]] = t
                t = pad
        out.append(t)
    return out[0], out[1]


def _reject_unsupported(args: HiPAttentionArgs) -> None:
    if args.offload_cache is not None or args.online_update_cache:
        raise NotImplementedError("host-offloaded KV (offload_cache / online_update_cache) is not part of this build")
    if args.using_extend != args.need_apply_rope:
        raise NotImplementedError("using_extend and need_apply_rope must be set together (rotation of already rotated "
                                  "q / k, attention_extend.py:299-323, is not built)")
    if args.using_extend:
        if args.rope_cos is None or args.rope_sin is None:
            raise ValueError("using_extend needs rope_cos and rope_sin")
        if args.sa_extend_backend != "streaming":
            raise NotImplementedError(f"sa_extend_backend {args.sa_extend_backend!r} is not built (streaming)")
        for st in args.stages:
            name = getattr(st, "stage_extend_backend", None) or args.scan_extend_backend
            if name not in _ROPE_MODES:
                raise NotImplementedError(f"scan_extend_backend {name!r} is not built (relative, streaming)")
    if args.low_percent > 0 and args.low_k_ratio < 1:
        raise NotImplementedError("low_percent / low_k_ratio is dead code in the reference and is not built")
    if not args.is_causal:
        raise NotImplementedError("is_causal=False is not built")
    if args.stage_early_terminate != 1:
        raise NotImplementedError("stage_early_terminate != 1 is not built")
    if args.sliding_window_indices is not None:
        raise NotImplementedError("sliding_window_indices is not built")
    if os.getenv("HIP_HEAD_REDUCE", "1") != "1":
        raise NotImplementedError("HIP_HEAD_REDUCE=0 (per-head masks) is not built")
    for name in ("HIP_DEBUG_TOPKMEAN", "HIP_DEBUG_UNION_HEAD", "HIP_DEBUG_ADD_DELAY_WINDOW", "HIP_DEBUG_SNAP_KV",
                 "APPLY_V_DOT", "HIP_CUMSUM"):
        if os.getenv(name, "0") == "1":
            raise NotImplementedError(f"{name}=1 selects a research branch of the reference that is not built")
    if not args.stages:
        raise ValueError("args.stages is empty")
    for i, st in enumerate(args.stages):
        if not isinstance(st, ScanStage):
            raise NotImplementedError(f"stage {i}: only ScanStage is built ({type(st).__name__} given)")
        if st.stage_stride != 1:
            raise NotImplementedError("stage_stride != 1 is not built")
        # the selection kernel always realigns, resets the scores and sorts by position; the reference does
        # each only when the stage asks for it (attention_extend.py:2075-2090, 2638)
        if i > 0 and not (st.require_realign_index and st.require_reset_score and st.require_post_sort):
            raise NotImplementedError(f"stage {i}: require_realign_index / require_reset_score / require_post_sort "
                                      "= False is not built")
        if st.stage_block_size_q != args.stages[0].stage_block_size_q:
            raise NotImplementedError("all stages must use the same stage_block_size_q")
        if st.stage_block_size_q % st.stage_block_stride_q:
            raise ValueError(f"stage {i}: stage_block_size_q must be a multiple of stage_block_stride_q")
    if args.stages[0].stage_k is not None:
        raise ValueError("first stage always quadratic: stages[0].stage_k must be None")
    for i in range(1, len(args.stages)):
        prev, cur = args.stages[i - 1], args.stages[i]
        if cur.stage_k is None or cur.stage_k % prev.stage_chunk_size:
            raise ValueError(f"stage {i}: stage_k {cur.stage_k} must be a multiple of the previous chunk size")
        if prev.stage_chunk_size % cur.stage_chunk_size:
            raise ValueError(f"stage {i}: chunk size {cur.stage_chunk_size} must divide {prev.stage_chunk_size}")
    if args.second_stage_k % args.stages[-1].stage_chunk_size:
        raise ValueError("second_stage_k must be a multiple of the last stage_chunk_size")


class _Mask:
    """Internal result of the estimator."""
    __slots__ = ("indices", "ks", "ks_start_end", "stage_inputs", "heads_share")


class PhaseTimer:
    """Optional per-phase CUDA-event timing of one call (events are recorded on the current stream;
    read them with ``milliseconds()`` after a synchronise)."""

    def __init__(self):
        self.marks = []

    def mark(self, name: str) -> None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.marks.append((name, ev))

    def milliseconds(self) -> dict:
        out = {}
        for (_, e0), (name, e1) in zip(self.marks[:-1], self.marks[1:]):
            out[name] = out.get(name, 0.0) + e0.elapsed_time(e1)
        return out


def _estimate_mask(q: Tensor, ktok: L.Tokens, T: int, HKV: int, pos: Tensor, args: HiPAttentionArgs,
                   restart: Optional[Tuple[int, Tensor, Tensor]], want_stage_inputs: bool,
                   debug: Optional[dict] = None, score_reduce=None, timer: Optional[PhaseTimer] = None,
                   rope: Optional[Tuple[Tensor, Tensor]] = None, access: Optional[Tensor] = None) -> _Mask:
    """Run the scan stages.  ``score_reduce(score_int32)`` is called after every scan, before the
    selection: a KV-head-parallel caller all-reduces (MAX) the head-reduced scores there."""
    lib = L.load()
    dev = q.device
    st = _stream(dev)
    status = status_word(dev)
    B, TQ, H, D = q.shape
    stages = args.stages
    bq = stages[0].stage_block_size_q
    BDST = _cdiv(TQ, bq)
    rows = B * BDST
    sink, sw = args.sink_token_size, args.sliding_window_size
    c0 = stages[0].stage_chunk_size
    scan_window = max(0, sw - c0)
    q_scale, k_scale = scan_scales(D, q.dtype)
    i32 = dict(dtype=torch.int32, device=dev)

    out = _Mask()
    out.stage_inputs = []
    first = 0
    if restart is not None:
        first, left, right = restart
        n = left.shape[-1]
        score = torch.empty((rows, n), dtype=torch.int32, device=dev)
        score.fill_(int(lib.hipattn_encode_score(SCORE_INIT)))
        out.stage_inputs = [None] * first
    else:
        n = _cdiv(max(0, T - sink - sw), c0)
        left = torch.empty((rows, n), **i32)
        right = torch.empty((rows, n), **i32)
        score = torch.empty((rows, n), **i32)
        L.check(lib.hipattn_init_chunks(_ptr(left), _ptr(right), _ptr(score), rows, n, sink, c0, T, scan_window, st),
                "init_chunks")
    if n > L.MAX_CHUNKS:
        raise NotImplementedError(f"{n} chunks per query block exceed the on-chip selection limit of {L.MAX_CHUNKS}")

    # scaled keys and their magnitudes (error radius) for the tensor-core scan (16-bit prefill only), once per call.
    # With in-kernel RoPE the stages whose backend is "relative" get two copies (keys rotated to table position 0 / 1 for
    # the left / right candidate); "streaming" stages (a key is rotated to its chunk's index, which changes from stage to
    # stage) get the keys as they are in a head-major copy, and the scan kernel rotates and scales them in its operand
    # tile (head dim 128; other shapes stay on the strict kernel).
    key_abs = k_scaled = key_abs_plain = k_plain = None
    rope_modes = [None] * len(stages)
    if rope is not None:
        rope_modes = [_ROPE_MODES[getattr(s_, "stage_extend_backend", None) or args.scan_extend_backend] for s_ in stages]
    R_min = min(bq // s_.stage_block_stride_q for s_ in stages)
    tensor_scan = (q.dtype != torch.float32 and D in (64, 128) and min(TQ, bq) > 1 and _scan_mode() != L.SCAN_STRICT
                   and all((bq // s_.stage_block_stride_q) % 16 == 0 for s_ in stages) and R_min >= 16 and n > 0)
    sides = 1
    want_plain = False
    if tensor_scan and rope is not None:
        sides = 2
        want_plain = D == 128 and L.ROPE_STREAMING in rope_modes[first:] and B * T * HKV < 2 ** 31 - 1
        tensor_scan = L.ROPE_RELATIVE in rope_modes[first:] and 2 * B * T * HKV < 2 ** 31 - 1
    if tensor_scan or want_plain:
        if timer: timer.mark("start")
        if tensor_scan:
            key_abs = torch.empty((sides, B, HKV, T), dtype=torch.float32, device=dev)
            if sides * B * T * HKV < 2 ** 31 - 1:
                k_scaled = torch.empty((sides, B, HKV, T, D), dtype=q.dtype, device=dev)
            if rope is None:
                L.check(lib.hipattn_scan_prepare_keys(C.byref(ktok), _DT[q.dtype], D, B, T, HKV, k_scale, _ptr(key_abs),
                                                      _ptr(k_scaled), status.data_ptr(), st), "scan_prepare_keys")
            else:
                # position -1: both copies (table positions 0 and 1) from one read of the keys
                L.check(lib.hipattn_scan_prepare_keys_rope(C.byref(ktok), _DT[q.dtype], D, B, T, HKV, k_scale, rope[0].data_ptr(),
                                                           rope[1].data_ptr(), rope[0].stride(0), rope[0].shape[0], -1,
                                                           _ptr(key_abs), _ptr(k_scaled), status.data_ptr(), st),
                        "scan_prepare_keys_rope")
        if want_plain:   # scale 1: the copy holds the keys' own values
            key_abs_plain = torch.empty((B, HKV, T), dtype=torch.float32, device=dev)
            k_plain = torch.empty((B, HKV, T, D), dtype=q.dtype, device=dev)
            L.check(lib.hipattn_scan_prepare_keys(C.byref(ktok), _DT[q.dtype], D, B, T, HKV, 1.0, _ptr(key_abs_plain),
                                                  _ptr(k_plain), status.data_ptr(), st), "scan_prepare_keys")
        if timer: timer.mark("prep")

    block_chunk = args.block_size_k
    n_st = len(stages)
    c_last = stages[-1].stage_chunk_size
    per_head_final = (sink % c_last) != 0
    K = 0
    for i in range(first, n_st):
        s_i = stages[i]
        out.stage_inputs.append(None if i == 0 else ((left, right) if want_stage_inputs else None))
        if n == 0:
            break
        block_chunk = max(16, _next_pow2(min(n, block_chunk)))
        last = i == n_st - 1
        left_out = right_out = score_out = None
        if (last and per_head_final) or debug is not None:
            left_out = torch.empty((rows, H, n), **i32)
        if debug is not None:
            right_out = torch.empty((rows, H, n), **i32)
            score_out = torch.empty((rows, H, n), dtype=torch.float32, device=dev)
        sp = L.ScanParams()
        sp.q, sp.q_stride_b, sp.q_stride_t, sp.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1), q.stride(2)
        sp.pos, sp.pos_stride_b, sp.pos_stride_t = pos.data_ptr(), pos.stride(0), pos.stride(1)
        sp.k = ktok
        sp.left, sp.right, sp.score_max = _ptr(left), _ptr(right), _ptr(score)
        sp.left_out, sp.right_out, sp.score_out = _ptr(left_out), _ptr(right_out), _ptr(score_out)
        sp.status = status.data_ptr()
        if rope is None or rope_modes[i] == L.ROPE_RELATIVE:
            sp.key_abs = _ptr(key_abs)
            sp.k_scaled = _ptr(k_scaled)
            sp.k_scaled_sides = sides if k_scaled is not None else 0
        elif k_plain is not None:   # streaming: the plain copy, rotated and scaled inside the scan kernel
            sp.key_abs = _ptr(key_abs_plain)
            sp.k_scaled = _ptr(k_plain)
            sp.k_scaled_sides = 1
        sp.dtype, sp.D, sp.B, sp.TQ, sp.H, sp.HKV, sp.T = _DT[q.dtype], D, B, TQ, H, HKV, T
        sp.block_size_q, sp.stride_q = bq, s_i.stage_block_stride_q
        sp.n_chunks, sp.block_chunk, sp.scan_window = n, block_chunk, scan_window
        sp.q_scale, sp.k_scale = q_scale, k_scale
        sp.mode = _scan_mode()
        sp.chunk_size = s_i.stage_chunk_size
        if access is not None:
            sp.access_counter, sp.access_n = access.data_ptr(), access.shape[-1]
            sp.access_stride_b, sp.access_stride_h = access.stride(0), access.stride(1)
        if rope is not None:
            sp.rope_cos, sp.rope_sin = rope[0].data_ptr(), rope[1].data_ptr()
            sp.rope_stride, sp.rope_rows = rope[0].stride(0), rope[0].shape[0]
            sp.rope_mode = rope_modes[i]
        if debug is not None and "scan_stats" in debug:
            sp.stats = debug["scan_stats"].data_ptr()
        if timer: timer.mark("start")
        L.check(lib.hipattn_scan_stage(C.byref(sp), st), f"scan_stage[{i}]")
        if timer: timer.mark(f"scan{i}")
        if score_reduce is not None:
            score_reduce(score)
            if timer: timer.mark("reduce")
        if debug is not None:
            debug.setdefault("stages", []).append(dict(left_in=left, right_in=right, left=left_out, right=right_out,
                                                       score=score_out, score_max=score, block_chunk=block_chunk))
        if not last:
            nxt = stages[i + 1]
            k_keep = min(nxt.stage_k // s_i.stage_chunk_size, n)
            split = s_i.stage_chunk_size // nxt.stage_chunk_size
            n2 = k_keep * split
            if n2 > L.MAX_CHUNKS:
                raise NotImplementedError(f"{n2} chunks per query block exceed the on-chip selection limit of {L.MAX_CHUNKS}")
            nl = torch.empty((rows, n2), **i32)
            nr = torch.empty((rows, n2), **i32)
            ns = torch.empty((rows, n2), **i32)
            L.check(lib.hipattn_select_stage(_ptr(score), _ptr(left), rows, n, k_keep, sink, s_i.stage_chunk_size,
                                             nxt.stage_chunk_size, _ptr(nl), _ptr(nr), _ptr(ns), st), f"select_stage[{i}]")
            if timer: timer.mark("select")
            left, right, score, n = nl, nr, ns, n2
        else:
            K = min(args.second_stage_k // c_last, n)
            indices = torch.empty((B * H, BDST, K), dtype=torch.int64, device=dev)
            ks = torch.empty((B * H, BDST), dtype=torch.int64, device=dev)
            kse = torch.empty((B * H, BDST, 2), dtype=torch.int32, device=dev)
            if per_head_final:
                lh, row_stride, head_stride = left_out, H * n, n
            else:
                lh, row_stride, head_stride = left, n, 0
            L.check(lib.hipattn_finalize_indices(_ptr(score), _ptr(lh), row_stride, head_stride, pos.data_ptr(),
                                                 pos.stride(0), pos.stride(1), B, BDST, H, n, K, c_last, bq,
                                                 _ptr(indices), _ptr(ks), _ptr(kse), st), "finalize_indices")
            if timer: timer.mark("select")
            out.indices, out.ks, out.ks_start_end = indices, ks, kse
    if n == 0:
        # nothing to scan: K shorter than sink + window
        while len(out.stage_inputs) < n_st:
            out.stage_inputs.append(None)
        out.indices = torch.empty((B * H, BDST, 0), dtype=torch.int64, device=dev)
        out.ks = torch.zeros((B * H, BDST), dtype=torch.int64, device=dev)
        out.ks_start_end = torch.zeros((B * H, BDST, 2), dtype=torch.int32, device=dev)
    out.heads_share = not per_head_final
    return out


def _scan_mode() -> int:
    """HIPATTN_SCAN_MODE = auto (default) | strict | check selects the arithmetic path of the scan kernels."""
    name = os.environ.get("HIPATTN_SCAN_MODE", "auto")
    try:
        return {"auto": L.SCAN_AUTO, "strict": L.SCAN_STRICT, "check": L.SCAN_CHECK}[name]
    except KeyError:
        raise ValueError(f"HIPATTN_SCAN_MODE={name!r}: expected auto, strict or check") from None


def _stage_cache_entry(left: Tensor, right: Tensor, B: int, BDST: int, H: int) -> HiPAttentionStageInputCache:
    """Reference layout of a stage-input cache: int64 [B, BDST, H, n], identical for every head."""
    lib = L.load()
    n = left.shape[-1]
    st = _stream(left.device)
    l64 = torch.empty((B, BDST, 1, n), dtype=torch.int64, device=left.device)
    r64 = torch.empty((B, BDST, 1, n), dtype=torch.int64, device=left.device)
    L.check(lib.hipattn_widen_i32(_ptr(left), _ptr(l64), left.numel(), st), "widen_i32")
    L.check(lib.hipattn_widen_i32(_ptr(right), _ptr(r64), right.numel(), st), "widen_i32")
    sc = torch.full((1, 1, 1, 1), SCORE_INIT, dtype=torch.float32, device=left.device)
    entry = HiPAttentionStageInputCache(indices_left=l64.expand(B, BDST, H, n), indices_right=r64.expand(B, BDST, H, n),
                                        out_scores=sc.expand(B, BDST, H, n))
    entry._left32, entry._right32 = left, right  # private: lets a restart skip the narrowing copy
    return entry


def _restart_inputs(entry: HiPAttentionStageInputCache, rows: int) -> Tuple[Tensor, Tensor]:
    l32 = getattr(entry, "_left32", None)
    if l32 is not None and l32.shape[0] == rows:
        return entry._left32.clone(), entry._right32.clone()
    # foreign cache (e.g. produced by the reference): per-head lists are identical under the head max-reduce
    l = entry.indices_left[:, :, 0, :].to(torch.int32).reshape(rows, -1).contiguous()
    r = entry.indices_right[:, :, 0, :].to(torch.int32).reshape(rows, -1).contiguous()
    return l, r


def _decode_splits(B: int, HKV: int, total_tokens: int) -> int:
    """Key ranges per (sequence, KV head).  One range when the batch alone fills the GPU (two CTAs per
    SM); otherwise enough ranges to do so, each at least four tiles (256 keys) long."""
    forced = os.environ.get("HIPATTN_DECODE_SPLITS")
    if forced:
        return max(1, min(64, int(forced)))
    units = max(1, B * HKV)
    if units >= 148:
        return 1
    return int(max(1, min(32, _cdiv(148 * 2, units), total_tokens // 256)))


def _attention(q: Tensor, ktok: L.Tokens, vtok: L.Tokens, T: int, HKV: int, pos: Tensor, indices: Tensor, ks: Tensor,
               *, sink: int, window: int, block_size_k: int, bsa_block_q: int, index_block_q: int, heads_share: bool,
               decode: bool, softcap: Optional[float], want_lse: bool,
               rope: Optional[Tuple[Tensor, Tensor]] = None, access: Optional[Tensor] = None) -> Tuple[Tensor, Optional[Tensor]]:
    lib = L.load()
    dev = q.device
    st = _stream(dev)
    B, TQ, H, D = q.shape
    out = torch.empty(q.shape, dtype=q.dtype, device=dev)
    lse = torch.empty((B, TQ, H), dtype=torch.float32, device=dev) if want_lse else None
    K = indices.shape[-1]
    if K == 0:
        indices = torch.zeros((indices.shape[0], indices.shape[1], 1), dtype=torch.int64, device=dev)
    bp = L.BsaParams()
    bp.q, bp.q_stride_b, bp.q_stride_t, bp.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1), q.stride(2)
    bp.out, bp.o_stride_b, bp.o_stride_t, bp.o_stride_h = out.data_ptr(), out.stride(0), out.stride(1), out.stride(2)
    bp.pos, bp.pos_stride_b, bp.pos_stride_t = pos.data_ptr(), pos.stride(0), pos.stride(1)
    bp.k, bp.v = ktok, vtok
    bp.indices, bp.idx_stride_n, bp.idx_stride_d = indices.data_ptr(), indices.stride(0), indices.stride(1)
    bp.ks, bp.ks_stride_n, bp.ks_stride_d = ks.data_ptr(), ks.stride(0), ks.stride(1)
    bp.status = status_word(dev).data_ptr()
    bp.dtype, bp.D, bp.B, bp.TQ, bp.H, bp.HKV, bp.T = _DT[q.dtype], D, B, TQ, H, HKV, T
    bp.block_size_q, bp.index_block_q, bp.block_size_k, bp.K = bsa_block_q, index_block_q, block_size_k, K
    bp.sink, bp.window = sink, window
    bp.heads_share_mask = int(heads_share or decode)
    bp.logit_softcap = float(softcap) if softcap else 0.0
    if rope is not None:
        bp.rope_cos, bp.rope_sin = rope[0].data_ptr(), rope[1].data_ptr()
        bp.rope_stride, bp.rope_rows = rope[0].stride(0), rope[0].shape[0]
    if access is not None:   # which tokens / pages the attention loads (require_cache_statistics)
        L.check(lib.hipattn_mark_attention_access(C.byref(bp), access.data_ptr(), access.stride(0), access.stride(1),
                                                  access.shape[-1], 1 if decode else bsa_block_q, st), "mark_attention_access")
    n_splits = _decode_splits(B, HKV, K * block_size_k + sink + window) if decode else 1
    bp.n_splits = n_splits
    if n_splits > 1:
        part_o = torch.empty((B, H, n_splits, D), dtype=torch.float32, device=dev)
        part_lse = torch.empty((B, H, n_splits), dtype=torch.float32, device=dev)
        bp.part_o, bp.part_lse = part_o.data_ptr(), part_lse.data_ptr()
        L.check(lib.hipattn_bsa_attention(C.byref(bp), st), "bsa_attention")
        o2 = out.view(B * TQ, H, D)
        if o2.stride(1) != D or o2.stride(0) != H * D:
            raise AssertionError("freshly allocated output must be contiguous")
        L.check(lib.hipattn_merge_partials(_ptr(part_o), _ptr(part_lse), B * H, n_splits, D, _DT[q.dtype], out.data_ptr(),
                                           D, _ptr(lse), st), "merge_partials")
    else:
        bp.lse_out = _ptr(lse)
        L.check(lib.hipattn_bsa_attention(C.byref(bp), st), "bsa_attention")
    return out, lse


def _check_inputs(q: Tensor, k: Optional[Tensor], v: Optional[Tensor], args: HiPAttentionArgs):
    if not isinstance(q, Tensor) or q.ndim != 4:
        raise ValueError("q must be a tensor [B, TQ, H, D]")
    if not q.is_cuda:
        raise RuntimeError("hip_attention_12 runs on a CUDA device only (B200, sm_100a); q is on " + str(q.device))
    if q.dtype not in _DT:
        raise NotImplementedError(f"q dtype {q.dtype} is not built (float32, float16, bfloat16)")
    if q.stride(-1) != 1:
        raise ValueError("q must have a contiguous last dim")
    if (k is None) != (v is None):
        raise ValueError("k and v must both be given or both be None")
    for name, t in (("k", k), ("v", v), ("k_cache", args.k_cache), ("v_cache", args.v_cache), ("q_mask", args.q_mask),
                    ("k_mask", args.k_mask)):
        if t is not None:
            if t.dtype in _FP8 and name in ("k", "v", "k_cache", "v_cache"):
                if q.dtype == torch.float32:
                    raise NotImplementedError("an fp8 (e5m2) KV cache needs float16 or bfloat16 queries")
            elif t.dtype != q.dtype:
                raise NotImplementedError(f"{name} dtype {t.dtype} differs from q dtype {q.dtype}")
            if t.device != q.device:
                raise ValueError(f"{name} is on {t.device}, q on {q.device}")
    if k is not None and k.shape != v.shape:
        raise ValueError("k and v must have the same shape")
    for a_, b_, what in ((k, v, "k and v"), (args.k_cache, args.v_cache, "k_cache and v_cache")):
        if a_ is not None and b_ is not None and (a_.dtype in _FP8) != (b_.dtype in _FP8):
            raise NotImplementedError(f"{what} must both be fp8 or both be q's dtype")
    if k is None and args.k_cache is None:
        raise ValueError("k is None and args.k_cache is None")
    if args.k_cache is not None and args.v_cache is None:
        raise ValueError("k_cache without v_cache")


def hip_attention_impl(q: Tensor, k: Optional[Tensor], v: Optional[Tensor], args: HiPAttentionArgs,
                       cached_metadata: Optional[HiPAttentionOutputMetadata] = None, *, return_lse: bool = False,
                       debug: Optional[dict] = None, score_reduce=None, timer: Optional[PhaseTimer] = None,
                       v_ready: Optional[torch.cuda.Event] = None):
    """Implementation behind ``hip_attention_12``.

    ``return_lse`` adds the base-2 log-sum-exp [B, TQ, H]; ``score_reduce`` is handed to the estimator
    (see ``_estimate_mask``); ``timer`` collects per-phase CUDA-event times; ``debug`` collects the
    per-head outputs of every scan stage.  ``v_ready``: the mask estimator reads only q and k, so a caller
    that streams its inputs to the device may issue the call as soon as q and k have arrived and pass the
    event that marks the arrival of v (dense ``v`` or the value cache); the attention launch waits for it."""
    _check_inputs(q, k, v, args)
    _reject_unsupported(args)
    args = args.clone()
    q_bsa = q
    if args.q_mask is not None:
        q = args.q_mask
        if q.shape != q_bsa.shape or q.stride(-1) != 1:
            raise ValueError("q_mask must have q's shape and a contiguous last dim")
    k_scan = k if args.k_mask is None else args.k_mask

    B, TQ, H, D = q.shape
    if k is not None:
        _, T, HKV, Dk = k.shape
        if k.shape[0] != B or Dk != D:
            raise ValueError(f"k shape {tuple(k.shape)} does not match q shape {tuple(q.shape)}")
    else:
        T = int(args.extend_context_length)
        HKV = args.k_cache.shape[-2]
        if args.k_cache.shape[-1] != D:
            raise ValueError("k_cache head_dim differs from q")
    if H % HKV:
        raise ValueError(f"{H} query heads are not a multiple of {HKV} KV heads")
    dev = q.device
    with torch.cuda.device(dev):
        if args.position_ids is not None:
            pos = args.position_ids
            if tuple(pos.shape) != (B, TQ):
                raise ValueError(f"position_ids shape {tuple(pos.shape)} != {(B, TQ)}")
            if pos.dtype != torch.int64:
                pos = pos.to(torch.int64)
        else:
            if torch.cuda.is_current_stream_capturing():
                raise ValueError("position_ids must be given under CUDA graph capture")
            pos = (torch.arange(0, TQ, device=dev, dtype=torch.int64) + (T - TQ))[None, :].expand(B, TQ)

        rope = _rope_tables(args, q)
        stages = args.stages
        bq = stages[-1].stage_block_size_q
        BDST = _cdiv(TQ, bq)
        c0, c_last = stages[0].stage_chunk_size, stages[-1].stage_chunk_size
        sw_attn = max(0, args.sliding_window_size - c0) + c0  # attention_extend.py:1976-1978, 2901

        # scan reads dense K when it is given, else the page pool (attention_extend.py:2524)
        if k_scan is not None:
            ktok_scan = _tokens(k_scan, None, None, None, "k")
        else:
            ktok_scan = _tokens(None, args.k_cache, args.block_table, args.cache_seq_lens, "k")
        # attention reads the page pool whenever one is given (attention_extend_bsa.py:1756)
        if args.k_cache is not None:
            ktok = _tokens(None, args.k_cache, args.block_table, args.cache_seq_lens, "k")
            vtok = _tokens(None, args.v_cache, args.block_table, args.cache_seq_lens, "v")
        else:
            ktok = _tokens(k, None, None, None, "k")
            vtok = _tokens(v, None, None, None, "v")

        stage_caches = None
        if args.require_stage_caches:
            if cached_metadata is None or cached_metadata.stage_caches is None:
                stage_caches = []
            else:
                stage_caches = cached_metadata.stage_caches  # extended in place, like the reference

        fresh_mask = cached_metadata is None or cached_metadata.indices is None
        # access statistics (attention_extend.py:1988-2010): one int32 per key position (dense) or page; no offload
        # cache exists here, so the miss counters stay zero
        mask_stats = sa_stats = None
        if args.require_cache_statistics:
            n_slots = args.k_cache.shape[0] if args.k_cache is not None else T
            sa_stats = torch.zeros((2, B, HKV, n_slots), dtype=torch.int32, device=dev)
            if fresh_mask:
                mask_stats = torch.zeros((2, B, HKV, n_slots), dtype=torch.int32, device=dev)
        if fresh_mask:
            restart = None
            if cached_metadata is not None and cached_metadata.stage_caches is not None and stage_caches is not None \
                    and len(stage_caches) > 1:
                if len(stage_caches) > len(stages):
                    raise ValueError("more stage caches than stages")
                i0 = len(stage_caches) - 1
                l32, r32 = _restart_inputs(stage_caches[i0], B * BDST)
                restart = (i0, l32, r32)
            m = _estimate_mask(q, ktok_scan, T, HKV, pos, args, restart, stage_caches is not None, debug,
                               score_reduce, timer, rope, None if mask_stats is None else mask_stats[0])
            if stage_caches is not None:
                for i in range(len(stage_caches), len(stages)):
                    si = m.stage_inputs[i] if i < len(m.stage_inputs) else None
                    if i == 0 or si is None:
                        stage_caches.append(HiPAttentionStageInputCache(None, None, None))
                    else:
                        stage_caches.append(_stage_cache_entry(si[0], si[1], B, BDST, H))
            indices, ks, ks_start_end = m.indices, m.ks, m.ks_start_end
            ks_count = ks.unsqueeze(-1)
            heads_share = m.heads_share
            index_block_q = bq
            bsa_bq = min(args.block_sparse_block_size_q or bq, bq)
            if args.mask_only:
                return None, None
        else:
            indices = cached_metadata.indices.clone()
            ks = cached_metadata.ks.clone()
            ks_count = cached_metadata.ks_count.clone()
            ks_start_end = cached_metadata.ks_start_end.clone()
            heads_share = bool(getattr(cached_metadata, "_heads_share", False))
            bsa_bq = min(args.block_sparse_block_size_q or bq, bq)
            # cached rows may already be broken down to the attention block size: the fresh path returns
            # BDST * (bq / bsa_bq) rows (repeat-interleave, attention_extend.py:3036-3051), of which a ragged
            # last block uses only the first cdiv(TQ, bsa_bq)
            index_block_q = bq if indices.shape[1] == BDST else bsa_bq
            if indices.shape[1] not in (BDST, _cdiv(TQ, bsa_bq), BDST * (bq // bsa_bq)) or indices.shape[0] != B * H:
                raise ValueError(f"cached indices shape {tuple(indices.shape)} does not fit this call")
            if indices.dtype != torch.int64 or ks.dtype != torch.int64:
                indices, ks = indices.to(torch.int64), ks.to(torch.int64)

        bsa_bq = min(bsa_bq, _next_pow2(TQ))
        if bq % bsa_bq:
            raise ValueError("block_sparse_block_size_q must divide stage_block_size_q")
        if sw_attn == 777:
            # window sentinel of the serving adapter (attention_extend.py:3070-3076): these queries see
            # everything the model context has room for beside the sink, the selected keys and their own block
            sw_attn = args.model_context_length - args.sink_token_size - args.second_stage_k - bsa_bq
            if sw_attn < 0:
                raise ValueError("the window sentinel 777 needs model_context_length > sink + second_stage_k + query block")
        decode = TQ == 1 and not args.disable_flashdecode and os.environ.get("HIP_DISABLE_FLASHDECODE", "0") != "1"
        if timer: timer.mark("start")
        if v_ready is not None:
            torch.cuda.current_stream(dev).wait_event(v_ready)
        context, lse = _attention(q_bsa, ktok, vtok, T, HKV, pos, indices, ks, sink=args.sink_token_size, window=sw_attn,
                                  block_size_k=c_last, bsa_block_q=bsa_bq, index_block_q=index_block_q,
                                  heads_share=heads_share, decode=decode, softcap=args.logit_softcap,
                                  want_lse=return_lse, rope=rope, access=None if sa_stats is None else sa_stats[0])
        if timer: timer.mark("attention")

        if fresh_mask and _cdiv(TQ, bsa_bq) != BDST:
            # break the mask down to the attention block size (attention_extend.py:3036-3051)
            rep = bq // bsa_bq
            indices = indices.repeat_interleave(rep, 1)
            ks = ks.repeat_interleave(rep, 1)
            ks_count = ks_count.repeat_interleave(rep, 1)
            ks_start_end = ks_start_end.repeat_interleave(rep, 1)

        def stats(t):
            return HiPAttentionCacheAccessStatistics(None, None) if t is None else HiPAttentionCacheAccessStatistics(t[0], t[1])
        md = HiPAttentionOutputMetadata(
            indices=indices, ks=ks, ks_count=ks_count, ks_start_end=ks_start_end,
            mask_cache_statistics=stats(mask_stats) if fresh_mask else None,
            sa_cache_statistics=stats(sa_stats), stage_caches=stage_caches)
        md._heads_share = heads_share
    if return_lse:
        return context, md, lse
    return context, md


def hip_attention_12(q: Tensor, k: Optional[Tensor], v: Optional[Tensor], args: Optional[HiPAttentionArgs] = None,
                     cached_metadata: Optional[HiPAttentionOutputMetadata] = None):
    """HiP attention: ``(context, metadata) = hip_attention_12(q, k, v, args, cached_metadata)``.

    q [B, TQ, H, D] must already carry the softmax scale; k, v [B, TK, HKV, D], or ``None`` with
    ``args.k_cache / v_cache / block_table / cache_seq_lens`` describing a paged cache.  Passing the
    returned metadata back skips the mask estimator; metadata with ``indices=None`` and a prefix of
    ``stage_caches`` restarts the estimator at the last cached stage.
    """
    return hip_attention_impl(q, k, v, args if args is not None else HiPAttentionArgs(), cached_metadata)
