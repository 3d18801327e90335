"""CPU oracle for HiP / InfiniteHiP attention (mask estimator + block-sparse attention).

TEST INFRASTRUCTURE ONLY.  This module is a plain torch-on-CPU restatement of the reference
operator ``hip_attention_12`` (= ``dual_stage_quadratic_hip_attention``,
``src/hip_attn/v1_2/attention_extend.py:1918-3133`` of DeepAuto-AI/hip-attention).  It is used by
``tests/``, by ``__graft_entry__.smoke()`` and by the ``cpu_baseline`` / ``--impl reference`` legs
of ``bench.py`` as the checker and the timed CPU baseline.  The product package never imports it.

Parity status: PINNED.  ``tests/test_oracle_golden.py`` checks this restatement against outputs of
the unmodified reference executed on the CPU (``tests/golden/gen_golden.py``; fixtures in
``tests/golden/*.npz``).

Two points where the reference leaves behaviour open are fixed here:

* Ordering among equal scores.  The reference uses ``topk(sorted=False)`` and
  ``sort(stable=False)`` (``attention_extend.py:2717-2726``); here ties go to the lower chunk
  position (stable descending order).
* Summation order of the representative-key dot product.  The reference calls ``tl.dot`` with an
  fp32 accumulator (``attention_extend.py:924-945``); here the accumulator runs sequentially over
  the head dimension in ascending order, one fp32 multiply and one fp32 add per element.  For
  16-bit inputs the products are exact in fp32, so this equals a chain of fused multiply-adds.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

INT64_MAX = torch.iinfo(torch.int64).max
SCORE_INIT = -32000.0


# --------------------------------------------------------------------------------------
# small helpers
# --------------------------------------------------------------------------------------
def cdiv(a: int, b: int) -> int:
    return -(-a // b)


def next_pow2(x: int) -> int:
    return 1 if x <= 1 else 1 << (x - 1).bit_length()


def round_to(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Round fp32 values through ``dtype`` and return them as fp32."""
    if dtype == torch.float32:
        return x.float()
    return x.to(dtype).float()


def scan_scales(D: int, dtype: torch.dtype) -> Tuple[float, float]:
    """Scales applied to pooled queries and to keys before the dot product.

    ``attention_extend.py:924-940``: q * (sqrt(D) / sqrt(sqrt(D))).to(dtype), k * (1 / sqrt(sqrt(D))).to(dtype),
    all square roots and divisions in fp32.
    """
    s = np.sqrt(np.float32(D)).astype(np.float32)
    ss = np.sqrt(s).astype(np.float32)
    qs = np.float32(s / ss)
    ks = np.float32(np.float32(1.0) / ss)
    qs = round_to(torch.tensor(float(qs), dtype=torch.float32), dtype).item()
    ks = round_to(torch.tensor(float(ks), dtype=torch.float32), dtype).item()
    return qs, ks


@dataclass
class OracleStage:
    """One ScanStage (``attention_metadata.py:56-60``)."""
    block_size_q: int
    stride_q: int
    chunk_size: int
    stage_k: Optional[int]


@dataclass
class OracleConfig:
    stages: List[OracleStage]
    sink: int
    sw: int
    second_stage_k: int
    block_size_k: int = 64  # BLOCK_CHUNK seed, ``attention_extend.py:1970``
    softcap: Optional[float] = None  # logit soft-cap of the attention kernels
    bsa_block_q: Optional[int] = None  # block_sparse_block_size_q when smaller than the estimator's query block
    rope: Optional["OracleRope"] = None  # in-kernel RoPE (``using_extend`` and ``need_apply_rope``)


@dataclass
class OracleRope:
    """Un-rotated q / k plus cos / sin tables [T, D]: the kernels rotate on the fly (``attention_extend.py:248-407,
    630-703``, ``attention_extend_bsa.py:126-392, 797-856``).  Backends built: scan ``relative`` / ``streaming``
    (per stage, ``ScanStage.stage_extend_backend`` overrides), attention ``streaming``."""
    cos: torch.Tensor
    sin: torch.Tensor
    scan_backend: str = "relative"
    stage_backends: Optional[List[Optional[str]]] = None   # per-stage override (None entries fall back)
    sa_backend: str = "streaming"

    def backend_of(self, i: int) -> str:
        b = self.stage_backends[i] if self.stage_backends is not None and self.stage_backends[i] is not None else self.scan_backend
        if b not in ("relative", "streaming"):
            raise NotImplementedError(f"scan_extend_backend {b!r}")
        return b


def rope_rotate(x: torch.Tensor, positions: torch.Tensor, rope: OracleRope, dtype: torch.dtype) -> torch.Tensor:
    """x [..., D] fp32 holding dtype-rounded values, positions [...] (broadcastable to x's leading dims) ->
    x * cos + rotate_half(x) * sin with cos / sin cast to ``dtype`` first and every product and the sum rounded to
    ``dtype`` (the reference computes in the element type: ``attention_extend.py:392-407, 690-703``)."""
    D = x.shape[-1]
    h = D // 2
    cos = round_to(rope.cos.float(), dtype)[positions.long()][..., :h]
    sin = round_to(rope.sin.float(), dtype)[positions.long()][..., :h]
    cos = torch.cat([cos, cos], -1)
    sin = torch.cat([sin, sin], -1)
    rot = torch.cat([-x[..., h:], x[..., :h]], -1)
    return round_to(round_to(x * cos, dtype) + round_to(rot * sin, dtype), dtype)


class DenseKV:
    """K or V stored as [B, T, HKV, D] (``uvm_gpu_cache.py:865-874``)."""

    def __init__(self, x: torch.Tensor):
        self.x = x
        self.T = x.shape[1]
        self.HKV = x.shape[2]
        self.dtype = x.dtype

    def rows(self, b: int, t: torch.Tensor, hkv: int) -> torch.Tensor:
        return self.x[b, t.clamp(0, self.T - 1), hkv]


class PagedKV:
    """K or V stored as a page pool [n_pages, P, HKV, D] addressed through a block table.

    ``uvm_gpu_cache.py:876-890, 1034-1042``: page = block_table[b, t // P] when 0 <= t < cache_seq_lens[b],
    otherwise page 0; row = cache[page, t % P, hkv].
    """

    def __init__(self, cache: torch.Tensor, block_table: torch.Tensor, cache_seq_lens: torch.Tensor, T: int):
        self.cache = cache
        self.table = block_table.long()
        self.seq = cache_seq_lens.long()
        self.P = cache.shape[1]
        self.HKV = cache.shape[2]
        self.T = T  # extent of the chunk grid (extend_context_length)
        self.dtype = cache.dtype

    def rows(self, b: int, t: torch.Tensor, hkv: int) -> torch.Tensor:
        ok = (t >= 0) & (t < self.seq[b])
        pidx = (t // self.P).clamp(0, self.table.shape[1] - 1)
        page = torch.where(ok, self.table[b][pidx], torch.zeros_like(t))
        return self.cache[page, t % self.P, hkv]


# --------------------------------------------------------------------------------------
# scan stage
# --------------------------------------------------------------------------------------
def strict_dot(qs: torch.Tensor, ks: torch.Tensor) -> torch.Tensor:
    """qs [..., R, D], ks [..., N, D] (fp32 holding dtype-rounded values) -> [..., R, N].

    Sequential fp32 accumulation over D in ascending order: acc = fl(acc + fl(q_d * k_d)).
    """
    D = qs.shape[-1]
    acc = torch.zeros(qs.shape[:-1] + (ks.shape[-2],), dtype=torch.float32)
    for d in range(D):
        prod = qs[..., :, d, None] * ks[..., None, :, d]
        acc = acc + prod
    return acc


def pooled_queries(q: torch.Tensor, pos: torch.Tensor, b: int, d: int, bq: int, sq: int, rope=None, new_tdst=None):
    """Mean-pooled, strided query rows of block d (``attention_extend.py:516-734``).

    ``rope`` / ``new_tdst(pos_rows)``: with in-kernel RoPE every loaded row is first rotated to the position
    ``new_tdst`` gives for the position of its group's FIRST row (``attention_extend.py:630-703``).
    Returns (Q̄ [H, R, D] fp32 holding dtype-rounded values, valid [R] bool, pmin int).
    """
    TQ = q.shape[1]
    R = bq // sq
    t = d * bq + torch.arange(R) * sq
    valid = t < TQ
    acc = torch.zeros((R, q.shape[2], q.shape[3]), dtype=torch.float32)
    cnt = torch.zeros((R,), dtype=torch.float32)
    for o in range(sq):
        ti = t + o
        ok = valid & (ti < TQ)
        rows = q[b, ti.clamp(max=TQ - 1)].float() * ok[:, None, None]
        if rope is not None:
            p_rows = torch.where(valid, pos[b, t.clamp(max=TQ - 1)], torch.zeros_like(t))
            rows = rope_rotate(rows, new_tdst(p_rows)[:, None].expand(R, q.shape[2]), rope, q.dtype) * ok[:, None, None]
        acc = acc + rows
        cnt = cnt + ok.float()
    qbar = acc / (cnt[:, None, None] + torch.tensor(1e-12, dtype=torch.float32))
    qbar = qbar * valid[:, None, None]
    qbar = round_to(qbar, q.dtype).permute(1, 0, 2).contiguous()  # [H, R, D]
    pmin = int(pos[b, t[valid]].min())
    return qbar, valid, pmin


def scan_block(qbar, valid, pmin, ksrc, b, left, right, *, bq, sw_r, G, block_chunk, dtype, rope=None, backend=None,
               touched=None):
    """Scan one (batch, query block) for all heads.

    left/right: int64 [H, n].  Returns narrowed (left, right) [H, n] and scores [H, n] fp32
    (``attention_extend.py:736-1249``).
    """
    H, n = left.shape
    D = qbar.shape[-1]
    q_scale, k_scale = scan_scales(D, dtype)
    qs = round_to(qbar * q_scale, dtype)  # [H, R, D]
    pt = max(pmin - sw_r, 0)
    left = left.clone()
    right = right.clone()
    scores = torch.full((H, n), SCORE_INIT, dtype=torch.float32)

    # rounds per group of block_chunk chunks: while m >= 1: m /= 2
    ngroup = cdiv(n, block_chunk)
    size = (right - left)
    pad = ngroup * block_chunk - n
    size_p = torch.nn.functional.pad(size, (0, pad), value=0).view(H, ngroup, block_chunk)
    gmax = size_p.max(-1).values  # [H, ngroup]
    left_p = torch.nn.functional.pad(left, (0, pad), value=ksrc.T).view(H, ngroup, block_chunk)
    gmin_left = left_p.min(-1).values
    # group skip test (result-neutral, kept for fidelity): ``attention_extend.py:595-597``
    g_run = (pmin + bq) >= gmin_left
    rounds = torch.where(gmax >= 1, torch.floor(torch.log2(gmax.clamp(min=1).double())).long() + 1,
                         torch.zeros_like(gmax))
    rounds = torch.where(g_run, rounds, torch.zeros_like(rounds))
    rounds_c = rounds[:, :, None].expand(H, ngroup, block_chunk).reshape(H, -1)[:, :n]  # [H, n]

    neg_inf = torch.tensor(float("-inf"))
    for it in range(int(rounds.max()) if rounds.numel() else 0):
        live = it < rounds_c
        act = live & (left < right) & (left <= pt) & (left >= 0)
        mid = (left + right) // 2
        tl_ = (left + mid) // 2
        tr_ = (mid + right) // 2

        def side(t, is_right=False):
            out = torch.empty((H, n), dtype=torch.float32)
            for hk in range(H // G):
                hs = slice(hk * G, (hk + 1) * G)
                rows = ksrc.rows(b, t[hs], hk).float() * act[hs][..., None]  # [G, n, D]
                rows = round_to(rows, dtype)
                if rope is not None:
                    # representative keys are rotated to the chunk's ordinal (streaming) or to 0 / 1 for the left /
                    # right candidate (relative), ``attention_extend.py:290-298``
                    if backend == "streaming":
                        new_t = torch.arange(n)[None, :].expand(G, n)
                    else:
                        new_t = torch.full((G, n), 1 if is_right else 0)
                    rows = rope_rotate(rows, new_t, rope, dtype) * act[hs][..., None]
                kk = round_to(rows * k_scale, dtype)
                s = round_to(strict_dot(qs[hs], kk), dtype)  # [G, R, n]
                s = torch.where(valid[None, :, None], s, neg_inf)
                out[hs] = s.max(1).values
            return torch.where(act, out, neg_inf)

        if touched is not None:   # access statistics: the candidate rows of the active chunks, per KV head
            for t_ in (tl_, tr_):
                for hk in range(H // G):
                    hs = slice(hk * G, (hk + 1) * G)
                    touched[hk].append(t_[hs][act[hs]])
        sl = side(tl_)
        sr = side(tr_, True)
        win = sl > sr
        left, right = (torch.where(act, torch.where(win, left, mid), left),
                       torch.where(act, torch.where(win, mid, right), right))
        scores = torch.maximum(scores, torch.where(act, torch.where(win, sl, sr), scores))
    return left, right, scores


# --------------------------------------------------------------------------------------
# estimator driver
# --------------------------------------------------------------------------------------
@dataclass
class OracleMask:
    indices: torch.Tensor          # [B*H, BDST, K] int64, ascending, padded with INT64_MAX
    ks: torch.Tensor               # [B*H, BDST] int64
    ks_count: torch.Tensor         # [B*H, BDST, 1] int64
    ks_start_end: torch.Tensor     # [B*H, BDST, 2] int32
    stage_inputs: List[Optional[Tuple[torch.Tensor, torch.Tensor]]] = field(default_factory=list)
    # per stage: (left, right, per-head scores, head-reduced scores) right after the scan
    stage_outputs: List[Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]] = field(default_factory=list)
    block_size_k: int = 0          # last stage chunk size
    block_size_q: int = 0
    mask_access: Optional[torch.Tensor] = None   # access statistics of the estimator (``statistics=True``)


def initial_chunks(T: int, cfg: OracleConfig, B: int, BDST: int, H: int):
    """``attention_extend.py:2027-2046``."""
    c0 = cfg.stages[0].chunk_size
    n0 = cdiv(max(0, T - cfg.sink - cfg.sw), c0)
    sw_r = max(0, cfg.sw - c0)
    left = (torch.arange(n0, dtype=torch.int64) * c0 + cfg.sink)[None, None, None, :].expand(B, BDST, H, n0).clone()
    right = (left + c0).clamp(max=T - sw_r)
    return left, right


def next_stage_inputs(left: torch.Tensor, cfg: OracleConfig, i: int):
    """Slice, realign, sort and split the selected chunks (``attention_extend.py:2072-2165``)."""
    c_prev = cfg.stages[i - 1].chunk_size
    c_new = cfg.stages[i].chunk_size
    stage_k = cfg.stages[i].stage_k
    assert stage_k % c_prev == 0 and c_prev % c_new == 0
    left = left[..., : stage_k // c_prev]
    left = (left - cfg.sink) // c_prev * c_prev + cfg.sink
    right = left + c_prev
    left, order = left.sort(dim=-1, stable=True)
    right = right.gather(-1, order)
    s = c_prev // c_new
    w = ((right - left).float() / s).clamp(min=0)
    ar = torch.arange(s)
    nl = (left[..., None] + (ar * w[..., None]).floor().long()).flatten(-2)
    nr = (right[..., None] - (((s - 1) - ar) * w[..., None]).floor().long()).flatten(-2)
    return nl, nr


def access_counter(ksrc, B: int, touched) -> torch.Tensor:
    """The reference's access statistics (``uvm_gpu_cache.py:846-909``): int32 [B, HKV, positions] (dense K) or
    [B, HKV, pages] (paged: the page the block table gives, page 0 for positions beyond the sequence), 1 where a
    token was loaded.  ``touched[b][hkv]`` = list of int64 token tensors."""
    paged = isinstance(ksrc, PagedKV)
    n = ksrc.cache.shape[0] if paged else ksrc.T
    out = torch.zeros((B, ksrc.HKV, n), dtype=torch.int32)
    for b in range(B):
        for hk in range(ksrc.HKV):
            if not touched[b][hk]:
                continue
            t = torch.cat([x.flatten() for x in touched[b][hk]])
            if paged:
                ok = (t >= 0) & (t < ksrc.seq[b])
                pidx = (t // ksrc.P).clamp(0, ksrc.table.shape[1] - 1)
                t = torch.where(ok, ksrc.table[b][pidx].long(), torch.zeros_like(t))
            out[b, hk, t.clamp(0, n - 1)] = 1
    return out


def attention_access(mask: "OracleMask", pos: torch.Tensor, ksrc, H: int, *, sink: int, sw: int, decode: bool) -> torch.Tensor:
    """Tokens the reference's attention kernels load for every (batch, KV head): sink tokens below the block's last
    position, the tokens of the selected blocks inside [sink, last position], and the window from
    last position + 1 - window - block rows up to the last position (``attention_extend_bsa.py:858-891, 1133-1137,
    1370-1383``; the decode kernel's block is one row)."""
    B, TQ = pos.shape
    G = H // ksrc.HKV
    bq = 1 if decode else mask.block_size_q
    touched = [[[] for _ in range(ksrc.HKV)] for _ in range(B)]
    for b in range(B):
        for d in range(cdiv(TQ, mask.block_size_q)):
            r0, r1 = d * mask.block_size_q, min((d + 1) * mask.block_size_q, TQ)
            cur = int(pos[b, r0:r1].max()) + 1
            for hk in range(ksrc.HKV):
                n = b * H + hk * G
                ks = int(mask.ks[n, d])
                sel = (mask.indices[n, d, :ks, None] + torch.arange(mask.block_size_k)[None, :]).flatten()
                sel = sel[(sel >= sink) & (sel < cur) & (sel < ksrc.T)]
                touched[b][hk] += [torch.arange(0, min(sink, cur)), sel]
                if sw > 0:
                    touched[b][hk].append(torch.arange(max(0, cur - sw - bq), cur))
    return access_counter(ksrc, B, touched)


def estimate_mask(q: torch.Tensor, ksrc, pos: torch.Tensor, cfg: OracleConfig,
                  restart: Optional[Tuple[int, torch.Tensor, torch.Tensor]] = None,
                  keep_stage_outputs: bool = False, score_reduce=None, statistics: bool = False) -> OracleMask:
    """Run the hierarchical mask estimator.

    q [B, TQ, H, D] (pre-scaled by the caller), ksrc a DenseKV/PagedKV over K, pos [B, TQ] int64.
    restart = (stage index i, left, right) resumes from the cached inputs of stage i
    (``attention_extend.py:2047-2071``).  score_reduce(tensor), if given, completes the head max in place
    across the processes of a KV-head-parallel run.
    """
    B, TQ, H, D = q.shape
    T = ksrc.T
    G = H // ksrc.HKV
    bq = cfg.stages[0].block_size_q
    BDST = cdiv(TQ, bq)
    sw_r = max(0, cfg.sw - cfg.stages[0].chunk_size)
    block_chunk = cfg.block_size_k
    out = OracleMask(None, None, None, None)
    touched = [[[] for _ in range(ksrc.HKV)] for _ in range(B)] if statistics else None

    left, right = initial_chunks(T, cfg, B, BDST, H)
    first = 0
    if restart is not None:
        first, left, right = restart
        left, right = left.clone(), right.clone()
        out.stage_inputs = [None] * first
        # BLOCK_CHUNK evolves through the skipped stages only via their chunk counts; the reference
        # does not replay that either (``attention_extend.py:2067-2071``)
    for i in range(first, len(cfg.stages)):
        st = cfg.stages[i]
        assert st.block_size_q == bq, "per-stage query block sizes are not supported by the oracle"
        if i > 0 and not (restart is not None and i == first):
            left, right = next_stage_inputs(left, cfg, i)
        if i == 0:
            assert st.stage_k is None
            out.stage_inputs.append(None)
        else:
            out.stage_inputs.append((left.clone(), right.clone()))
        n = left.shape[-1]
        block_chunk = max(16, next_pow2(min(n, block_chunk)))
        scores = torch.full((B, BDST, H, n), SCORE_INIT, dtype=torch.float32)
        nl = left.clone()
        nr = right.clone()
        for b in range(B):
            for d in range(BDST):
                backend = new_tdst = None
                if cfg.rope is not None:
                    backend = cfg.rope.backend_of(i)
                    if backend == "relative":      # ``attention_extend.py:641``
                        new_tdst = lambda p: torch.full_like(p, 1 + sw_r)
                    else:                          # streaming, ``:644-647``
                        new_tdst = lambda p, n=n: torch.minimum(p, torch.full_like(p, n + sw_r))
                qbar, valid, pmin = pooled_queries(q, pos, b, d, bq, st.stride_q, cfg.rope, new_tdst)
                l2, r2, s2 = scan_block(qbar, valid, pmin, ksrc, b, left[b, d], right[b, d], bq=bq, sw_r=sw_r,
                                        G=G, block_chunk=block_chunk, dtype=q.dtype, rope=cfg.rope, backend=backend,
                                        touched=None if touched is None else touched[b])
                nl[b, d], nr[b, d], scores[b, d] = l2, r2, s2
        red = scores.max(dim=2, keepdim=True).values  # head reduce, ``attention_extend.py:2566-2570``
        if score_reduce is not None:  # heads split over processes: finish the max across them
            red = red.contiguous()
            score_reduce(red)
        if keep_stage_outputs:
            out.stage_outputs.append((nl.clone(), nr.clone(), scores.clone(), red[:, :, 0].clone()))
        if i < len(cfg.stages) - 1:
            kk = min(cfg.stages[i + 1].stage_k // st.chunk_size, n)
        else:
            kk = n
        order = red.sort(dim=-1, descending=True, stable=True).indices[..., :kk].expand(B, BDST, H, kk)
        left = nl.gather(-1, order)
        right = nr.gather(-1, order)

    c_last = cfg.stages[-1].chunk_size
    assert cfg.second_stage_k % c_last == 0
    idx = left[..., : cfg.second_stage_k // c_last] // c_last * c_last
    if statistics:
        out.mask_access = access_counter(ksrc, B, touched)
    return finalize_indices(idx, pos, H, bq, c_last, out)


def finalize_indices(idx: torch.Tensor, pos: torch.Tensor, H: int, bq: int, c_last: int,
                     out: Optional[OracleMask] = None) -> OracleMask:
    """``attention_extend.py:2906-2925``: idx [B, BDST, H, K] -> sorted unique block starts + counts."""
    out = out or OracleMask(None, None, None, None)
    idx = idx.permute(0, 2, 1, 3).flatten(0, 1)
    idx = idx.sort(-1).values
    idx = idx // c_last * c_last
    uniq = torch.roll(idx, 1, -1) != idx
    idx = torch.where(uniq, idx, torch.full_like(idx, INT64_MAX)).sort(-1).values
    lim = pos[:, ::bq, None].repeat_interleave(H, 0) + bq
    ks = (idx < lim).int().sum(-1)
    out.indices = idx
    out.ks = ks
    out.ks_count = ks.unsqueeze(-1)
    se = torch.zeros((ks.shape[0], ks.shape[1], 2), dtype=torch.int32)
    se[:, :, 1] = ks.int()
    out.ks_start_end = se
    out.block_size_k = c_last
    out.block_size_q = bq
    return out


# --------------------------------------------------------------------------------------
# attention on a given mask
# --------------------------------------------------------------------------------------
def attended_columns(indices_row: torch.Tensor, ks: int, pos_rows: torch.Tensor, *, sink: int, sw: int,
                     c_last: int, T: int):
    """Columns one query block can attend and the per-row allow mask.

    Rules (``attention_extend_bsa.py:511-525, 858-891, 1133-1137, 1370-1383``), for a row at position p
    in a block whose largest position is pmax:
      window   {t : p - sw < t <= p}
      sink     {t < sink, t <= p - sw}
      selected {t in [idx_j, idx_j + c_last), j < ks : sink <= t <= pmax, t < T, t <= p - sw}
    Returns (cols [C] int64 ascending, allow [rows, C] bool).
    """
    pmax = int(pos_rows.max())
    pmin = int(pos_rows.min())
    sel = indices_row[:ks]
    sel_t = (sel[:, None] + torch.arange(c_last)[None, :]).flatten()
    sel_t = sel_t[(sel_t >= sink) & (sel_t <= pmax) & (sel_t < T) & (sel_t >= 0)]
    win_t = torch.arange(max(0, pmin - sw + 1), pmax + 1)
    sink_t = torch.arange(0, min(sink, pmax + 1))
    cols = torch.unique(torch.cat([sink_t, sel_t, win_t]))
    is_sel = torch.isin(cols, sel_t)
    p = pos_rows[:, None]
    t = cols[None, :]
    window = (t <= p) & (t > p - sw)
    far = t <= p - sw
    allow = window | (far & (t < sink)) | (far & is_sel[None, :])
    return cols, allow


def rope_attention_block(q_rows, pos_rows, idx_row, ks: int, ksrc, vsrc, b: int, hkv: int, *, sink: int, sw: int, c_last: int,
                         rope: OracleRope, dtype):
    """Logits and values of one (query block, head) with in-kernel RoPE, attention backend ``streaming``.

    Queries are rotated to their own position (``attention_extend_bsa.py:797-856``).  Window keys are rotated to
    their own position; sink keys and selected-block keys to ``max(0, j * c_last + i + pmin - sw - sink - ks * c_last
    + 1)`` with j the key's block rank in the list [sink blocks | selected blocks], i its offset in the block, pmin the
    block's smallest query position and ks * c_last the number of selected tokens of the block (``:256-270, 1120,
    1359``).  A token can sit in two groups; the admission rules of the groups are disjoint per row.
    Returns (s [rows, C] fp64 logits with -inf where not admitted, values [C, D] fp64)."""
    T = ksrc.T
    pmax, pmin = int(pos_rows.max()), int(pos_rows.min())
    qd = q_rows.dtype
    qr = rope_rotate(q_rows.float(), pos_rows, rope, qd).to(dtype)
    sel_start = idx_row[:ks]
    jb = torch.arange(ks)[:, None].expand(ks, c_last).flatten()
    io = torch.arange(c_last)[None, :].expand(ks, c_last).flatten()
    sel_t = (sel_start[:, None] + torch.arange(c_last)[None, :]).flatten()
    ok = (sel_t >= sink) & (sel_t <= pmax) & (sel_t < T) & (sel_t >= 0)
    sel_t, jb, io = sel_t[ok], jb[ok], io[ok]
    shift = pmin - sw - sink - ks * c_last + 1
    sel_new = ((jb + sink // c_last) * c_last + io + shift).clamp(min=0)
    sink_t = torch.arange(0, min(sink, pmax + 1, T))
    sink_new = (sink_t + shift).clamp(min=0)
    win_t = torch.arange(max(0, pmin - sw + 1), min(pmax + 1, T))
    p = pos_rows[:, None]
    parts = []
    for t, new_t, is_win in ((sink_t, sink_new, False), (sel_t, sel_new, False), (win_t, win_t, True)):
        if t.numel() == 0:
            continue
        kk = rope_rotate(ksrc.rows(b, t, hkv).to(qd).float(), new_t, rope, qd).to(dtype)
        allow = ((t[None, :] <= p) & (t[None, :] > p - sw)) if is_win else (t[None, :] <= p - sw)
        parts.append(((qr @ kk.T).masked_fill(~allow, float("-inf")), vsrc.rows(b, t, hkv).to(dtype)))
    if not parts:
        return torch.full((q_rows.shape[0], 0), float("-inf"), dtype=dtype), torch.zeros((0, q_rows.shape[-1]), dtype=dtype)
    return torch.cat([x[0] for x in parts], 1), torch.cat([x[1] for x in parts], 0)


def attention_on_mask(q: torch.Tensor, ksrc, vsrc, pos: torch.Tensor, mask: OracleMask, *, sink: int, sw: int,
                      bsa_block_q: Optional[int] = None, return_lse: bool = False, dtype=torch.float64,
                      softcap: Optional[float] = None, rope: Optional[OracleRope] = None):
    """Masked softmax attention recomputed in high precision on the estimator's mask.

    ``sw`` is the attention window (the reference restores ``max(sw, c_0)``, ``attention_extend.py:2901``).
    Logits are q·k (q pre-scaled), optionally soft-capped as tanh(x / cap) * cap
    (``attention_extend_bsa.py:389-390, 507-508``); softmax rows with an empty set give 0
    (``attention_extend_bsa.py:1623-1625``).
    Returns out [B, TQ, H, D] (and the base-2 log-sum-exp [B, TQ, H] when ``return_lse``).
    """
    B, TQ, H, D = q.shape
    G = H // ksrc.HKV
    bq = mask.block_size_q
    out = torch.zeros((B, TQ, H, D), dtype=dtype)
    lse = torch.full((B, TQ, H), float("-inf"), dtype=dtype)
    LOG2E = 1.4426950408889634
    for b in range(B):
        for d in range(cdiv(TQ, bq)):
            r0, r1 = d * bq, min((d + 1) * bq, TQ)
            for h in range(H):
                n = b * H + h
                if rope is not None:
                    s, vv = rope_attention_block(q[b, r0:r1, h], pos[b, r0:r1], mask.indices[n, d], int(mask.ks[n, d]), ksrc,
                                                 vsrc, b, h // G, sink=sink, sw=sw, c_last=mask.block_size_k, rope=rope, dtype=dtype)
                    if softcap:
                        s = torch.where(torch.isinf(s), s, torch.tanh(s / softcap) * softcap)
                else:
                    cols, allow = attended_columns(mask.indices[n, d], int(mask.ks[n, d]), pos[b, r0:r1], sink=sink,
                                                   sw=sw, c_last=mask.block_size_k, T=ksrc.T)
                    kk = ksrc.rows(b, cols, h // G).to(dtype)
                    vv = vsrc.rows(b, cols, h // G).to(dtype)
                    s = q[b, r0:r1, h].to(dtype) @ kk.T
                    if softcap:
                        s = torch.tanh(s / softcap) * softcap
                    s = s.masked_fill(~allow, float("-inf"))
                m = s.max(-1, keepdim=True).values
                m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
                p = torch.exp(s - m)
                l = p.sum(-1, keepdim=True)
                out[b, r0:r1, h] = torch.where(l > 0, (p @ vv) / l.clamp(min=1e-300), torch.zeros_like(p @ vv))
                lse[b, r0:r1, h] = torch.where(l[:, 0] > 0, (m[:, 0] + torch.log(l[:, 0].clamp(min=1e-300))) * LOG2E,
                                               torch.full_like(m[:, 0], float("-inf")))
    if return_lse:
        return out, lse
    return out


def merge_partials(o: torch.Tensor, lse2: torch.Tensor):
    """Merge per-split partial outputs (``attention_decode_bsa.py:1192-1225``).

    o [S, ..., D] normalised partial outputs, lse2 [S, ...] base-2 log-sum-exp (-inf = empty split).
    Returns (out [..., D], lse2 [...]).
    """
    m = lse2.max(0).values
    m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w = torch.exp2(lse2 - m_safe)
    w = torch.where(torch.isinf(lse2), torch.zeros_like(w), w)
    tot = w.sum(0)
    out = (o * w[..., None]).sum(0) / tot.clamp(min=1e-20)[..., None]
    return out, torch.where(tot > 0, m_safe + torch.log2(tot.clamp(min=1e-300)), torch.full_like(m, float("-inf")))


# --------------------------------------------------------------------------------------
# whole operator
# --------------------------------------------------------------------------------------
def hip_attention_oracle(q, k, v, pos, cfg: OracleConfig, *, paged=None, restart=None, mask: Optional[OracleMask] = None,
                         keep_stage_outputs: bool = False, out_dtype=torch.float64):
    """Estimator + attention.  ``paged`` = (k_cache, v_cache, block_table, cache_seq_lens, T_grid)."""
    if paged is not None:
        kc, vc, table, seq, T = paged
        ksrc, vsrc = PagedKV(kc, table, seq, T), PagedKV(vc, table, seq, T)
    else:
        ksrc, vsrc = DenseKV(k), DenseKV(v)
    if mask is None:
        mask = estimate_mask(q, ksrc, pos, cfg, restart=restart, keep_stage_outputs=keep_stage_outputs)
        bq, TQ = mask.block_size_q, q.shape[1]
        if cfg.bsa_block_q and cdiv(TQ, cfg.bsa_block_q) != cdiv(TQ, bq):
            # break the mask down to the attention block size (``attention_extend.py:3035-3051``)
            assert bq % cfg.bsa_block_q == 0
            rep = bq // cfg.bsa_block_q
            mask.indices, mask.ks = mask.indices.repeat_interleave(rep, 1), mask.ks.repeat_interleave(rep, 1)
            mask.ks_count = mask.ks_count.repeat_interleave(rep, 1)
            mask.ks_start_end = mask.ks_start_end.repeat_interleave(rep, 1)
            mask.block_size_q = cfg.bsa_block_q
    sw_attn = max(0, cfg.sw - cfg.stages[0].chunk_size) + cfg.stages[0].chunk_size
    out = attention_on_mask(q, ksrc, vsrc, pos, mask, sink=cfg.sink, sw=sw_attn, dtype=out_dtype, softcap=cfg.softcap,
                            rope=cfg.rope)
    return out, mask


def config_from_case(c) -> OracleConfig:
    return OracleConfig(stages=[OracleStage(*s) for s in c["stages"]], sink=c["sink"], sw=c["sw"],
                        second_stage_k=c["second_k"], softcap=c.get("softcap"), bsa_block_q=c.get("bsa_bq"),
                        rope=rope_from_case(c))


def rope_from_case(c) -> Optional[OracleRope]:
    """cos / sin tables of a golden case with in-kernel RoPE (``rope_in_kernel`` = scan backend name)."""
    if "rope_in_kernel" not in c:
        return None
    import cases
    T = max(c.get("ext", c["T"]), c["T"]) + 8
    cos, sin = cases.rope_tables(T, c["D"], c.get("rope_theta", 10000.0))
    return OracleRope(cos=torch.from_numpy(cos), sin=torch.from_numpy(sin), scan_backend=c["rope_in_kernel"],
                      stage_backends=c.get("stage_backends"))
