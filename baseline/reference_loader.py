"""Import the UNMODIFIED reference operator from ``baseline/_ref`` (a git-ignored copy of the reference's
``src/hip_attn`` package) so that it can be timed and compared on the same GPU.

Nothing of this project is on that path: ``load_reference()`` returns the reference's own
``dual_stage_quadratic_hip_attention`` (``hip_attn/v1_2/attention_extend.py:1918``), ``HiPAttentionArgs``
and ``ScanStage`` (``hip_attn/v1_2/attention_metadata.py``), running its Triton kernels.

The reference's package ``__init__`` imports optional modules this image does not have (``nvtx``,
``matplotlib``, ``cupy``); none of them is used by the operator.  The package is therefore entered through a
namespace shim that skips ``__init__`` and the three names resolve to empty stand-in modules.  The reference
compiles one small C++ torch extension at import (``hip_attn/v1_1/offload_runner/tensor_from_pointer.py``);
its build directory is kept under ``baseline/_ref`` so that it is built once and travels with the copy.
"""
from __future__ import annotations

import os
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def available() -> bool:
    return os.path.isfile(os.path.join(REF, "hip_attn", "v1_2", "attention_extend.py"))


def load_reference(interpret: bool = False):
    """Returns ``(operator, HiPAttentionArgs, ScanStage)`` of the reference.

    ``interpret=True`` runs its Triton kernels on the CPU through the Triton interpreter (no bf16 there);
    otherwise they are compiled for the current GPU.  Must be called before anything else imports triton
    when ``interpret`` is set."""
    if not available():
        raise FileNotFoundError(f"no reference copy under {REF}")
    if interpret:
        os.environ["TRITON_INTERPRET"] = "1"
    os.environ.setdefault("HIP_DISABLE_AUTOTUNE", "1")
    os.environ.setdefault("HIP_DISABLE_AUTOTUNE_WARNINGS", "1")
    os.environ.setdefault("TORCH_EXTENSIONS_DIR", os.path.join(REF, "torch_extensions"))
    tmp = tempfile.mkdtemp(prefix="hipref_shim_")
    os.makedirs(os.path.join(tmp, "shim", "hip_attn"))
    with open(os.path.join(tmp, "shim", "hip_attn", "__init__.py"), "w") as f:
        f.write(f"__path__ = [{os.path.join(REF, 'hip_attn')!r}]\n")
    for mod in ("matplotlib/__init__.py", "matplotlib/pyplot.py", "cupy/__init__.py", "nvtx.py"):
        name = mod.split("/")[0].replace(".py", "")
        try:
            __import__(name)
            continue            # the real module exists: no stand-in
        except ImportError:
            pass
        p = os.path.join(tmp, "stubs", mod)
        os.makedirs(os.path.dirname(p), exist_ok=True)
        open(p, "w").close()
    sys.path[:0] = [os.path.join(tmp, "shim"), os.path.join(tmp, "stubs")]
    import torch
    if interpret:
        torch.cuda.is_current_stream_capturing = lambda: False
        torch.cuda.current_device = lambda: 0
        torch.cuda.set_device = lambda d: None
        torch.cuda.get_device_name = lambda *a: "cpu"
    import hip_attn.v1_2.attention_extend as ext
    from hip_attn.v1_2.attention_metadata import HiPAttentionArgs, ScanStage
    return ext.dual_stage_quadratic_hip_attention, HiPAttentionArgs, ScanStage


def reference_args(Args, ScanStage, *, bq, strides, chunks, keep, sink, sw, **kw):
    """Reference argument object for a stage list given as chunk sizes / kept tokens / query strides."""
    stages = [ScanStage(stage_block_size_q=bq, stage_block_stride_q=strides[i], stage_chunk_size=c,
                        stage_k=None if i == 0 else keep[i - 1], stage_stride=1) for i, c in enumerate(chunks)]
    kw.setdefault("require_cache_statistics", False)   # the benchmarks of this project switch the access counters off
    return Args(sink_token_size=sink, sliding_window_size=sw, second_stage_k=keep[-1], stages=stages,
                block_sparse_block_size_q=bq, using_extend=False, need_apply_rope=False, **kw)
