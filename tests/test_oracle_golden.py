"""The CPU oracle must reproduce the reference operator's recorded outputs (tests/golden/*.npz)."""
import os

import numpy as np
import pytest
import torch

from cases import CASES, make_inputs, make_paged
from oracle import hip_oracle as O

GOLD = os.path.join(os.path.dirname(__file__), "golden")
FAST = [n for n in CASES if n != "config1_fp32"]


def run_oracle(name, **kw):
    q, k, v, pos, c = make_inputs(name)
    cfg = O.config_from_case(c)
    paged = None
    if "page" in c:
        kc, vc, table = make_paged(k, v, c["page"], c["seed"])
        paged = (kc, vc, table, torch.full((c["B"],), c["T"], dtype=torch.int64), c["ext"])
    return O.hip_attention_oracle(q, k, v, pos, cfg, paged=paged, **kw), (q, k, v, pos, c, cfg)


def check_against_golden(name):
    g = np.load(os.path.join(GOLD, f"{name}.npz"))
    (out, m), (q, k, v, pos, c, cfg) = run_oracle(name)
    assert np.array_equal(m.indices.numpy(), g["indices"]), "indices differ from the reference"
    assert np.array_equal(m.ks.numpy(), g["ks"])
    assert np.array_equal(m.ks_count.numpy(), g["ks_count"])
    assert np.array_equal(m.ks_start_end.numpy(), g["ks_start_end"])
    assert m.ks_start_end.dtype == torch.int32 and m.indices.dtype == torch.int64 and m.ks.dtype == torch.int64
    for i in range(1, len(cfg.stages)):
        l, r = m.stage_inputs[i]
        assert np.array_equal(l.numpy(), g[f"stage{i}_left"]), f"stage {i} input left"
        assert np.array_equal(r.numpy(), g[f"stage{i}_right"]), f"stage {i} input right"
        assert (g[f"stage{i}_scores"] == -32000.0).all()
    rs = c.get("out_row_stride", 1)
    ref = g["out"]
    tol = 2e-6 if c["dtype"] == "fp32" else 2e-3  # fp16 reference rounds P and the output to fp16
    err = np.abs(out.float().numpy()[:, ::rs] - ref).max()
    assert err < tol, f"attention output differs from the reference by {err}"
    return g, m, (q, k, v, pos, c, cfg)


@pytest.mark.parametrize("name", FAST)
def test_oracle_matches_reference(name):
    check_against_golden(name)


def test_oracle_matches_reference_config1():
    """benchmark configuration 1 (fp32, 4096 x 4096); the reference took minutes through the interpreter."""
    if not os.path.exists(os.path.join(GOLD, "config1_fp32.npz")):
        pytest.skip("fixture not generated")
    check_against_golden("config1_fp32")


@pytest.mark.parametrize("name", ["prefill_fp32", "ragged_fp16"])
def test_oracle_stage_cache_restart(name):
    """Restarting from the cached inputs of stage n-1 reproduces the full result
    (reference invariant: tests/v1_2/test_gen3_stage_caching.py:170-186)."""
    g = np.load(os.path.join(GOLD, f"{name}.npz"))
    (out, m), (q, k, v, pos, c, cfg) = run_oracle(name)
    for n in range(2, len(cfg.stages) + 1):
        l, r = m.stage_inputs[n - 1]
        (o2, m2), _ = run_oracle(name, restart=(n - 1, l, r))
        assert torch.equal(m2.indices, m.indices)
        assert np.array_equal(m2.indices.numpy(), g[f"indices_restart{n}"])
        assert ((o2 - out) ** 2).sum() < 1e-8
