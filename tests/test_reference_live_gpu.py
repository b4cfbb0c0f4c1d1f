"""Live parity against the reference's OWN code on the same box: the float64 torch definition
(`slotkern_kv._ref_scan_kv_impl`) and the reference's production CUDA kernel (`slotkern_cuda.kv_scan_c`), both run
unmodified from baseline/_ref/ (staged by baseline/stage_reference.py; git-ignored) in a process of their own, on
inputs from the same seeded generator.  Skipped when the staging is absent.  The committed golden vectors
(tests/golden/) pin the same functions without needing the reference at run time; this test adds shapes at the
production head size and the reference's CUDA kernel itself."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.scan_cases import make_inputs, rel_to_max

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SCRIPT = os.path.join(ROOT, "baseline", "run_reference_scan.py")
STAGED = os.path.isfile(os.path.join(ROOT, "baseline", "_ref", "gqa25", "slotkern_kv.py"))

CASES = [  # name, dist, B, T, H, N, DK, DV, G, hard, hard_gate, occ_bin, detach, frtok, sepq, seed, reference CUDA kernel too
    ("sh25_head_hard_detached", "bench", 1, 96, 2, 192, 128, 128, 8, 1, 0, 1, 1, 1, 1, 31, True),
    ("clustered_many_rows", "clustered", 1, 128, 2, 192, 128, 128, 8, 1, 0, 1, 1, 1, 1, 32, True),
    ("d64_n96_scalar_fr_q_none", "gates01", 2, 80, 2, 96, 64, 64, 16, 1, 0, 0, 1, 0, 0, 33, True),
    ("soft_attached", "clustered", 1, 48, 2, 24, 16, 16, 4, 0, 0, 1, 0, 1, 1, 34, False),
]


@pytest.mark.skipif(not STAGED, reason="baseline/_ref is not staged (no reference checkout at build time)")
@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_against_the_reference_run_live(case, tmp_path):
    import slotscan_b200 as S
    name, dist, B, T, H, N, DK, DV, G, hard, hard_gate, occ_bin, detach, frtok, sepq, seed, with_cuda = case
    out = str(tmp_path / "ref.npz")
    cmd = [sys.executable, SCRIPT, out, dist] + [str(x) for x in (B, T, H, N, DK, DV, G, hard, hard_gate, occ_bin, detach, frtok, sepq, seed)]
    if with_cuda:
        cmd.append("--cuda")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    z = np.load(out)
    inp = make_inputs(dist, B, T, H, DK, DV, seed=seed, frtok=bool(frtok), sepq=bool(sepq))
    dev = "cuda"
    leaves = {n: inp[n].to(dev).requires_grad_() for n in ("k", "v", "gate", "fr")}
    q = inp["q"].to(dev).requires_grad_() if inp["q"] is not None else None
    tp = torch.tensor(float(inp["temp"]), device=dev, requires_grad=True)
    kb, vb = S.kv_scan_g(leaves["k"], leaves["v"], leaves["gate"], leaves["fr"], N, tp, G=G, hard=bool(hard),
                         hard_gate=bool(hard_gate), detach_addr=bool(detach), q=q, occ_bin=bool(occ_bin))
    ((kb * torch.from_numpy(z["wk"]).to(dev)).sum() + (vb * torch.from_numpy(z["wv"]).to(dev)).sum()).backward()
    mine = dict(kbuf=kb, vbuf=vb, dk=leaves["k"].grad, dv=leaves["v"].grad, dgate=leaves["gate"].grad, dfr=leaves["fr"].grad, dtemp=tp.grad)
    if q is not None:
        mine["dq"] = q.grad
    mine = {n: x.detach().float().cpu().numpy() for n, x in mine.items()}
    keep = np.ones((B, H), bool)
    if hard:   # a near-tie of the float64 definition may fall either way in float32: those sequences are left out, and counted
        ref = O.scan_fwd(inp["k"], inp["v"], inp["gate"], inp["fr"], N=N, temp=inp["temp"], G=G, hard=True, hard_gate=bool(hard_gate),
                         q=inp["q"], occ_bin=bool(occ_bin), dtype=np.float64)
        assert np.array_equal(ref["addr"], z["addr"]), "the oracle and the reference disagree on an address"
        keep = ref["margin"].min(axis=1) > 1e-4                                   # (B, T, H) -> (B, H)
        print("%s: sequences with a near-tie (< 1e-4): %d of %d" % (name, int((~keep).sum()), keep.size))
        assert keep.any()
    m5, m4, m3 = keep[:, None, :, None, None], keep[:, None, :, None], keep[:, None, :]
    for n in ("kbuf", "vbuf"):
        assert (np.abs(mine[n] - z[n]) * m5).max() < 2e-5, n
    for n, m in (("dk", m4), ("dv", m4), ("dgate", m3), ("dfr", m3 if frtok else None), ("dq", m4)):
        if n not in mine:
            continue
        a, b = mine[n].reshape(z[n].shape), z[n]
        if m is not None:
            a, b = a * m, b * m
        assert rel_to_max(a, b) < 1e-4, n
    if keep.all():
        assert rel_to_max(mine["dtemp"], z["dtemp"]) < 1e-4
    if with_cuda:
        # the reference's own CUDA kernel on the same inputs: float32 against float32
        for n in ("kbuf", "vbuf"):
            assert (np.abs(mine[n] - z["c_" + n]) * m5).max() < 2e-5, n
        for n, m in (("dk", m4), ("dv", m4), ("dgate", m3), ("dq", m4)):
            if n in mine and "c_" + n in z:
                assert rel_to_max(mine[n].reshape(z["c_" + n].shape) * m, z["c_" + n] * m) < 2e-4, n
