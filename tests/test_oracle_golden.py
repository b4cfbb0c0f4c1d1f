"""Pins the CPU oracle (oracle/) to fixtures produced by the reference's own torch code (tests/golden/make_golden.py).

Forward snapshots, addresses and every gradient of every scan mode; the cosine read with per-token sharpness; the
midrise quantiser.  float64 oracle vs the float64 reference: agreement to round-off, far inside the 1e-4 the
reference's own kernel tests accept (gqa25/test_kvg.py:38-39).
"""
import glob
import os

import numpy as np
import pytest

from oracle import oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
SCAN = sorted(glob.glob(os.path.join(GOLDEN, "scan_*.npz")))


def rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-12))


def load(path):
    z = np.load(path)
    B, T, H, N, DK, DV, G, hard, hard_gate, occ_bin, detach, frtok, sepq = (int(x) for x in z["meta"])
    kw = dict(N=N, temp=float(z["temp"]), G=G, hard=bool(hard), hard_gate=bool(hard_gate), eps=1e-4,
              q=z["q"] if sepq else None, occ_bin=bool(occ_bin))
    return z, kw, bool(detach)


def test_fixture_list_complete():
    assert len(SCAN) == 13, SCAN
    for f in ("read_rsharp_nq2.npz", "quant_fq.npz"):
        assert os.path.exists(os.path.join(GOLDEN, f))


@pytest.mark.parametrize("path", SCAN, ids=[os.path.basename(p)[5:-4] for p in SCAN])
def test_scan_forward_matches_reference(path):
    z, kw, _ = load(path)
    out = O.scan_fwd(z["k"], z["v"], z["gate"], z["fr"], dtype=np.float64, **kw)
    assert rel(out["kbuf"], z["kbuf"]) < 1e-9
    assert rel(out["vbuf"], z["vbuf"]) < 1e-9
    if kw["hard"]:
        assert np.array_equal(out["addr"], z["addr"])
    # snapshot 0 is the all-zero state (pre-write)
    assert np.abs(out["kbuf"][:, 0]).max() == 0 and np.abs(out["vbuf"][:, 0]).max() == 0
    # the float32 oracle against the reference's float32 wrapper: same recurrence, float32 round-off
    out32 = O.scan_fwd(z["k"], z["v"], z["gate"], z["fr"], dtype=np.float32, **kw)
    if kw["hard"] and np.array_equal(out32["addr"], z["addr"]):
        assert rel(out32["kbuf"], z["kbuf_f32"]) < 1e-5
        assert rel(out32["vbuf"], z["vbuf_f32"]) < 1e-5


@pytest.mark.parametrize("path", SCAN, ids=[os.path.basename(p)[5:-4] for p in SCAN])
def test_scan_backward_matches_reference_autograd(path):
    z, kw, detach = load(path)
    g = O.scan_bwd(z["k"], z["v"], z["gate"], z["fr"], dkbuf=z["wk"], dvbuf=z["wv"], detach_addr=detach,
                   dtype=np.float64, **kw)
    names = ["dk", "dv", "dgate", "dfr", "dtemp"] + (["dq"] if kw["q"] is not None else [])
    for n in names:
        want = z[n].reshape(g[n].shape)
        assert rel(g[n], want) < 1e-7, (n, rel(g[n], want))


def test_read_matches_reference():
    z = np.load(os.path.join(GOLDEN, "read_rsharp_nq2.npz"))
    G = int(z["G"])
    kinv, valid = O.epilogue(z["kbuf"])
    assert rel(kinv, z["kinv"]) < 1e-12 and np.array_equal(valid, z["valid"])
    # the reference casts its logits to float32 (memlm_sh.py:383 `.float()`), so agreement is float32 round-off
    rd = O.read_fwd(z["qr"], z["sharp"], z["kbuf"], z["vbuf"], kinv, valid, G)
    assert rel(rd, z["rd"]) < 2e-6
    # block 0 reads the empty memory: exactly zero (gqa25/test_sh.py:87-88)
    assert np.abs(rd[:, :G]).max() == 0
    # kinv is computed from kbuf under autograd in the fixture, so differentiate it too
    g = O.read_bwd(z["qr"], z["sharp"], z["kbuf"], z["vbuf"], kinv, valid, G, z["drd"], kinv_const=False)
    assert rel(g["dqr"], z["dqr"]) < 1e-5
    assert rel(g["dvbuf"], z["dvbuf"]) < 1e-5
    assert rel(g["dkbuf"], z["dkbuf"]) < 1e-5
    C = float(z["C"])
    ds_raw = g["dsharp"] * z["sharp"] * (1 - np.tanh(z["s_raw"].reshape(z["sharp"].shape) / C) ** 2)
    assert rel(ds_raw.reshape(z["ds_raw"].shape), z["ds_raw"]) < 1e-5


def test_quantiser_matches_reference():
    z = np.load(os.path.join(GOLDEN, "quant_fq.npz"))
    for bits in (2, 3, 4, 8):
        for group in (16, 64):
            y = O.fq(z["x"], bits, group, dtype=np.float32)
            assert np.array_equal(y, z["fq_b%d_g%d" % (bits, group)]), (bits, group)
    y = O.fq(z["x"], 3, 16)
    assert np.abs(y[0, 0, 0, 0]).max() == 0                      # never-written row stays exactly zero
    kq = O.fq(z["x"], 3, 16)
    kinv, valid = O.epilogue(kq, dtype=np.float32)
    assert np.array_equal(valid, z["qm_valid"]) and rel(kinv[valid], z["qm_kinv"][valid]) < 1e-6


KEYLESS = sorted(glob.glob(os.path.join(GOLDEN, "keyless_*.npz")))


@pytest.mark.parametrize("path", KEYLESS, ids=[os.path.basename(p)[8:-4] for p in KEYLESS])
def test_keyless_scan_matches_reference(path):
    """The keyless scan (gqa25/slotkern_v.py: ref_scan_v) and its adjoint against the reference's float64 run + autograd."""
    z = np.load(path)
    B, T, H, N, DV, G, hard, hard_gate = (int(x) for x in z["meta"])
    kw = dict(N=N, G=G, hard=bool(hard), hard_gate=bool(hard_gate))
    out = O.scan_v_fwd(z["v"], z["wa"], z["gate"], z["fr"], dtype=np.float64, **kw)
    assert rel(out["buf"], z["buf"]) < 1e-9
    g = O.scan_v_bwd(z["v"], z["wa"], z["gate"], z["fr"], dbuf=z["w"], dtype=np.float64, **kw)
    for n in ("dv", "dwa", "dgate", "dfr"):
        assert rel(g[n].reshape(z[n].shape), z[n]) < 1e-7, n


def test_keyless_fixture_list_complete():
    assert len(KEYLESS) == 3, KEYLESS
