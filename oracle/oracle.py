"""ctypes front end of the CPU oracle (liboracle.so) -- TEST INFRASTRUCTURE, not product code.

Only tests/, __graft_entry__.smoke() and the cpu-baseline legs of bench.py import this module.  All arrays are
numpy, C-contiguous, float32 or float64 (the `dtype` argument picks the arithmetic the oracle runs in).

Layouts (same as the reference, gqa25/slotkern_cuda.py:97 and :501):
    k, q (B,T,H,DK)   v (B,T,H,DV)   gate, fr (B,T,H) [fr may be a 1-element array]   snapshots (B,NB,H,N,D)
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


class _Cfg(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in
                ("B", "T", "H", "N", "DK", "DV", "G", "hard", "hard_gate", "occ_bin", "detach_addr", "fr_per_token")] + \
               [("eps", ctypes.c_double), ("temp", ctypes.c_double)]


def build():
    """Compile liboracle.so with the Makefile beside this file (gcc, a second or two)."""
    subprocess.run(["make", "-s", "-C", _HERE], check=True)


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liboracle.so")
        src_m = max(os.path.getmtime(os.path.join(_HERE, f)) for f in ("slotscan_oracle.c", "slotscan_oracle_impl.h"))
        if not os.path.exists(path) or os.path.getmtime(path) < src_m:
            build()
        _LIB = ctypes.CDLL(path)
    return _LIB


def use_timed_build():
    """For the TIMED CPU-baseline legs of bench.py only: switch to a build of the same source compiled for speed on
    the host it runs on (-O3 -march=native, contraction allowed), so the baseline is not handicapped by the flags the
    parity build needs (no FMA contraction, to match the reference's torch arithmetic bit for bit where it can).
    Falls back to the parity build if the compiler refuses.  Returns the flags in use."""
    global _LIB
    path = os.path.join(_HERE, "liboracle_timed.so")
    flags = ["-O3", "-march=native", "-fPIC", "-fopenmp"]
    try:
        subprocess.run(["gcc"] + flags + ["-shared", "-o", path, os.path.join(_HERE, "slotscan_oracle.c"), "-lm"],
                       check=True, capture_output=True)
        _LIB = ctypes.CDLL(path)
        return " ".join(flags)
    except Exception:
        lib()
        return "-O2 -ffp-contract=off (parity build)"


def threads():
    return lib().slotscan_oracle_threads()


def set_threads(n):
    lib().slotscan_oracle_set_threads(int(n))


def _np(x, dt):
    if x is None:
        return None
    if hasattr(x, "detach"):
        x = x.detach().cpu().numpy()
    return np.ascontiguousarray(np.asarray(x), dtype=dt)


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _suffix(dt):
    return "_f64" if np.dtype(dt) == np.float64 else "_f32"


def _cfg(k, v, N, G, temp, hard, hard_gate, occ_bin, detach_addr, fr, eps):
    B, T, H, DK = k.shape
    return _Cfg(B, T, H, N, DK, v.shape[-1], G, int(hard), int(hard_gate), int(occ_bin), int(detach_addr),
                int(fr.ndim == 3), float(eps), float(temp))


def scan_fwd(k, v, gate, fr, N, temp, G=1, hard=False, hard_gate=False, eps=1e-4, q=None, occ_bin=False,
             dtype=np.float64):
    """Forward scan.  Returns dict(kbuf, vbuf, addr, margin, kfin, vfin, ofin)."""
    k, v, gate, q = _np(k, dtype), _np(v, dtype), _np(gate, dtype), _np(q, dtype)
    fr = _np(fr, dtype)
    if fr.ndim != 3:
        fr = fr.reshape(1)
    c = _cfg(k, v, N, G, temp, hard, hard_gate, occ_bin, False, fr, eps)
    B, T, H, DK = k.shape
    DV = v.shape[-1]
    NB = (T + G - 1) // G
    out = dict(kbuf=np.empty((B, NB, H, N, DK), dtype), vbuf=np.empty((B, NB, H, N, DV), dtype),
               addr=np.empty((B, T, H), np.int32), margin=np.empty((B, T, H), dtype),
               kfin=np.empty((B, H, N, DK), dtype), vfin=np.empty((B, H, N, DV), dtype),
               ofin=np.empty((B, H, N), dtype))
    fn = getattr(lib(), "slotscan_oracle_fwd" + _suffix(dtype))
    rc = fn(ctypes.byref(c), _p(k), _p(q), _p(v), _p(gate), _p(fr), _p(out["kbuf"]), _p(out["vbuf"]),
            _p(out["addr"]), _p(out["margin"]), _p(out["kfin"]), _p(out["vfin"]), _p(out["ofin"]))
    assert rc == 0
    return out


def scan_bwd(k, v, gate, fr, N, temp, dkbuf, dvbuf, G=1, hard=False, hard_gate=False, eps=1e-4, detach_addr=False,
             q=None, occ_bin=False, dtype=np.float64):
    """Gradients of sum(kbuf*dkbuf)+sum(vbuf*dvbuf).  Returns dict(dk, dq (None when q is None), dv, dgate, dfr, dtemp)."""
    k, v, gate, q = _np(k, dtype), _np(v, dtype), _np(gate, dtype), _np(q, dtype)
    fr = _np(fr, dtype)
    if fr.ndim != 3:
        fr = fr.reshape(1)
    dkbuf, dvbuf = _np(dkbuf, dtype), _np(dvbuf, dtype)
    c = _cfg(k, v, N, G, temp, hard, hard_gate, occ_bin, detach_addr, fr, eps)
    out = dict(dk=np.zeros_like(k), dq=None if q is None else np.zeros_like(q), dv=np.zeros_like(v),
               dgate=np.zeros_like(gate), dfr=np.zeros_like(fr), dtemp=np.zeros(1, dtype))
    fn = getattr(lib(), "slotscan_oracle_bwd" + _suffix(dtype))
    rc = fn(ctypes.byref(c), _p(k), _p(q), _p(v), _p(gate), _p(fr), _p(dkbuf), _p(dvbuf), _p(out["dk"]),
            _p(out["dq"]), _p(out["dv"]), _p(out["dgate"]), _p(out["dfr"]), _p(out["dtemp"]))
    assert rc == 0
    return out


def epilogue(kbuf, dtype=np.float64):
    """kinv, valid per snapshot row (memlm_sh.py:474-475)."""
    kbuf = _np(kbuf, dtype)
    rows = int(np.prod(kbuf.shape[:-1]))
    kinv = np.empty(kbuf.shape[:-1], dtype)
    valid = np.empty(kbuf.shape[:-1], np.uint8)
    getattr(lib(), "slotscan_oracle_epilogue" + _suffix(dtype))(_p(kbuf), ctypes.c_long(rows), kbuf.shape[-1],
                                                                _p(kinv), _p(valid))
    return kinv, valid.astype(bool)


def read_fwd(qr, sharp, kbuf, vbuf, kinv, valid, G, dtype=np.float64, want_att=False):
    """Cosine read.  qr (B,T,H,NQ,DK), sharp (B,T,H,NQ) -> rd (B,T,H,NQ,DV)."""
    qr, sharp, kbuf, vbuf, kinv = (_np(a, dtype) for a in (qr, sharp, kbuf, vbuf, kinv))
    valid = np.ascontiguousarray(_np(valid, np.uint8))
    B, T, H, NQ, DK = qr.shape
    N, DV = vbuf.shape[-2], vbuf.shape[-1]
    rd = np.empty((B, T, H, NQ, DV), dtype)
    att = np.empty((B, T, H, NQ, N), dtype) if want_att else None
    getattr(lib(), "slotscan_oracle_read_fwd" + _suffix(dtype))(B, T, H, NQ, N, DK, DV, G, _p(qr), _p(sharp), _p(kbuf),
                                                                _p(vbuf), _p(kinv), _p(valid), _p(rd), _p(att))
    return (rd, att) if want_att else rd


def read_bwd(qr, sharp, kbuf, vbuf, kinv, valid, G, drd, kinv_const=True, dtype=np.float64):
    """Adjoint of read_fwd: dict(dqr, dsharp, dkbuf, dvbuf)."""
    qr, sharp, kbuf, vbuf, kinv, drd = (_np(a, dtype) for a in (qr, sharp, kbuf, vbuf, kinv, drd))
    valid = np.ascontiguousarray(_np(valid, np.uint8))
    B, T, H, NQ, DK = qr.shape
    N, DV = vbuf.shape[-2], vbuf.shape[-1]
    out = dict(dqr=np.zeros_like(qr), dsharp=np.zeros_like(sharp), dkbuf=np.zeros_like(kbuf), dvbuf=np.zeros_like(vbuf))
    getattr(lib(), "slotscan_oracle_read_bwd" + _suffix(dtype))(
        B, T, H, NQ, N, DK, DV, G, _p(qr), _p(sharp), _p(kbuf), _p(vbuf), _p(kinv), _p(valid), _p(drd),
        _p(out["dqr"]), _p(out["dsharp"]), _p(out["dkbuf"]), _p(out["dvbuf"]), int(bool(kinv_const)))
    return out


def fq(x, bits, group, dtype=np.float32):
    """Midrise group quantiser (memlm_sh.py:221-229), forward value only."""
    x = _np(x, dtype)
    assert x.shape[-1] % group == 0
    y = np.empty_like(x)
    getattr(lib(), "slotscan_oracle_fq" + _suffix(dtype))(_p(x), ctypes.c_long(x.size // group), int(group), int(bits),
                                                         _p(y))
    return y


def scan_v_fwd(v, wa, gate, fr, N, G=1, hard=False, hard_gate=False, dtype=np.float64):
    """Keyless scan (gqa25/slotkern_v.py:242-261).  v (B,T,H,DV), wa (B,T,H,N), gate (B,T,H), fr scalar.
    Returns dict(buf (B,NB,H,N,DV), addr (B,T,H))."""
    v, wa, gate = _np(v, dtype), _np(wa, dtype), _np(gate, dtype)
    fr = _np(fr, dtype).reshape(1)
    B, T, H, DV = v.shape
    NB = (T + G - 1) // G
    out = dict(buf=np.empty((B, NB, H, N, DV), dtype), addr=np.empty((B, T, H), np.int32))
    rc = getattr(lib(), "slotscan_oracle_v_fwd" + _suffix(dtype))(B, T, H, int(N), DV, int(G), int(hard), int(hard_gate),
                                                                  _p(v), _p(wa), _p(gate), _p(fr), _p(out["buf"]), _p(out["addr"]))
    assert rc == 0
    return out


def scan_v_bwd(v, wa, gate, fr, N, dbuf, G=1, hard=False, hard_gate=False, dtype=np.float64):
    """Gradients of sum(buf * dbuf): dict(dv, dwa, dgate, dfr (1,))."""
    v, wa, gate, dbuf = _np(v, dtype), _np(wa, dtype), _np(gate, dtype), _np(dbuf, dtype)
    fr = _np(fr, dtype).reshape(1)
    B, T, H, DV = v.shape
    out = dict(dv=np.zeros_like(v), dwa=np.zeros_like(wa), dgate=np.zeros_like(gate), dfr=np.zeros(1, dtype))
    rc = getattr(lib(), "slotscan_oracle_v_bwd" + _suffix(dtype))(B, T, H, int(N), DV, int(G), int(hard), int(hard_gate),
                                                                  _p(v), _p(wa), _p(gate), _p(fr), _p(dbuf), _p(out["dv"]),
                                                                  _p(out["dwa"]), _p(out["dgate"]), _p(out["dfr"]))
    assert rc == 0
    return out


def fp8_e4m3_rows(x):
    """Per-row fp8-e4m3 storage: s = absmax/448 per row, y = e4m3(x/s) * s.  The reference has no fp8 format
    (only a comment, memlm_sh.py:217-218), so this restatement is PARITY-UNPINNED by any reference test."""
    import torch
    t = torch.as_tensor(np.asarray(x, np.float32))
    a = t.abs().amax(-1, keepdim=True)
    s = (a / 448.0).clamp_min(1e-30)
    y = (t / s).to(torch.float8_e4m3fn).float() * s
    return torch.where(a > 0, y, torch.zeros_like(y)).numpy()
