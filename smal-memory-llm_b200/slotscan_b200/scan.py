"""Host side of the slot scan, mirroring the reference's Python interface.

    kv_scan_g(k, v, gate, fr, N, temp, G=16, hard=False, hard_gate=False, eps=1e-4, detach_addr=False, q=None,
              nw=None, nwb=None, occ_bin=False) -> (kbuf, vbuf)           gqa25/slotkern_kvg.py:257
    kv_scan_c(...same...)                                                  gqa25/slotkern_cuda.py:536
    scan_kv(k, v, gate, fr, N, temp, G=1, hard=False, hard_gate=False, eps=1e-4, detach_addr=False, q=None)
                                                                           gqa25/slotkern_kv.py:29

Same argument meaning and the same result contract: (kbuf, vbuf), each (B, ceil(T/G), H, N, D), the PRE-write state
at t = 0, G, 2G, ...; gradients for k, q (if given), v, gate, fr, temp.  Differences from the reference, all additive:
  * k, q, v may be bfloat16: they are then read as bf16 by the kernels (no float32 copy) and their gradients come
    back as bf16.  Anything else is cast to contiguous float32 as the reference does (slotkern_cuda.py:488-489).
  * out_dtype=torch.bfloat16 makes the kernels emit bf16 snapshots directly (the reference emits float32 and the
    model casts, memlm_sh.py:475).  Default float32 = the reference contract.
  * nw / nwb (Triton warp hints) are accepted and ignored.
There is no Triton path, no dispatch and no CPU fallback: CPU tensors and unimplemented modes raise.
"""
import torch

from . import ops


def _as_f32(x):
    return x.contiguous().to(torch.float32)


def _token_streams(k, v, q):
    """The dtype policy of the token streams: bf16 kernels only when k, v and q (if given) are ALL bfloat16; anything
    else is cast to contiguous float32 as the reference does (slotkern_cuda.py:488-489)."""
    bf = k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16 and (q is None or q.dtype == torch.bfloat16)
    conv = (lambda x: x.contiguous()) if bf else _as_f32
    return conv(k), conv(v), (None if q is None else conv(q))


def kv_scan_g(k, v, gate, fr, N, temp, G=16, hard=False, hard_gate=False, eps=1e-4, detach_addr=False, q=None, nw=None,
              nwb=None, occ_bin=False, out_dtype=torch.float32):
    if not k.is_cuda:
        raise RuntimeError("slotscan_b200.kv_scan_g: CUDA tensors only (no CPU path in this package)")
    if not (hard and detach_addr):
        raise NotImplementedError("slotscan_b200: only the hard-address scan with a detached address gradient "
                                  "(hard=True, detach_addr=True, the training mode of the reference run) is built")
    if out_dtype not in (torch.float32, torch.bfloat16):
        raise ValueError("out_dtype must be float32 or bfloat16")
    B, T, H, DK = k.shape
    assert v.shape[:3] == (B, T, H) and gate.shape == (B, T, H), (k.shape, v.shape, gate.shape)
    k_, v_, q_ = _token_streams(k, v, q)
    g_ = _as_f32(gate)
    if torch.is_tensor(fr) and fr.dim() == 3:
        assert fr.shape == gate.shape, (fr.shape, gate.shape)            # slotkern_cuda.py:493
        fr_ = _as_f32(fr)
    else:
        fr_ = torch.as_tensor(fr, dtype=torch.float32, device=k.device).reshape(1)
    temp_ = torch.as_tensor(temp, dtype=torch.float32, device=k.device).reshape(1)   # slotkern_cuda.py:497
    out = ops.hard_fwd(k_, q_, v_, g_, fr_, temp_, int(N), int(G), bool(hard_gate), float(eps), bool(occ_bin),
                       out_dtype == torch.bfloat16)
    return out[0], out[1]


def kv_scan_c(k, v, gate, fr, N, temp, G=16, hard=False, hard_gate=False, eps=1e-4, detach_addr=False, q=None, nw=None,
              nwb=None, occ_bin=False, out_dtype=torch.float32):
    """Name under which the reference binds its CUDA scan (memlm_sh.py:48-50)."""
    return kv_scan_g(k, v, gate, fr, N, temp, G=G, hard=hard, hard_gate=hard_gate, eps=eps, detach_addr=detach_addr, q=q,
                     nw=nw, nwb=nwb, occ_bin=occ_bin, out_dtype=out_dtype)


def scan_kv(k, v, gate, fr, N, temp, G=1, hard=False, hard_gate=False, eps=1e-4, detach_addr=False, q=None):
    """The older per-layer model's entry point (memlm_kv.py:510-514): same scan, stride 1 by default, no occ_bin."""
    return kv_scan_g(k, v, gate, fr, N, temp, G=G, hard=hard, hard_gate=hard_gate, eps=eps, detach_addr=detach_addr, q=q)


def scan_with_log(k, v, gate, fr, N, temp, G=16, hard_gate=False, eps=1e-4, q=None, occ_bin=False,
                  out_dtype=torch.float32):
    """Forward only, returning the snapshots AND the log (addresses, undo rows, final state): what a caller that
    inspects addresses or streams a long context needs.  Keys: kbuf, vbuf, addr, oold, kold, vold, kfin, vfin, ofin,
    tfirst (include/slotscan.h: slotscan_log)."""
    if not k.is_cuda:
        raise RuntimeError("slotscan_b200.scan_with_log: CUDA tensors only (no CPU path in this package)")
    k_, v_, q_ = _token_streams(k, v, q)
    fr_ = _as_f32(fr) if (torch.is_tensor(fr) and fr.dim() == 3) else \
        torch.as_tensor(fr, dtype=torch.float32, device=k.device).reshape(1)
    temp_ = torch.as_tensor(temp, dtype=torch.float32, device=k.device).reshape(1)
    with torch.no_grad():
        out = ops.hard_fwd(k_, q_, v_, _as_f32(gate), fr_, temp_, int(N), int(G),
                           bool(hard_gate), float(eps), bool(occ_bin), out_dtype == torch.bfloat16)
    names = ("kbuf", "vbuf", "addr", "oold", "kold", "vold", "kfin", "vfin", "ofin", "tfirst", "kiold")
    return dict(zip(names, out))
