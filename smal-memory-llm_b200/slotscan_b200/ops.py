"""torch custom ops over the C-ABI library: `slotscan::hard_fwd` / `slotscan::hard_bwd` with a registered autograd
formula and fake (meta) implementations, so the op can sit inside torch.compile'd model blocks without a graph
break (the reference calls its scan from compiled blocks, gqa25/train_sh.py:783-793).

torch is plumbing here -- it owns device memory and the stream; every computation is a kernel of libslotscan.so.
"""
import ctypes
from typing import Optional, Tuple

import torch

from . import _lib

_DT = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(dev):
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _params(k, v, gate, fr, N, G, hard_gate, eps, occ_bin, snap_dtype):
    B, T, H, DK = k.shape
    return _lib.Params(B, T, H, N, DK, v.shape[-1], G, int(hard_gate), int(occ_bin), int(fr.dim() == 3),
                       _DT[k.dtype], _DT[snap_dtype], float(eps))


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("slotscan ops run on CUDA tensors only: there is no CPU implementation in this package "
                               "(the CPU oracle lives in the test tree)")


@torch.library.custom_op("slotscan::hard_fwd", mutates_args=())
def hard_fwd(k: torch.Tensor, q: Optional[torch.Tensor], v: torch.Tensor, gate: torch.Tensor, fr: torch.Tensor,
             temp: torch.Tensor, N: int, G: int, hard_gate: bool, eps: float, occ_bin: bool,
             snap_bf16: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
                                       torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
                                       torch.Tensor]:
    """k, q, v: contiguous f32 or bf16 (same dtype); gate, fr, temp: contiguous f32.
    Returns kbuf, vbuf, then the log: addr, oold, kold, vold, kfin, vfin, ofin, tfirst, kiold (include/slotscan.h)."""
    _require_cuda(k, q, v, gate, fr, temp)
    B, T, H, DK = k.shape
    DV = v.shape[-1]
    NB = (T + G - 1) // G
    dev = k.device
    sdt = torch.bfloat16 if snap_bf16 else torch.float32
    e = lambda *s, dt=torch.float32: torch.empty(*s, device=dev, dtype=dt)
    kbuf, vbuf = e(B, NB, H, N, DK, dt=sdt), e(B, NB, H, N, DV, dt=sdt)
    addr, oold = e(B, T, H, dt=torch.int32), e(B, T, H)
    kold, vold = e(B, T, H, DK), e(B, T, H, DV)
    kfin, vfin, ofin = e(B * H, N, DK), e(B * H, N, DV), e(B * H, N)
    tfirst = e(B * H, N, dt=torch.int32)
    kiold = e(B, T, H)
    p = _params(k, v, gate, fr, N, G, hard_gate, eps, occ_bin, sdt)
    log = _lib.Log(*(t.data_ptr() for t in (addr, oold, kold, vold, kfin, vfin, ofin, tfirst, kiold)))
    with torch.cuda.device(dev):
        rc = _lib.lib().slotscan_hard_fwd(ctypes.byref(p), _ptr(k), _ptr(q), _ptr(v), _ptr(gate), _ptr(fr), _ptr(temp),
                                          _ptr(kbuf), _ptr(vbuf), ctypes.byref(log), _stream(dev))
    _lib.check(rc, "slotscan_hard_fwd")
    return kbuf, vbuf, addr, oold, kold, vold, kfin, vfin, ofin, tfirst, kiold


@hard_fwd.register_fake
def _(k, q, v, gate, fr, temp, N, G, hard_gate, eps, occ_bin, snap_bf16):
    B, T, H, DK = k.shape
    DV = v.shape[-1]
    NB = (T + G - 1) // G
    sdt = torch.bfloat16 if snap_bf16 else torch.float32
    e = lambda *s, dt=torch.float32: k.new_empty(s, dtype=dt)
    return (e(B, NB, H, N, DK, dt=sdt), e(B, NB, H, N, DV, dt=sdt), e(B, T, H, dt=torch.int32), e(B, T, H),
            e(B, T, H, DK), e(B, T, H, DV), e(B * H, N, DK), e(B * H, N, DV), e(B * H, N), e(B * H, N, dt=torch.int32),
            e(B, T, H))


@torch.library.custom_op("slotscan::hard_bwd", mutates_args=())
def hard_bwd(k: torch.Tensor, q: Optional[torch.Tensor], v: torch.Tensor, gate: torch.Tensor, fr: torch.Tensor,
             temp: torch.Tensor, addr: torch.Tensor, oold: torch.Tensor, kold: torch.Tensor, vold: torch.Tensor,
             kfin: torch.Tensor, vfin: torch.Tensor, ofin: torch.Tensor, tfirst: torch.Tensor, kiold: torch.Tensor,
             dkbuf: Optional[torch.Tensor], dvbuf: Optional[torch.Tensor], N: int, G: int, hard_gate: bool,
             eps: float, occ_bin: bool, snap_bf16: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor,
                                                                   torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns dk, dq, dv (dtype of k), dgate (B,T,H) f32, dfr (shape of fr) f32, dtemp (1,) f32.
    With q None, dq holds the search-path part, which the kernel has already added into dk."""
    _require_cuda(k, v)
    dev = k.device
    sdt = torch.bfloat16 if snap_bf16 else torch.float32
    p = _params(k, v, gate, fr, N, G, hard_gate, eps, occ_bin, sdt)
    L = _lib.lib()
    nbytes = L.slotscan_hard_bwd_scratch_bytes(ctypes.byref(p))
    scratch = torch.empty(nbytes, device=dev, dtype=torch.uint8)
    dk, dq, dv = torch.empty_like(k), torch.empty_like(k), torch.empty_like(v)
    dgate = torch.empty(gate.shape, device=dev, dtype=torch.float32)
    dfr = torch.empty(fr.shape, device=dev, dtype=torch.float32)
    dtemp = torch.empty(1, device=dev, dtype=torch.float32)
    log = _lib.Log(*(t.data_ptr() for t in (addr, oold, kold, vold, kfin, vfin, ofin, tfirst, kiold)))
    with torch.cuda.device(dev):
        rc = L.slotscan_hard_bwd(ctypes.byref(p), _ptr(k), _ptr(q), _ptr(v), _ptr(gate), _ptr(fr), _ptr(temp),
                                 ctypes.byref(log), _ptr(dkbuf), _ptr(dvbuf), _ptr(scratch), nbytes, _ptr(dk), _ptr(dq),
                                 _ptr(dv), _ptr(dgate), _ptr(dfr), _ptr(dtemp), _stream(dev))
    _lib.check(rc, "slotscan_hard_bwd")
    return dk, dq, dv, dgate, dfr, dtemp


@hard_bwd.register_fake
def _(k, q, v, gate, fr, temp, addr, oold, kold, vold, kfin, vfin, ofin, tfirst, kiold, dkbuf, dvbuf, N, G, hard_gate,
      eps, occ_bin, snap_bf16):
    f = lambda t: t.new_empty(t.shape, dtype=torch.float32)
    return torch.empty_like(k), torch.empty_like(k), torch.empty_like(v), f(gate), f(fr), gate.new_empty(1)


def _setup(ctx, inputs, output):
    k, q, v, gate, fr, temp, N, G, hard_gate, eps, occ_bin, snap_bf16 = inputs
    ctx.save_for_backward(k, q, v, gate, fr, temp, *output[2:])
    ctx.meta = (N, G, hard_gate, eps, occ_bin, snap_bf16)
    ctx.set_materialize_grads(False)


def _backward(ctx, dkbuf, dvbuf, *unused):
    k, q, v, gate, fr, temp, addr, oold, kold, vold, kfin, vfin, ofin, tfirst, kiold = ctx.saved_tensors
    N, G, hard_gate, eps, occ_bin, snap_bf16 = ctx.meta
    sdt = torch.bfloat16 if snap_bf16 else torch.float32
    c = lambda g: None if g is None else g.contiguous().to(sdt)
    dk, dq, dv, dgate, dfr, dtemp = hard_bwd(k, q, v, gate, fr, temp, addr, oold, kold, vold, kfin, vfin, ofin, tfirst,
                                             kiold, c(dkbuf), c(dvbuf), N, G, hard_gate, eps, occ_bin, snap_bf16)
    return dk, (None if q is None else dq), dv, dgate, dfr, dtemp, None, None, None, None, None, None


hard_fwd.register_autograd(_backward, setup_context=_setup)
