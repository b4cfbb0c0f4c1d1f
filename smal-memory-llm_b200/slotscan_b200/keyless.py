"""The keyless scan behind the reference's call signature (gqa25/slotkern_v.py:232):

    slot_scan_v(v, wa, gate, fr, N, C=256, G=1, buf_dtype=torch.float32, hard=False, hard_gate=False) -> buf

v (B,T,H,DV), wa (B,T,H,N) address logits (temperature already applied), gate (B,T,H), fr a scalar tensor; returns the
pre-write value buffer (B, ceil(T/G), H, N, DV) in buf_dtype.  Gradients for v, wa, gate, fr.  `C` (the checkpoint
interval of the reference's Triton backward) is accepted and ignored: the emitted buffer is the checkpoint here.
CUDA only: two kernels of libslotscan.so (slotscan_v_fwd / slotscan_v_bwd), no other implementation behind it.
"""
import ctypes
from typing import Optional, Tuple

import torch

from . import _lib
from .ops import _ptr, _require_cuda, _stream

_DT = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}


def _params(v, wa, G, hard, hard_gate):
    B, T, H, DV = v.shape
    return _lib.KeylessParams(B, T, H, wa.shape[-1], DV, G, int(hard), int(hard_gate), _DT[v.dtype])


@torch.library.custom_op("slotscan::keyless_fwd", mutates_args=())
def keyless_fwd(v: torch.Tensor, wa: torch.Tensor, gate: torch.Tensor, fr: torch.Tensor, G: int, hard: bool,
                hard_gate: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns buf (B,NB,H,N,DV) f32, obuf (B,NB,H,N) f32, addr (B,T,H) int32."""
    _require_cuda(v, wa, gate, fr)
    B, T, H, DV = v.shape
    N = wa.shape[-1]
    NB = (T + G - 1) // G
    buf = torch.empty(B, NB, H, N, DV, device=v.device, dtype=torch.float32)
    obuf = torch.empty(B, NB, H, N, device=v.device, dtype=torch.float32)
    addr = torch.empty(B, T, H, device=v.device, dtype=torch.int32)
    p = _params(v, wa, G, hard, hard_gate)
    _lib.check(_lib.lib().slotscan_v_check(ctypes.byref(p)), "slotscan_v_check")
    with torch.cuda.device(v.device):
        rc = _lib.lib().slotscan_v_fwd(ctypes.byref(p), _ptr(v), _ptr(wa), _ptr(gate), _ptr(fr), _ptr(buf), _ptr(obuf),
                                       _ptr(addr), _stream(v.device))
    _lib.check(rc, "slotscan_v_fwd")
    return buf, obuf, addr


@keyless_fwd.register_fake
def _(v, wa, gate, fr, G, hard, hard_gate):
    B, T, H, DV = v.shape
    N = wa.shape[-1]
    NB = (T + G - 1) // G
    return (v.new_empty((B, NB, H, N, DV), dtype=torch.float32), v.new_empty((B, NB, H, N), dtype=torch.float32),
            v.new_empty((B, T, H), dtype=torch.int32))


@torch.library.custom_op("slotscan::keyless_bwd", mutates_args=())
def keyless_bwd(v: torch.Tensor, wa: torch.Tensor, gate: torch.Tensor, fr: torch.Tensor, buf: torch.Tensor,
                obuf: torch.Tensor, dbuf: Optional[torch.Tensor], G: int, hard: bool, hard_gate: bool
                ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """dv (dtype of v), dwa, dgate, dfr (1,)."""
    _require_cuda(v, wa, buf)
    dev = v.device
    p = _params(v, wa, G, hard, hard_gate)
    L = _lib.lib()
    nbytes = L.slotscan_v_bwd_scratch_bytes(ctypes.byref(p))
    scratch = torch.empty(nbytes, device=dev, dtype=torch.uint8)
    dv, dwa = torch.empty_like(v), torch.empty_like(wa)
    dgate = torch.empty(gate.shape, device=dev, dtype=torch.float32)
    dfr = torch.empty(1, device=dev, dtype=torch.float32)
    with torch.cuda.device(dev):
        rc = L.slotscan_v_bwd(ctypes.byref(p), _ptr(v), _ptr(wa), _ptr(gate), _ptr(fr), _ptr(buf), _ptr(obuf), _ptr(dbuf),
                              _ptr(scratch), nbytes, _ptr(dv), _ptr(dwa), _ptr(dgate), _ptr(dfr), _stream(dev))
    _lib.check(rc, "slotscan_v_bwd")
    return dv, dwa, dgate, dfr


@keyless_bwd.register_fake
def _(v, wa, gate, fr, buf, obuf, dbuf, G, hard, hard_gate):
    return torch.empty_like(v), torch.empty_like(wa), gate.new_empty(gate.shape, dtype=torch.float32), gate.new_empty(1)


def _setup(ctx, inputs, output):
    v, wa, gate, fr, G, hard, hard_gate = inputs
    ctx.save_for_backward(v, wa, gate, fr, output[0], output[1])
    ctx.meta = (G, hard, hard_gate)
    ctx.set_materialize_grads(False)


def _backward(ctx, dbuf, *unused):
    v, wa, gate, fr, buf, obuf = ctx.saved_tensors
    d = None if dbuf is None else dbuf.contiguous().to(torch.float32)
    dv, dwa, dgate, dfr = keyless_bwd(v, wa, gate, fr, buf, obuf, d, *ctx.meta)
    return dv, dwa, dgate, dfr, None, None, None


keyless_fwd.register_autograd(_backward, setup_context=_setup)


def slot_scan_v(v, wa, gate, fr, N, C=256, G=1, buf_dtype=torch.float32, hard=False, hard_gate=False):
    if not v.is_cuda:
        raise RuntimeError("slotscan_b200.slot_scan_v: CUDA tensors only (no CPU path in this package)")
    if wa.shape[-1] != N or wa.shape[:3] != v.shape[:3]:
        raise ValueError("wa must be (B, T, H, N) with N = %d, got %s" % (N, tuple(wa.shape)))
    v_ = v.contiguous() if v.dtype == torch.bfloat16 else v.contiguous().to(torch.float32)
    f = lambda x: x.contiguous().to(torch.float32)
    fr_ = torch.as_tensor(fr, dtype=torch.float32, device=v.device).reshape(1)     # slotkern_v.py:239
    buf = keyless_fwd(v_, f(wa), f(gate), fr_, int(G), bool(hard), bool(hard_gate))[0]
    return buf.to(buf_dtype)
