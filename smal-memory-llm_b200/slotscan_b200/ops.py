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
# position of each output of hard_fwd
OUT = ("kbuf", "vbuf", "addr", "oold", "kold", "vold", "kfin", "vfin", "ofin", "tfirst", "kiold", "nsqfin", "kinv", "valid")


def _ptr(t):
    return None if t is None or t.numel() == 0 else ctypes.c_void_p(t.data_ptr())


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


def _addr(t):
    return 0 if t is None or t.numel() == 0 else t.data_ptr()


def _fwd_shapes(k, v, N, G, snap_bf16, want_norm, undo_log, new):
    """The output tensors of hard_fwd; `new(shape, dtype)` allocates (real or fake).  Outputs that were not asked
    for have zero elements."""
    B, T, H, DK = k.shape
    DV = v.shape[-1]
    NB = (T + G - 1) // G
    sdt = torch.bfloat16 if snap_bf16 else torch.float32
    f32, i32 = torch.float32, torch.int32
    return (new((B, NB, H, N, DK), sdt), new((B, NB, H, N, DV), sdt), new((B, T, H), i32), new((B, T, H), f32),
            new((B, T, H, DK) if undo_log else (0,), f32), new((B, T, H, DV) if undo_log else (0,), f32),
            new((B * H, N, DK), f32), new((B * H, N, DV), f32), new((B * H, N), f32), new((B * H, N), i32),
            new((B, T, H), f32), new((B * H, N), torch.float64),
            new((B, NB, H, N) if want_norm else (0,), f32), new((B, NB, H, N) if want_norm else (0,), torch.uint8))


@torch.library.custom_op("slotscan::hard_fwd", mutates_args=())
def hard_fwd(k: torch.Tensor, q: Optional[torch.Tensor], v: torch.Tensor, gate: torch.Tensor, fr: torch.Tensor,
             temp: torch.Tensor, K0: Optional[torch.Tensor], V0: Optional[torch.Tensor], o0: Optional[torch.Tensor],
             nsq0: Optional[torch.Tensor], N: int, G: int, hard_gate: bool, eps: float, occ_bin: bool,
             snap_bf16: bool, want_norm: bool, undo_log: bool
             ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
                        torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """k, q, v: contiguous f32 or bf16 (same dtype); gate, fr, temp: contiguous f32.  K0, V0, o0 (f32), nsq0 (f64):
    the state carried in from the preceding chunk, or None.  Returns, in the order of `OUT`: kbuf, vbuf, the log
    (addr, oold, kold, vold, kfin, vfin, ofin, tfirst, kiold; include/slotscan.h), nsqfin, kinv, valid."""
    _require_cuda(k, q, v, gate, fr, temp, K0, V0, o0, nsq0)
    dev = k.device
    out = _fwd_shapes(k, v, N, G, snap_bf16, want_norm, undo_log, lambda s, dt: torch.empty(s, device=dev, dtype=dt))
    kbuf, vbuf, addr, oold, kold, vold, kfin, vfin, ofin, tfirst, kiold, nsqfin, kinv, valid = out
    p = _params(k, v, gate, fr, N, G, hard_gate, eps, occ_bin, kbuf.dtype)
    log = _lib.Log(*(_addr(t) for t in (addr, oold, kold, vold, kfin, vfin, ofin, tfirst, kiold)))
    c = lambda t, dt: None if t is None else t.contiguous().to(dt)
    K0, V0, o0, nsq0 = c(K0, torch.float32), c(V0, torch.float32), c(o0, torch.float32), c(nsq0, torch.float64)
    ex = _lib.FwdExtra(_addr(K0), _addr(V0), _addr(o0), _addr(nsq0), _addr(nsqfin), _addr(kinv), _addr(valid),
                       0 if undo_log else 1)
    with torch.cuda.device(dev):
        rc = _lib.lib().slotscan_hard_fwd_ex(ctypes.byref(p), _ptr(k), _ptr(q), _ptr(v), _ptr(gate), _ptr(fr), _ptr(temp),
                                             _ptr(kbuf), _ptr(vbuf), ctypes.byref(log), ctypes.byref(ex), _stream(dev))
    _lib.check(rc, "slotscan_hard_fwd_ex")
    return out


@hard_fwd.register_fake
def _(k, q, v, gate, fr, temp, K0, V0, o0, nsq0, N, G, hard_gate, eps, occ_bin, snap_bf16, want_norm, undo_log):
    return _fwd_shapes(k, v, N, G, snap_bf16, want_norm, undo_log, lambda s, dt: k.new_empty(s, dtype=dt))


@torch.library.custom_op("slotscan::hard_bwd", mutates_args=())
def hard_bwd(k: torch.Tensor, q: Optional[torch.Tensor], v: torch.Tensor, gate: torch.Tensor, fr: torch.Tensor,
             temp: torch.Tensor, addr: torch.Tensor, oold: torch.Tensor, kold: torch.Tensor, vold: torch.Tensor,
             kfin: torch.Tensor, vfin: torch.Tensor, ofin: torch.Tensor, tfirst: torch.Tensor, kiold: torch.Tensor,
             dkbuf: Optional[torch.Tensor], dvbuf: Optional[torch.Tensor], dkinv: Optional[torch.Tensor], N: int, G: int,
             hard_gate: bool, eps: float, occ_bin: bool, snap_bf16: bool
             ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns dk, dq, dv (dtype of k), dgate (B,T,H) f32, dfr (shape of fr) f32, dtemp (1,) f32.
    With q None, dq holds the search-path part, which the kernel has already added into dk.
    dkinv: the gradient that reached the kinv output of the forward (B,NB,H,N) f32, or None."""
    _require_cuda(k, v)
    if kold.numel() == 0 or vold.numel() == 0:
        raise RuntimeError("slotscan: this forward was run without its undo log (forward-only mode); it has no backward")
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
        rc = L.slotscan_hard_bwd_ex(ctypes.byref(p), _ptr(k), _ptr(q), _ptr(v), _ptr(gate), _ptr(fr), _ptr(temp),
                                    ctypes.byref(log), _ptr(dkbuf), _ptr(dvbuf), _ptr(dkinv), _ptr(scratch), nbytes,
                                    _ptr(dk), _ptr(dq), _ptr(dv), _ptr(dgate), _ptr(dfr), _ptr(dtemp), _stream(dev))
    _lib.check(rc, "slotscan_hard_bwd_ex")
    return dk, dq, dv, dgate, dfr, dtemp


@hard_bwd.register_fake
def _(k, q, v, gate, fr, temp, addr, oold, kold, vold, kfin, vfin, ofin, tfirst, kiold, dkbuf, dvbuf, dkinv, N, G,
      hard_gate, eps, occ_bin, snap_bf16):
    f = lambda t: t.new_empty(t.shape, dtype=torch.float32)
    return torch.empty_like(k), torch.empty_like(k), torch.empty_like(v), f(gate), f(fr), gate.new_empty(1)


def _setup(ctx, inputs, output):
    k, q, v, gate, fr, temp, K0, V0, o0, nsq0, N, G, hard_gate, eps, occ_bin, snap_bf16, want_norm, undo_log = inputs
    ctx.save_for_backward(k, q, v, gate, fr, temp, *output[2:11])
    ctx.meta = (N, G, hard_gate, eps, occ_bin, snap_bf16)
    ctx.set_materialize_grads(False)


def _backward(ctx, *grads):
    dkbuf, dvbuf, dkinv = grads[0], grads[1], grads[12]
    k, q, v, gate, fr, temp, addr, oold, kold, vold, kfin, vfin, ofin, tfirst, kiold = ctx.saved_tensors
    N, G, hard_gate, eps, occ_bin, snap_bf16 = ctx.meta
    sdt = torch.bfloat16 if snap_bf16 else torch.float32
    c = lambda g, dt: None if g is None else g.contiguous().to(dt)
    dk, dq, dv, dgate, dfr, dtemp = hard_bwd(k, q, v, gate, fr, temp, addr, oold, kold, vold, kfin, vfin, ofin, tfirst,
                                             kiold, c(dkbuf, sdt), c(dvbuf, sdt), c(dkinv, torch.float32), N, G, hard_gate,
                                             eps, occ_bin, snap_bf16)
    # no gradient for the carried-in state (K0, V0, o0, nsq0) nor for the integer / flag arguments
    return (dk, (None if q is None else dq), dv, dgate, dfr, dtemp) + (None,) * 12


hard_fwd.register_autograd(_backward, setup_context=_setup)


# ------------------------------------------------------------------------------------------------------------------
# The general scan (soft address, attached address gradient): slotscan_dense_fwd / slotscan_dense_bwd.
def _dense_params(k, v, gate, fr, N, G, hard, hard_gate, eps, detach_addr, occ_bin):
    base = _params(k, v, gate, fr, N, G, hard_gate, eps, occ_bin, torch.float32)
    return _lib.DenseParams(base, int(hard), int(detach_addr))


@torch.library.custom_op("slotscan::dense_fwd", mutates_args=())
def dense_fwd(k: torch.Tensor, q: Optional[torch.Tensor], v: torch.Tensor, gate: torch.Tensor, fr: torch.Tensor,
              temp: torch.Tensor, N: int, G: int, hard: bool, hard_gate: bool, eps: float, detach_addr: bool,
              occ_bin: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
                                      torch.Tensor]:
    """Any mode of the scan.  Returns kbuf, vbuf (float32), obuf (B,NB,H,N), addr (B,T,H) int32, kfin, vfin, ofin."""
    _require_cuda(k, q, v, gate, fr, temp)
    B, T, H, DK = k.shape
    DV = v.shape[-1]
    NB = (T + G - 1) // G
    dev = k.device
    e = lambda *s, dt=torch.float32: torch.empty(*s, device=dev, dtype=dt)
    kbuf, vbuf, obuf = e(B, NB, H, N, DK), e(B, NB, H, N, DV), e(B, NB, H, N)
    addr = e(B, T, H, dt=torch.int32)
    kfin, vfin, ofin = e(B * H, N, DK), e(B * H, N, DV), e(B * H, N)
    p = _dense_params(k, v, gate, fr, N, G, hard, hard_gate, eps, detach_addr, occ_bin)
    _lib.check(_lib.lib().slotscan_dense_check(ctypes.byref(p)), "slotscan_dense_check")
    with torch.cuda.device(dev):
        rc = _lib.lib().slotscan_dense_fwd(ctypes.byref(p), _ptr(k), _ptr(q), _ptr(v), _ptr(gate), _ptr(fr), _ptr(temp),
                                           _ptr(kbuf), _ptr(vbuf), _ptr(obuf), _ptr(addr), _ptr(kfin), _ptr(vfin),
                                           _ptr(ofin), _stream(dev))
    _lib.check(rc, "slotscan_dense_fwd")
    return kbuf, vbuf, obuf, addr, kfin, vfin, ofin


@dense_fwd.register_fake
def _(k, q, v, gate, fr, temp, N, G, hard, hard_gate, eps, detach_addr, occ_bin):
    B, T, H, DK = k.shape
    DV = v.shape[-1]
    NB = (T + G - 1) // G
    e = lambda *s, dt=torch.float32: k.new_empty(s, dtype=dt)
    return (e(B, NB, H, N, DK), e(B, NB, H, N, DV), e(B, NB, H, N), e(B, T, H, dt=torch.int32), e(B * H, N, DK),
            e(B * H, N, DV), e(B * H, N))


@torch.library.custom_op("slotscan::dense_bwd", mutates_args=())
def dense_bwd(k: torch.Tensor, q: Optional[torch.Tensor], v: torch.Tensor, gate: torch.Tensor, fr: torch.Tensor,
              temp: torch.Tensor, kbuf: torch.Tensor, vbuf: torch.Tensor, obuf: torch.Tensor,
              dkbuf: Optional[torch.Tensor], dvbuf: Optional[torch.Tensor], N: int, G: int, hard: bool, hard_gate: bool,
              eps: float, detach_addr: bool, occ_bin: bool
              ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """dk, dq, dv (dtype of k), dgate, dfr (shape of fr), dtemp (1,).  With q None the search-path part in dq has
    already been added into dk."""
    _require_cuda(k, v, kbuf)
    dev = k.device
    p = _dense_params(k, v, gate, fr, N, G, hard, hard_gate, eps, detach_addr, occ_bin)
    L = _lib.lib()
    nbytes = L.slotscan_dense_bwd_scratch_bytes(ctypes.byref(p))
    scratch = torch.empty(nbytes, device=dev, dtype=torch.uint8)
    dk, dq, dv = torch.empty_like(k), torch.empty_like(k), torch.empty_like(v)
    dgate = torch.empty(gate.shape, device=dev, dtype=torch.float32)
    dfr = torch.empty(fr.shape, device=dev, dtype=torch.float32)
    dtemp = torch.empty(1, device=dev, dtype=torch.float32)
    with torch.cuda.device(dev):
        rc = L.slotscan_dense_bwd(ctypes.byref(p), _ptr(k), _ptr(q), _ptr(v), _ptr(gate), _ptr(fr), _ptr(temp), _ptr(kbuf),
                                  _ptr(vbuf), _ptr(obuf), _ptr(dkbuf), _ptr(dvbuf), _ptr(scratch), nbytes, _ptr(dk),
                                  _ptr(dq), _ptr(dv), _ptr(dgate), _ptr(dfr), _ptr(dtemp), _stream(dev))
    _lib.check(rc, "slotscan_dense_bwd")
    return dk, dq, dv, dgate, dfr, dtemp


@dense_bwd.register_fake
def _(k, q, v, gate, fr, temp, kbuf, vbuf, obuf, dkbuf, dvbuf, N, G, hard, hard_gate, eps, detach_addr, occ_bin):
    f = lambda t: t.new_empty(t.shape, dtype=torch.float32)
    return torch.empty_like(k), torch.empty_like(k), torch.empty_like(v), f(gate), f(fr), gate.new_empty(1)


def _dense_setup(ctx, inputs, output):
    k, q, v, gate, fr, temp, N, G, hard, hard_gate, eps, detach_addr, occ_bin = inputs
    ctx.save_for_backward(k, q, v, gate, fr, temp, output[0], output[1], output[2])
    ctx.meta = (N, G, hard, hard_gate, eps, detach_addr, occ_bin)
    ctx.set_materialize_grads(False)


def _dense_backward(ctx, dkbuf, dvbuf, *unused):
    k, q, v, gate, fr, temp, kbuf, vbuf, obuf = ctx.saved_tensors
    c = lambda g: None if g is None else g.contiguous().to(torch.float32)
    dk, dq, dv, dgate, dfr, dtemp = dense_bwd(k, q, v, gate, fr, temp, kbuf, vbuf, obuf, c(dkbuf), c(dvbuf), *ctx.meta)
    return (dk, (None if q is None else dq), dv, dgate, dfr, dtemp) + (None,) * 7


dense_fwd.register_autograd(_dense_backward, setup_context=_dense_setup)
