"""Cosine read of the stride-G snapshots: the core of `SharedMixer._read` (gqa25/memlm_sh.py:379-397) after the
caller's projections, forward and backward.  Two CUDA kernels (slotscan_read_fwd / slotscan_read_bwd); no other
implementation behind them."""
from typing import Tuple

import ctypes

import torch

from . import _lib
from .ops import _ptr, _require_cuda, _stream

_CODE = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}


@torch.library.custom_op("slotscan::read_fwd", mutates_args=())
def _read_op(qr: torch.Tensor, sharp: torch.Tensor, kbuf: torch.Tensor, vbuf: torch.Tensor, kinv: torch.Tensor,
             valid: torch.Tensor, G: int) -> torch.Tensor:
    _require_cuda(qr, sharp, kbuf, vbuf, kinv, valid)
    if qr.dtype not in _CODE or kbuf.dtype not in _CODE or vbuf.dtype != kbuf.dtype:
        raise TypeError("read: float32 or bfloat16 queries and snapshots (keys and values alike)")
    B, T, H, NQ, DK = qr.shape
    NB, N, DV = kbuf.shape[1], kbuf.shape[3], vbuf.shape[-1]
    if NB != (T + G - 1) // G or kbuf.shape != (B, NB, H, N, DK) or vbuf.shape != (B, NB, H, N, DV):
        raise ValueError("read: snapshots %s / %s do not match queries %s with G = %d"
                         % (tuple(kbuf.shape), tuple(vbuf.shape), tuple(qr.shape), G))
    if sharp.shape != (B, T, H, NQ) or kinv.shape != (B, NB, H, N) or valid.shape != (B, NB, H, N):
        raise ValueError("read: sharp / kinv / valid have the wrong shape")
    p = _lib.ReadParams(B, T, H, NQ, N, DK, DV, G, _CODE[qr.dtype], _CODE[kbuf.dtype])
    _lib.check(_lib.lib().slotscan_read_check(ctypes.byref(p)), "slotscan_read_check")
    qr, kbuf, vbuf = qr.contiguous(), kbuf.contiguous(), vbuf.contiguous()
    sharp, kinv = sharp.float().contiguous(), kinv.float().contiguous()
    valid = valid.to(torch.uint8).contiguous()
    rd = torch.empty(B, T, H, NQ, DV, dtype=qr.dtype, device=qr.device)
    with torch.cuda.device(qr.device):
        rc = _lib.lib().slotscan_read_fwd(ctypes.byref(p), _ptr(qr), _ptr(sharp), _ptr(kbuf), _ptr(vbuf), _ptr(kinv),
                                          _ptr(valid), _ptr(rd), _stream(qr.device))
    _lib.check(rc, "slotscan_read_fwd")
    return rd


@_read_op.register_fake
def _(qr, sharp, kbuf, vbuf, kinv, valid, G):
    return torch.empty(*qr.shape[:-1], vbuf.shape[-1], dtype=qr.dtype, device=qr.device)


def _prep(qr, sharp, kbuf, vbuf, kinv, valid, G):
    B, T, H, NQ, DK = qr.shape
    NB, N, DV = kbuf.shape[1], kbuf.shape[3], vbuf.shape[-1]
    p = _lib.ReadParams(B, T, H, NQ, N, DK, DV, G, _CODE[qr.dtype], _CODE[kbuf.dtype])
    _lib.check(_lib.lib().slotscan_read_check(ctypes.byref(p)), "slotscan_read_check")
    return (p, qr.contiguous(), sharp.float().contiguous(), kbuf.contiguous(), vbuf.contiguous(),
            kinv.float().contiguous(), valid.to(torch.uint8).contiguous())


@torch.library.custom_op("slotscan::read_bwd", mutates_args=())
def _read_bwd_op(qr: torch.Tensor, sharp: torch.Tensor, kbuf: torch.Tensor, vbuf: torch.Tensor, kinv: torch.Tensor,
                 valid: torch.Tensor, drd: torch.Tensor, G: int
                 ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    _require_cuda(qr, sharp, kbuf, vbuf, kinv, valid, drd)
    p, qr, sharp, kbuf, vbuf, kinv, valid = _prep(qr, sharp, kbuf, vbuf, kinv, valid, G)
    drd = drd.to(qr.dtype).contiguous()
    dqr, dsharp = torch.empty_like(qr), torch.empty_like(sharp)
    dkbuf, dvbuf, dkinv = torch.empty_like(kbuf), torch.empty_like(vbuf), torch.empty_like(kinv)
    with torch.cuda.device(qr.device):
        rc = _lib.lib().slotscan_read_bwd(ctypes.byref(p), _ptr(qr), _ptr(sharp), _ptr(kbuf), _ptr(vbuf), _ptr(kinv),
                                          _ptr(valid), _ptr(drd), _ptr(dqr), _ptr(dsharp), _ptr(dkbuf), _ptr(dvbuf),
                                          _ptr(dkinv), _stream(qr.device))
    _lib.check(rc, "slotscan_read_bwd")
    return dqr, dsharp, dkbuf, dvbuf, dkinv


@_read_bwd_op.register_fake
def _(qr, sharp, kbuf, vbuf, kinv, valid, drd, G):
    return (torch.empty_like(qr), torch.empty_like(sharp, dtype=torch.float32), torch.empty_like(kbuf),
            torch.empty_like(vbuf), torch.empty_like(kinv, dtype=torch.float32))


def _rd_setup(ctx, inputs, output):
    qr, sharp, kbuf, vbuf, kinv, valid, G = inputs
    ctx.save_for_backward(qr, sharp, kbuf, vbuf, kinv, valid)
    ctx.G = G
    ctx.dtypes = (sharp.dtype, kinv.dtype)


def _rd_backward(ctx, drd):
    qr, sharp, kbuf, vbuf, kinv, valid = ctx.saved_tensors
    dqr, dsharp, dkbuf, dvbuf, dkinv = _read_bwd_op(qr, sharp, kbuf, vbuf, kinv, valid, drd, ctx.G)
    return dqr, dsharp.to(ctx.dtypes[0]), dkbuf, dvbuf, dkinv.to(ctx.dtypes[1]), None, None


_read_op.register_autograd(_rd_backward, setup_context=_rd_setup)


def read_snapshots(qr, sharp, kbuf, vbuf, kinv, valid, G):
    """rd (B,T,H,NQ,dv): token t reads the snapshot of block t // G.  `qr` (B,T,H,NQ,dk) are the projected read
    queries (normalised inside, memlm_sh.py:379), `sharp` (B,T,H,NQ) the sharpness multiplier the caller forms
    (:383-393), `kinv`, `valid` come from `writer_epilogue`.  Differentiable in qr, sharp, kbuf, vbuf and kinv."""
    return _read_op(qr, sharp, kbuf, vbuf, kinv, valid, int(G))
