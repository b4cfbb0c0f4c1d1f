"""Writer epilogue and storage quantiser of the shared memory, on the snapshots the scan emitted.

Mirrors, with the reference's names and argument meaning (gqa25/memlm_sh.py):
  _fq(x, bits, group)                      :221-229   midrise group quantiser, straight-through gradient
  _quantize_mem(kbuf, buf, bits, group)    :231-234   (kq, vq, kinv, valid) from the quantised keys
  the unquantised epilogue                 :474-475   nsq = sum kbuf^2, kinv = rsqrt(max(nsq, 1e-12)), valid = nsq > 1e-12,
                                                      snapshots cast to the model dtype
One CUDA pass per tensor (slotscan_writer_epilogue); there is no other implementation behind these functions.
"""
import ctypes
from typing import Tuple

import torch

from . import _lib
from .ops import _ptr, _require_cuda, _stream

_CODE = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}
E4M3 = "e4m3"            # value of `bits` / `qbits` for fp8-e4m3 storage with one absmax scale per row (SLOTSCAN_BITS_E4M3)


def _bits(bits):
    """2, 3, 4, 8 (the reference's midrise quantiser), 0 (none) or "e4m3" -> the C ABI's code."""
    return -8 if bits == E4M3 else int(bits)


def _run(x, out_dtype, bits, group, want_y, want_norm):
    _require_cuda(x)
    if x.dtype not in _CODE or out_dtype not in _CODE:
        raise TypeError("writer epilogue: float32 or bfloat16 tensors only, got %s -> %s" % (x.dtype, out_dtype))
    x = x.contiguous()
    D = x.shape[-1]
    rows = x.numel() // D if D else 0
    p = _lib.EpilogueParams(rows, D, _CODE[x.dtype], _CODE[out_dtype], int(bits), int(group))
    _lib.check(_lib.lib().slotscan_epilogue_check(ctypes.byref(p)), "slotscan_epilogue_check")
    y = torch.empty(x.shape, dtype=out_dtype, device=x.device) if want_y else None
    kinv = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device) if want_norm else None
    valid = torch.empty(x.shape[:-1], dtype=torch.uint8, device=x.device) if want_norm else None
    if rows == 0:                                      # nothing to launch; an empty tensor has no address to pass
        return y, kinv, valid
    with torch.cuda.device(x.device):
        rc = _lib.lib().slotscan_writer_epilogue(ctypes.byref(p), _ptr(x), _ptr(y) if want_y else None,
                                                 _ptr(kinv) if want_norm else None, _ptr(valid) if want_norm else None,
                                                 _stream(x.device))
    _lib.check(rc, "slotscan_writer_epilogue")
    return y, kinv, valid


@torch.library.custom_op("slotscan::fq", mutates_args=())
def _fq_op(x: torch.Tensor, bits: int, group: int) -> torch.Tensor:
    return _run(x, x.dtype, bits, group, True, False)[0]


@_fq_op.register_fake
def _(x, bits, group):
    return torch.empty_like(x)


def _fq_setup(ctx, inputs, output):
    pass


def _fq_backward(ctx, dy):
    return dy, None, None                              # straight-through (memlm_sh.py:229)


_fq_op.register_autograd(_fq_backward, setup_context=_fq_setup)


def fq(x, bits, group=16):
    """`_fq(x, bits, group)` of the reference (memlm_sh.py:221-229): forward the quantised value, gradient identity.
    bits = "e4m3": fp8-e4m3 storage with one scale per row (no counterpart in the reference; `group` ignored)."""
    if bits != E4M3 and x.shape[-1] % group:
        raise ValueError("group %d does not divide the channel count %d" % (group, x.shape[-1]))
    return _fq_op(x, _bits(bits), int(group))


@torch.library.custom_op("slotscan::epilogue", mutates_args=())
def _epilogue_op(kbuf: torch.Tensor, out_bf16: bool, bits: int, group: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    y, kinv, valid = _run(kbuf, torch.bfloat16 if out_bf16 else torch.float32, bits, group, True, True)
    return y, kinv, valid


@_epilogue_op.register_fake
def _(kbuf, out_bf16, bits, group):
    return (torch.empty(kbuf.shape, dtype=torch.bfloat16 if out_bf16 else torch.float32, device=kbuf.device),
            torch.empty(kbuf.shape[:-1], dtype=torch.float32, device=kbuf.device),
            torch.empty(kbuf.shape[:-1], dtype=torch.uint8, device=kbuf.device))


def _ep_setup(ctx, inputs, output):
    kbuf, out_bf16, bits, group = inputs
    ctx.in_bf16 = kbuf.dtype == torch.bfloat16
    ctx.bits, ctx.group = int(bits), int(group)
    # d nsq / d kbuf = 2 * (the value the norm was taken of): the quantised keys BEFORE the cast to the output dtype when
    # bits != 0 [memlm_sh.py:232-234, 471-472].  The emitted keys may be bf16-rounded, so the backward requantises the
    # saved input in its own precision (one more pass of the quantiser kernel) instead of saving the output.
    ctx.save_for_backward(kbuf, output[1], output[2])


def _ep_backward(ctx, dy, dkinv, dvalid):
    # kinv = nsq^(-1/2) where valid: d nsq = -kinv^3 / 2 * dkinv, d kbuf = 2 kq * d nsq; the cast and the quantiser
    # pass dy straight through.  Elementwise torch ops on the device: not a kernel of this library yet.
    kq, kinv, valid = ctx.saved_tensors
    if ctx.bits:
        kq = _fq_op(kq, ctx.bits, ctx.group)
    in_dtype = torch.bfloat16 if ctx.in_bf16 else torch.float32
    g = dy.to(in_dtype)
    if dkinv is not None:
        w = torch.where(valid.bool(), -(kinv ** 3) * dkinv, torch.zeros_like(kinv))
        g = g + (w.unsqueeze(-1) * kq.float()).to(in_dtype)
    return g, None, None, None


_epilogue_op.register_autograd(_ep_backward, setup_context=_ep_setup)


def writer_epilogue(kbuf, buf, out_dtype, qbits=0, qgroup=16):
    """What the writer hands to the readers (memlm_sh.py:464-475): `(kbuf', buf', kinv, valid)` with the snapshots
    cast to `out_dtype`, quantised first when `qbits` is 2, 3, 4 or 8 (`_quantize_mem`) or "e4m3" (fp8 storage, one
    scale per row).  `valid` is a bool tensor."""
    if out_dtype not in _CODE:
        raise TypeError("out_dtype must be float32 or bfloat16")
    kq, kinv, valid = _epilogue_op(kbuf, out_dtype == torch.bfloat16, _bits(qbits), int(qgroup))
    vq = fq(buf, qbits, qgroup).to(out_dtype) if qbits else buf.to(out_dtype)
    return kq, vq, kinv, valid.bool()


def quantize_mem(kbuf, buf, bits, group):
    """`_quantize_mem(kbuf, buf, bits, group)` of the reference (memlm_sh.py:231-234): dtypes unchanged."""
    kq, kinv, valid = _epilogue_op(kbuf, kbuf.dtype == torch.bfloat16, _bits(bits), int(group))
    return kq, fq(buf, bits, group), kinv, valid.bool()
