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
  * hard=True with detach_addr=True (the training mode of the reference run) takes the specialised kernels; every other
    combination (soft address, attached address gradient) the general ones (csrc/slotscan_dense.cu).
  * write_memory(...) is the writer layer's whole hand-over in one call: scan + the epilogue of memlm_sh.py:464-475
    (kinv, valid, storage quantisation); StreamingScan carries the slot state from one chunk of a long context to
    the next (the reference keeps no state across calls, memlm_sh.py:676).
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
    if not (hard and detach_addr):
        # soft address and / or address gradient attached to the stored keys: the general kernels (float32 snapshots,
        # which are also the checkpoints of their backward; a bf16 hand-over is a cast of the result)
        out = ops.dense_fwd(k_, q_, v_, g_, fr_, temp_, int(N), int(G), bool(hard), bool(hard_gate), float(eps),
                            bool(detach_addr), bool(occ_bin))
        return out[0].to(out_dtype), out[1].to(out_dtype)
    out = ops.hard_fwd(k_, q_, v_, g_, fr_, temp_, None, None, None, None, int(N), int(G), bool(hard_gate), float(eps),
                       bool(occ_bin), out_dtype == torch.bfloat16, False, True)
    return out[0], out[1]


def kv_scan_c(k, v, gate, fr, N, temp, G=16, hard=False, hard_gate=False, eps=1e-4, detach_addr=False, q=None, nw=None,
              nwb=None, occ_bin=False, out_dtype=torch.float32):
    """Name under which the reference binds its CUDA scan (memlm_sh.py:48-50)."""
    return kv_scan_g(k, v, gate, fr, N, temp, G=G, hard=hard, hard_gate=hard_gate, eps=eps, detach_addr=detach_addr, q=q,
                     nw=nw, nwb=nwb, occ_bin=occ_bin, out_dtype=out_dtype)


def scan_kv(k, v, gate, fr, N, temp, G=1, hard=False, hard_gate=False, eps=1e-4, detach_addr=False, q=None):
    """The older per-layer model's entry point (memlm_kv.py:510-514): same scan, stride 1 by default, no occ_bin."""
    return kv_scan_g(k, v, gate, fr, N, temp, G=G, hard=hard, hard_gate=hard_gate, eps=eps, detach_addr=detach_addr, q=q)


def _scalars(fr, temp, device):
    fr_ = _as_f32(fr) if (torch.is_tensor(fr) and fr.dim() == 3) else \
        torch.as_tensor(fr, dtype=torch.float32, device=device).reshape(1)
    return fr_, torch.as_tensor(temp, dtype=torch.float32, device=device).reshape(1)


def scan_with_log(k, v, gate, fr, N, temp, G=16, hard_gate=False, eps=1e-4, q=None, occ_bin=False,
                  out_dtype=torch.float32, state=None, want_norm=False, undo_log=True):
    """Forward only, returning the snapshots AND the log (addresses, undo rows, final state): what a caller that
    inspects addresses or streams a long context needs.  Keys: kbuf, vbuf, addr, oold, kold, vold, kfin, vfin, ofin,
    tfirst, kiold (include/slotscan.h: slotscan_log), nsqfin, and with want_norm kinv, valid (bool).
    state: (K0, V0, o0) or (K0, V0, o0, nsq0) -- kfin, vfin, ofin[, nsqfin] of the call that scanned the preceding
    tokens; snapshot 0 is then that state.  undo_log=False skips the rows-before-each-write log (kold, vold come back
    empty): less memory and traffic for inference."""
    if not k.is_cuda:
        raise RuntimeError("slotscan_b200.scan_with_log: CUDA tensors only (no CPU path in this package)")
    k_, v_, q_ = _token_streams(k, v, q)
    fr_, temp_ = _scalars(fr, temp, k.device)
    st = (None, None, None, None) if state is None else (tuple(state) + (None,))[:4]
    with torch.no_grad():
        out = ops.hard_fwd(k_, q_, v_, _as_f32(gate), fr_, temp_, st[0], st[1], st[2], st[3], int(N), int(G),
                           bool(hard_gate), float(eps), bool(occ_bin), out_dtype == torch.bfloat16, bool(want_norm),
                           bool(undo_log))
    d = dict(zip(ops.OUT, out))
    if want_norm:
        d["valid"] = d["valid"].bool()
    else:
        del d["kinv"], d["valid"]
    return d


def write_memory(k, v, gate, fr, N, temp, G=16, hard_gate=False, eps=1e-4, q=None, occ_bin=False,
                 out_dtype=torch.bfloat16, qbits=0, qgroup=16):
    """What a writer layer hands to its readers, in one call: `(kbuf', buf', kinv, valid)`  [memlm_sh.py:454-475: the
    scan, then nsq / kinv / valid from the float32 keys, the cast to the model dtype, and `_quantize_mem` when the
    storage is quantised].  Hard address, address gradient detached (the reference's training mode).
    qbits = 0: the scan kernels emit the snapshots in `out_dtype` and kinv / valid from the float32 state while each
    key row is in registers -- no pass over the snapshots at all; in the backward the kinv gradient enters the key rows
    inside the reverse row scan.  qbits in {2,3,4,8}: float32 snapshots, then one quantiser pass (`writer_epilogue`).
    Differentiable in k, q, v, gate, fr, temp."""
    if not k.is_cuda:
        raise RuntimeError("slotscan_b200.write_memory: CUDA tensors only (no CPU path in this package)")
    if out_dtype not in (torch.float32, torch.bfloat16):
        raise ValueError("out_dtype must be float32 or bfloat16")
    if qbits:
        from .epilogue import writer_epilogue
        kb, vb = kv_scan_g(k, v, gate, fr, N, temp, G=G, hard=True, hard_gate=hard_gate, eps=eps, detach_addr=True, q=q,
                           occ_bin=occ_bin, out_dtype=torch.float32)
        return writer_epilogue(kb, vb, out_dtype, qbits=qbits, qgroup=qgroup)
    k_, v_, q_ = _token_streams(k, v, q)
    fr_, temp_ = _scalars(fr, temp, k.device)
    out = ops.hard_fwd(k_, q_, v_, _as_f32(gate), fr_, temp_, None, None, None, None, int(N), int(G), bool(hard_gate),
                       float(eps), bool(occ_bin), out_dtype == torch.bfloat16, True, True)
    return out[0], out[1], out[12], out[13].bool()


class StreamingScan:
    """A long context scanned chunk by chunk with the slot state carried across calls, forward only: memory use is that
    of one chunk, whatever the total length.  Each `push` takes the next tokens of every sequence and returns what the
    readers of that chunk need, `(kbuf', buf', kinv, valid)` as `write_memory` does (snapshots of the chunk only; the
    first one is the state the previous chunk ended in).  Chunk lengths must be multiples of G except the last one.
    [The reference scans a long context in one call and keeps no state across calls (memlm_sh.py:676); its CUDA kernel
    cannot run T = 131,072 at all (8 T bytes of dynamic shared memory, slotkern_cuda.py:507).]"""

    def __init__(self, N, temp, G=16, hard_gate=False, eps=1e-4, occ_bin=False, out_dtype=torch.bfloat16, qbits=0,
                 qgroup=16):
        self.kw = dict(N=N, temp=temp, G=G, hard_gate=hard_gate, eps=eps, occ_bin=occ_bin)
        self.out_dtype, self.qbits, self.qgroup, self.G = out_dtype, qbits, qgroup, G
        self.state, self.tokens = None, 0

    def push(self, k, v, gate, fr, q=None):
        if self.tokens % self.G:
            raise ValueError("StreamingScan: only the last chunk may have a length that is not a multiple of G")
        emit = torch.float32 if self.qbits else self.out_dtype
        lg = scan_with_log(k, v, gate, fr, q=q, out_dtype=emit, state=self.state, want_norm=not self.qbits,
                           undo_log=False, **self.kw)
        self.state = (lg["kfin"], lg["vfin"], lg["ofin"], lg["nsqfin"])
        self.tokens += k.shape[1]
        if self.qbits:
            from .epilogue import writer_epilogue
            return writer_epilogue(lg["kbuf"], lg["vbuf"], self.out_dtype, qbits=self.qbits, qgroup=self.qgroup)
        return lg["kbuf"], lg["vbuf"], lg["kinv"], lg["valid"]
