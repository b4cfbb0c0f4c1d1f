"""The scratch-free backward entry point (slotscan_hard_bwd_noalloc), called straight through the C ABI.

It exists for hosts that cannot give the library a scratch buffer -- device memory fully owned by their own arena, or
no allocator reachable from their binding -- so the table the backward needs sits in a fixed array inside the library.
Checked here: two calls in a row (different inputs, so the second one meets the first one's leftovers in the shared
array) each reproduce the ordinary entry point bit for bit, and a problem larger than the fixed array is refused
before anything is launched.  Collected last on purpose: a failure here cannot hide any other test's result.
"""
import ctypes

import pytest
import torch

from tests.scan_cases import make_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _forward(inp, N, G):
    import slotscan_b200 as S
    d = lambda x: x.to(DEV).contiguous()
    k, q, v, g, fr = d(inp["k"]), d(inp["q"]), d(inp["v"]), d(inp["gate"]), d(inp["fr"])
    lg = S.scan_with_log(k, v, g, fr, N, 16.0, G=G, q=q, occ_bin=True)
    return (k, q, v, g, fr), lg


def _both_backwards(tensors, lg, N, G, seed):
    from slotscan_b200 import _lib
    L = _lib.lib()
    k, q, v, g, fr = tensors
    B, T, H, DK = k.shape
    temp = torch.tensor([16.0], device=DEV)
    p = _lib.Params(B, T, H, N, DK, v.shape[-1], G, 0, 1, 1, _lib.F32, _lib.F32, 1e-4)
    log = _lib.Log(*(lg[n].data_ptr() for n in ("addr", "oold", "kold", "vold", "kfin", "vfin", "ofin", "tfirst", "kiold")))
    gen = torch.Generator(device=DEV).manual_seed(seed)
    dkb = torch.randn(lg["kbuf"].shape, device=DEV, generator=gen)
    dvb = torch.randn(lg["vbuf"].shape, device=DEV, generator=gen)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def outputs():
        return [torch.full_like(k, float("nan")), torch.full_like(k, float("nan")), torch.full_like(v, float("nan")),
                torch.full_like(g, float("nan")), torch.full_like(fr, float("nan")), torch.full((1,), float("nan"), device=DEV)]

    nbytes = L.slotscan_hard_bwd_scratch_bytes(ctypes.byref(p))
    assert nbytes <= L.slotscan_hard_bwd_noalloc_capacity()
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
    a = outputs()
    rc = L.slotscan_hard_bwd(ctypes.byref(p), _ptr(k), _ptr(q), _ptr(v), _ptr(g), _ptr(fr), _ptr(temp), ctypes.byref(log),
                             _ptr(dkb), _ptr(dvb), _ptr(scratch), nbytes, *(_ptr(t) for t in a), stream)
    assert rc == 0
    b = outputs()
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    rc = L.slotscan_hard_bwd_noalloc(ctypes.byref(p), _ptr(k), _ptr(q), _ptr(v), _ptr(g), _ptr(fr), _ptr(temp),
                                     ctypes.byref(log), _ptr(dkb), _ptr(dvb), *(_ptr(t) for t in b), stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    return a, b


def test_noalloc_backward_matches_ordinary_backward_twice():
    N, G = 48, 8
    for call, (dist, seed) in enumerate((("clustered", 21), ("bench", 22))):
        inp = make_inputs(dist, 2, 256, 3, 64, 64, seed=seed)
        tensors, lg = _forward(inp, N, G)
        a, b = _both_backwards(tensors, lg, N, G, seed=70 + call)
        for name, x, y in zip(("dk", "dq", "dv", "dgate", "dfr", "dtemp"), a, b):
            assert torch.isfinite(y).all(), (call, name)
            assert torch.equal(x, y), (call, name, (x - y).abs().max().item())


def test_noalloc_backward_refuses_what_does_not_fit():
    from slotscan_b200 import _lib
    L = _lib.lib()
    p = _lib.Params(64, 1024, 6, 192, 128, 128, 8, 0, 1, 1, _lib.F32, _lib.F32, 1e-4)      # table of 75 M entries
    assert L.slotscan_hard_bwd_scratch_bytes(ctypes.byref(p)) > L.slotscan_hard_bwd_noalloc_capacity()
    one = torch.zeros(64, device=DEV)
    log = _lib.Log(*([one.data_ptr()] * 9))
    rc = L.slotscan_hard_bwd_noalloc(ctypes.byref(p), *([_ptr(one)] * 6), ctypes.byref(log), None, None,
                                     *([_ptr(one)] * 6), None)
    assert rc == -6                                                                         # SLOTSCAN_E_TOO_LARGE
