"""CPU-side checks of the boundary: the C-ABI library loads and exports every function include/slotscan.h declares,
argument validation rejects bad shapes without touching a GPU, the Python host mirrors the reference signatures, and
the product refuses to run without CUDA (no fallback)."""
import ctypes
import inspect
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    src = open(os.path.join(ROOT, "include", "slotscan.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(slotscan_[a-z0-9_]+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    from slotscan_b200 import _lib
    L = _lib.lib()
    names = declared_functions()
    assert len(names) >= 10, names
    for n in names:
        assert hasattr(L, n), "libslotscan.so does not export %s" % n
    assert L.slotscan_abi_version() == 2


def test_argument_validation_needs_no_gpu():
    from slotscan_b200 import _lib
    L = _lib.lib()
    ok = _lib.Params(2, 16, 3, 12, 16, 16, 8, 0, 1, 1, 0, 0, 1e-4)
    assert L.slotscan_check(ctypes.byref(ok)) == 0
    for field, val in (("DK", 12), ("DV", 256), ("N", 0), ("G", 0), ("in_dtype", 7), ("N", 20000)):
        p = _lib.Params(2, 16, 3, 12, 16, 16, 8, 0, 1, 1, 0, 0, 1e-4)
        setattr(p, field, val)
        assert L.slotscan_check(ctypes.byref(p)) < 0, field
    # sizes whose launch grid or partial-sum table would overflow are refused before anything is launched
    for B, T, H in ((70000, 8, 1), (1, 32 * 65536, 1), (400000, 40000, 4)):
        p = _lib.Params(B, T, H, 12, 16, 16, 8, 0, 1, 1, 0, 0, 1e-4)
        assert L.slotscan_check(ctypes.byref(p)) in (0, -2)
    big = _lib.Params(1, 32 * 65536 + 1, 1, 12, 16, 16, 8, 0, 1, 1, 0, 0, 1e-4)
    assert L.slotscan_check(ctypes.byref(big)) == -2                   # token chunks ride on grid.y
    big = _lib.Params(400000, 40000, 4, 12, 16, 16, 8, 0, 1, 1, 0, 0, 1e-4)
    assert L.slotscan_check(ctypes.byref(big)) == -2                   # partial-sum table beyond int range
    assert L.slotscan_check(ctypes.byref(_lib.Params(70000, 8, 1, 12, 16, 16, 8, 0, 1, 1, 0, 0, 1e-4))) == 0   # B*H > 65535 is fine
    assert L.slotscan_check(None) == -1
    assert L.slotscan_hard_bwd_scratch_bytes(ctypes.byref(ok)) >= 4 * 2 * 3 * 16 * 12
    # NULL pointers are refused before any launch
    assert L.slotscan_hard_fwd(ctypes.byref(ok), None, None, None, None, None, None, None, None, None, None) == -1
    assert L.slotscan_hard_fwd_ex(ctypes.byref(ok), None, None, None, None, None, None, None, None, None, None, None) == -1


def test_python_host_mirrors_reference_signatures():
    import slotscan_b200 as S
    import slotkern_cuda, slotkern_kvg                                   # the drop-in module names
    want = ["k", "v", "gate", "fr", "N", "temp", "G", "hard", "hard_gate", "eps", "detach_addr", "q", "nw", "nwb", "occ_bin"]
    for fn in (S.kv_scan_g, S.kv_scan_c, slotkern_cuda.kv_scan_c, slotkern_kvg.kv_scan_g):
        ps = list(inspect.signature(fn).parameters)
        assert ps[:len(want)] == want, ps                               # gqa25/slotkern_kvg.py:257, slotkern_cuda.py:536
        d = {n: p.default for n, p in inspect.signature(fn).parameters.items()}
        assert d["G"] == 16 and d["hard"] is False and d["eps"] == 1e-4 and d["q"] is None and d["occ_bin"] is False
    ps = list(inspect.signature(S.scan_kv).parameters)                  # gqa25/slotkern_kv.py:29
    assert ps == ["k", "v", "gate", "fr", "N", "temp", "G", "hard", "hard_gate", "eps", "detach_addr", "q"]
    assert inspect.signature(S.scan_kv).parameters["G"].default == 1


def test_token_stream_dtype_policy():
    """bf16 kernels only when k, v and q are all bfloat16; any mix is cast to float32 (slotkern_cuda.py:488-489) --
    in kv_scan_g and in scan_with_log alike."""
    from slotscan_b200 import scan
    kb, vb = torch.zeros(1, 2, 1, 8, dtype=torch.bfloat16), torch.zeros(1, 2, 1, 8, dtype=torch.bfloat16)
    kf = kb.float()
    assert [t.dtype for t in scan._token_streams(kb, vb, kb)] == [torch.bfloat16] * 3
    assert scan._token_streams(kb, vb, None)[2] is None and scan._token_streams(kb, vb, None)[0].dtype == torch.bfloat16
    for k, v, q in ((kb, kf, kb), (kb, vb, kf), (kf, vb, None), (kb.half(), vb, kb)):
        out = scan._token_streams(k, v, q)
        assert all(t is None or t.dtype == torch.float32 for t in out), [None if t is None else t.dtype for t in out]
    src = inspect.getsource(scan.scan_with_log)
    assert "_token_streams" in src


def test_drop_in_kernel_attrs_signature():
    import slotkern_cuda
    ps = inspect.signature(slotkern_cuda.kernel_attrs).parameters           # gqa25/slotkern_cuda.py:467
    assert list(ps) == ["N", "D", "occb", "frt", "eps"]


def test_no_cpu_fallback():
    import slotscan_b200 as S
    k = torch.randn(1, 8, 2, 16)
    with pytest.raises(RuntimeError, match="CUDA"):
        S.kv_scan_g(k, k, torch.rand(1, 8, 2), 1.0, 4, 16.0, G=4, hard=True, detach_addr=True)


def test_product_does_not_import_the_oracle():
    """Nothing under the package may import, include, link or load the CPU oracle."""
    pkg = os.path.join(ROOT, "smal-memory-llm_b200")
    bad = re.compile(r"(import\s+oracle|from\s+oracle|liboracle|#include\s*[<\"][^>\"]*oracle|oracle/)")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")) or f == "Makefile":
                text = open(os.path.join(dirpath, f)).read()
                assert not bad.search(text), os.path.join(dirpath, f)


def test_custom_op_has_fake_kernel_for_compiled_callers():
    """The reference calls its scan from torch.compile'd blocks (gqa25/train_sh.py:783-793): the op must trace on
    meta tensors without a graph break."""
    from slotscan_b200 import ops
    k = torch.empty(2, 16, 3, 32, device="meta")
    g = torch.empty(2, 16, 3, device="meta")
    t1 = torch.empty(1, device="meta")
    out = torch.ops.slotscan.hard_fwd(k, k, k, g, g, t1, None, None, None, None, 24, 8, False, 1e-4, True, True, True, True)
    assert out[0].shape == (2, 2, 3, 24, 32) and out[0].dtype == torch.bfloat16 and out[2].dtype == torch.int32
    assert out[11].dtype == torch.float64 and out[12].shape == (2, 2, 3, 24) and out[13].dtype == torch.uint8
    gr = torch.ops.slotscan.hard_bwd(k, k, k, g, g, t1, *out[2:11], out[0], out[1], out[12], 24, 8, False, 1e-4, True, True)
    assert gr[0].shape == k.shape and gr[5].shape == (1,)
    # forward-only form: no undo log, no norms -> those outputs are empty
    out = torch.ops.slotscan.hard_fwd(k, None, k, g, g, t1, out[6], out[7], out[8], out[11], 24, 8, False, 1e-4, True,
                                      False, False, False)
    assert out[4].numel() == 0 and out[5].numel() == 0 and out[12].numel() == 0 and out[0].dtype == torch.float32


def test_epilogue_validation_and_host_names():
    """Writer epilogue / quantiser boundary: argument checks need no GPU; the host functions carry the reference's
    argument order (gqa25/memlm_sh.py:221, :231) and trace on meta tensors."""
    import slotscan_b200 as S
    from slotscan_b200 import _lib
    L = _lib.lib()
    ok = _lib.EpilogueParams(100, 128, 1, 1, 3, 16)
    assert L.slotscan_epilogue_check(ctypes.byref(ok)) == 0
    for field, val in (("D", 48), ("rows", -1), ("in_dtype", 5), ("bits", 5), ("group", 24), ("group", 2), ("group", 256)):
        p = _lib.EpilogueParams(100, 128, 1, 1, 3, 16)
        setattr(p, field, val)
        assert L.slotscan_epilogue_check(ctypes.byref(p)) < 0, field
    assert L.slotscan_epilogue_check(None) == -1
    assert L.slotscan_writer_epilogue(ctypes.byref(ok), None, None, None, None, None) == -1
    assert list(inspect.signature(S.fq).parameters) == ["x", "bits", "group"]
    assert list(inspect.signature(S.quantize_mem).parameters) == ["kbuf", "buf", "bits", "group"]
    with pytest.raises(RuntimeError, match="CUDA"):
        S.fq(torch.randn(4, 64), 3, 16)
    x = torch.empty(2, 5, 3, 7, 64, device="meta")
    assert torch.ops.slotscan.fq(x, 3, 16).shape == x.shape
    kq, kinv, valid = torch.ops.slotscan.epilogue(x, True, 3, 16)
    assert kq.dtype == torch.bfloat16 and kinv.shape == (2, 5, 3, 7) and valid.dtype == torch.uint8


def test_read_validation_and_fake_kernel():
    import slotscan_b200 as S
    from slotscan_b200 import _lib
    L = _lib.lib()
    ok = _lib.ReadParams(2, 40, 3, 2, 24, 128, 128, 8, 1, 1)
    assert L.slotscan_read_check(ctypes.byref(ok)) == 0
    for field, val in (("DK", 129), ("DV", 0), ("N", 0), ("N", 4096), ("G", 0), ("NQ", 0), ("q_dtype", 3)):
        p = _lib.ReadParams(2, 40, 3, 2, 24, 128, 128, 8, 1, 1)
        setattr(p, field, val)
        assert L.slotscan_read_check(ctypes.byref(p)) < 0, field
    assert L.slotscan_read_fwd(ctypes.byref(ok), None, None, None, None, None, None, None, None) == -1
    m = lambda *s, dt=torch.float32: torch.empty(*s, device="meta", dtype=dt)
    rd = torch.ops.slotscan.read_fwd(m(2, 40, 3, 2, 64), m(2, 40, 3, 2), m(2, 5, 3, 24, 64), m(2, 5, 3, 24, 32),
                                     m(2, 5, 3, 24), m(2, 5, 3, 24, dt=torch.uint8), 8)
    assert rd.shape == (2, 40, 3, 2, 32)
    with pytest.raises(RuntimeError, match="CUDA"):
        S.read_snapshots(torch.randn(1, 4, 1, 1, 8), torch.ones(1, 4, 1, 1), torch.randn(1, 1, 1, 2, 8),
                         torch.randn(1, 1, 1, 2, 8), torch.ones(1, 1, 1, 2), torch.ones(1, 1, 1, 2, dtype=torch.bool), 4)
