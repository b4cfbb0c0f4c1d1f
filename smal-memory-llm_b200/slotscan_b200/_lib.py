"""Loader of libslotscan.so, the C-ABI CUDA library (include/slotscan.h).  There is no fallback of any kind:
if the library is missing or an entry point rejects a call, the caller gets an exception."""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libslotscan.so")

F32, BF16 = 0, 1
ABI_VERSION = 2

ERRORS = {-1: "a required pointer is NULL", -2: "unsupported shape", -3: "unknown dtype code",
          -4: "a pointer is not 16-byte aligned", -5: "mode not implemented by this entry point",
          -6: "beyond the fixed capacity of the no-allocation entry point"}


class Params(ctypes.Structure):
    """slotscan_params of include/slotscan.h."""
    _fields_ = [(n, ctypes.c_int32) for n in ("B", "T", "H", "N", "DK", "DV", "G", "hard_gate", "occ_bin",
                                              "fr_per_token", "in_dtype", "snap_dtype")] + [("eps", ctypes.c_float)]


class Log(ctypes.Structure):
    """slotscan_log of include/slotscan.h."""
    _fields_ = [(n, ctypes.c_void_p) for n in ("addr", "oold", "kold", "vold", "kfin", "vfin", "ofin", "tfirst", "kiold")]


class DenseParams(ctypes.Structure):
    """slotscan_dense_params of include/slotscan.h."""
    _fields_ = [("base", Params), ("hard", ctypes.c_int32), ("detach_addr", ctypes.c_int32)]


class KeylessParams(ctypes.Structure):
    """slotscan_v_params of include/slotscan.h."""
    _fields_ = [(n, ctypes.c_int32) for n in ("B", "T", "H", "N", "DV", "G", "hard", "hard_gate", "in_dtype")]


class FwdExtra(ctypes.Structure):
    """slotscan_fwd_extra of include/slotscan.h."""
    _fields_ = [(n, ctypes.c_void_p) for n in ("K0", "V0", "o0", "nsq0", "nsqfin", "kinv", "valid")] + \
               [("no_undo_log", ctypes.c_int32)]


class EpilogueParams(ctypes.Structure):
    """slotscan_epilogue_params of include/slotscan.h."""
    _fields_ = [("rows", ctypes.c_int64), ("D", ctypes.c_int32), ("in_dtype", ctypes.c_int32),
                ("out_dtype", ctypes.c_int32), ("bits", ctypes.c_int32), ("group", ctypes.c_int32)]


class ReadParams(ctypes.Structure):
    """slotscan_read_params of include/slotscan.h."""
    _fields_ = [(n, ctypes.c_int32) for n in ("B", "T", "H", "NQ", "N", "DK", "DV", "G", "q_dtype", "snap_dtype")]


class KernelAttr(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char * 48), ("regs", ctypes.c_int32), ("local_bytes", ctypes.c_int32),
                ("static_smem", ctypes.c_int32), ("max_threads", ctypes.c_int32)]


class KernelTime(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char * 48), ("launches", ctypes.c_int32), ("total_ms", ctypes.c_float)]


_lib = None


def lib():
    """The loaded library.  Raises if it has not been built (run `make` in smal-memory-llm_b200/ or
    __graft_entry__.build())."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError("libslotscan.so is not built (%s): the slot scan has no other implementation; "
                               "build it with `make -C smal-memory-llm_b200`" % LIB_PATH)
        L = ctypes.CDLL(LIB_PATH)
        vp, ci, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
        PP, LP = ctypes.POINTER(Params), ctypes.POINTER(Log)
        L.slotscan_abi_version.restype = ci
        L.slotscan_check.argtypes = [PP]
        L.slotscan_hard_fwd.argtypes = [PP, vp, vp, vp, vp, vp, vp, vp, vp, LP, vp]
        L.slotscan_hard_fwd_ex.argtypes = [PP, vp, vp, vp, vp, vp, vp, vp, vp, LP, ctypes.POINTER(FwdExtra), vp]
        L.slotscan_hard_fwd_ex.restype = ci
        L.slotscan_hard_bwd_ex.argtypes = [PP, vp, vp, vp, vp, vp, vp, LP, vp, vp, vp, vp, sz, vp, vp, vp, vp, vp, vp, vp]
        L.slotscan_hard_bwd_ex.restype = ci
        DP = ctypes.POINTER(DenseParams)
        L.slotscan_dense_check.argtypes = [DP]
        L.slotscan_dense_check.restype = ci
        L.slotscan_dense_fwd.argtypes = [DP] + [vp] * 14
        L.slotscan_dense_fwd.restype = ci
        L.slotscan_dense_bwd_scratch_bytes.argtypes = [DP]
        L.slotscan_dense_bwd_scratch_bytes.restype = sz
        L.slotscan_dense_bwd.argtypes = [DP] + [vp] * 12 + [sz] + [vp] * 7
        L.slotscan_dense_bwd.restype = ci
        KP = ctypes.POINTER(KeylessParams)
        L.slotscan_v_check.argtypes = [KP]
        L.slotscan_v_check.restype = ci
        L.slotscan_v_fwd.argtypes = [KP] + [vp] * 8
        L.slotscan_v_fwd.restype = ci
        L.slotscan_v_bwd_scratch_bytes.argtypes = [KP]
        L.slotscan_v_bwd_scratch_bytes.restype = sz
        L.slotscan_v_bwd.argtypes = [KP] + [vp] * 8 + [sz] + [vp] * 5
        L.slotscan_v_bwd.restype = ci
        L.slotscan_hard_bwd_scratch_bytes.argtypes = [PP]
        L.slotscan_hard_bwd_scratch_bytes.restype = sz
        L.slotscan_hard_bwd.argtypes = [PP, vp, vp, vp, vp, vp, vp, LP, vp, vp, vp, sz, vp, vp, vp, vp, vp, vp, vp]
        L.slotscan_hard_bwd_noalloc.argtypes = [PP, vp, vp, vp, vp, vp, vp, LP, vp, vp, vp, vp, vp, vp, vp, vp, vp]
        L.slotscan_hard_bwd_noalloc.restype = ci
        L.slotscan_hard_bwd_noalloc_capacity.restype = sz
        L.slotscan_epilogue_check.argtypes = [ctypes.POINTER(EpilogueParams)]
        L.slotscan_epilogue_check.restype = ci
        L.slotscan_writer_epilogue.argtypes = [ctypes.POINTER(EpilogueParams), vp, vp, vp, vp, vp]
        L.slotscan_writer_epilogue.restype = ci
        L.slotscan_read_check.argtypes = [ctypes.POINTER(ReadParams)]
        L.slotscan_read_check.restype = ci
        L.slotscan_read_fwd.argtypes = [ctypes.POINTER(ReadParams), vp, vp, vp, vp, vp, vp, vp, vp]
        L.slotscan_read_fwd.restype = ci
        L.slotscan_read_bwd.argtypes = [ctypes.POINTER(ReadParams)] + [vp] * 13
        L.slotscan_read_bwd.restype = ci
        L.slotscan_device_status.restype = ci
        L.slotscan_query_attrs.argtypes = [ctypes.POINTER(KernelAttr), ci]
        L.slotscan_profile_enable.argtypes = [ci]
        L.slotscan_profile_read.argtypes = [ctypes.POINTER(KernelTime), ci]
        for f in ("slotscan_profile_enable", "slotscan_profile_read", "slotscan_check", "slotscan_hard_fwd", "slotscan_hard_bwd", "slotscan_query_attrs"):
            getattr(L, f).restype = ci
        assert L.slotscan_abi_version() == ABI_VERSION, "libslotscan.so / Python host ABI mismatch"
        _lib = L
    return _lib


def check(rc, what):
    if rc == 0:
        return
    if rc < 0:
        raise ValueError("%s rejected the call: %s (code %d)" % (what, ERRORS.get(rc, "?"), rc))
    raise RuntimeError("%s: CUDA error %d" % (what, rc))


def kernel_attrs():
    """{kernel name: (registers, spilled bytes, static shared memory, max threads)} -- the analogue of the
    reference's kernel_attrs (gqa25/slotkern_cuda.py:467-479).  Needs a CUDA device."""
    buf = (KernelAttr * 32)()
    n = lib().slotscan_query_attrs(buf, 32)
    return {buf[i].name.decode(): (buf[i].regs, buf[i].local_bytes, buf[i].static_smem, buf[i].max_threads)
            for i in range(min(n, 32))}


def device_status():
    """Synchronises the device; 1 if a kernel gave up on a bounded wait since the last call (its results are then
    incomplete), else 0."""
    return lib().slotscan_device_status()


def profile_enable(on=True):
    """Bracket every kernel launch of the library with CUDA events (on the launching stream) until switched off."""
    lib().slotscan_profile_enable(int(bool(on)))


def profile_read():
    """{kernel: (launches, total device ms)} since the last read; waits for the recorded events."""
    buf = (KernelTime * 16)()
    n = lib().slotscan_profile_read(buf, 16)
    return {buf[i].name.decode(): (buf[i].launches, buf[i].total_ms) for i in range(min(n, 16))}
