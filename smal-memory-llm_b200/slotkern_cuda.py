"""Drop-in for the reference module of the same name (gqa25/slotkern_cuda.py): put this directory ahead of the
reference's on sys.path and `KV_CUDA=1` makes memlm_sh.py bind this kv_scan_c as its kv_scan_g (memlm_sh.py:48-50)."""
from slotscan_b200 import kv_scan_c  # noqa: F401
from slotscan_b200 import kernel_attrs as _kernel_attrs


def kernel_attrs(N=None, D=None, occb=True, frt=True, eps=1e-4):
    """Signature of the reference's kernel_attrs(N, D, occb, frt, eps) (slotkern_cuda.py:467-479), which compiles for
    that shape and returns {addr_fwd, val_fwd, rows_bwd, addr_bwd: (registers, local bytes)}.  The kernels here are
    compiled ahead of time for every shape, so the arguments only pick the D = 128 entries that correspond to the
    reference's four kernels; the full table (every instantiation, with shared memory and thread limits) is
    slotscan_b200.kernel_attrs()."""
    full = _kernel_attrs()
    pick = {"addr_fwd": "addr_fwd<128,rows<=64>", "val_fwd": "replay_rows<128,f32,f32>",
            "rows_bwd": "rows_bwd<128,f32,f32>", "addr_bwd": "addr_bwd_gather<128>"}
    return {ref: tuple(full[mine][:2]) for ref, mine in pick.items() if mine in full}

