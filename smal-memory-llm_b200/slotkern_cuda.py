"""Drop-in for the reference module of the same name (gqa25/slotkern_cuda.py): put this directory ahead of the
reference's on sys.path and `KV_CUDA=1` makes memlm_sh.py bind this kv_scan_c as its kv_scan_g (memlm_sh.py:48-50)."""
from slotscan_b200 import kernel_attrs, kv_scan_c  # noqa: F401
