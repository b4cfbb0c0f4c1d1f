"""Drop-in for the reference module of the same name (gqa25/slotkern_kvg.py:257): memlm_sh.py imports kv_scan_g
from here (memlm_sh.py:41-44) and tests monkey-patch it (kvu/gradcheck.py:49)."""
from slotscan_b200 import kv_scan_g  # noqa: F401
