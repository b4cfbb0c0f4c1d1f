"""Drop-in for the reference module of the same name (gqa25/slotkern_v.py:232): memlm_kv.py imports slot_scan_v from here
(memlm_kv.py:27)."""
from slotscan_b200 import slot_scan_v  # noqa: F401
