"""slotscan_b200: the slot-scan hot path of smal-memory-llm as hand-written sm_100a CUDA behind the reference's own
Python call signature.  Importing this package loads nothing; the first op call loads libslotscan.so and fails
loudly if it is not built."""
from .scan import StreamingScan, kv_scan_c, kv_scan_g, scan_kv, scan_with_log, write_memory  # noqa: F401
from ._lib import kernel_attrs  # noqa: F401
from .epilogue import E4M3, fq, quantize_mem, writer_epilogue  # noqa: F401
from .read import read_snapshots  # noqa: F401
from .keyless import slot_scan_v  # noqa: F401
