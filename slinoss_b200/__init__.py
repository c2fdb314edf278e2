"""B200-native (sm_100a) backend of the SLinOSS v2x2ssd scan path.

Hand-written CUDA kernels behind a C ABI (``include/slinoss_b200.h``), called
from thin torch host code.  Importing this package does not need a GPU; calling
an op does, and needs the built library (``python -m slinoss_b200.build``).
"""

from ._lib import read_scan_status, read_tc_status, set_tensor_path
from .backends import (B200CConv1dBackend, B200MixerDecodeBackend, B200ScanBackend,
                       B200ScanPrepBackend, use_b200_backends)
from .ops import (cconv1d_b200, cconv1d_update_b200, gate_skip_b200, chunk_increment_b200, chunk_scan_b200, mixer_decode_step_b200,
                  scanprep_b200, state_passing_b200, v2x2ssd_b200)
from .types import ScanInputs, ScanPrepInputs, ScanState

__all__ = [
    "v2x2ssd_b200", "chunk_increment_b200", "state_passing_b200", "chunk_scan_b200",
    "scanprep_b200", "cconv1d_b200", "cconv1d_update_b200", "gate_skip_b200", "B200ScanBackend", "B200ScanPrepBackend",
    "B200CConv1dBackend", "B200MixerDecodeBackend", "use_b200_backends", "mixer_decode_step_b200", "ScanInputs", "ScanPrepInputs", "ScanState", "set_tensor_path",
    "read_tc_status", "read_scan_status",
]
