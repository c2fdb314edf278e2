"""Operators of the B200 scan backend (all backed by the C-ABI library)."""

from .cconv1d import cconv1d_b200, cconv1d_update_b200
from .decode import mixer_decode_step_b200
from .glue import gate_skip_b200
from .scanprep import scanprep_b200
from .v2x2ssd import chunk_increment_b200, chunk_scan_b200, state_passing_b200, v2x2ssd_b200

__all__ = ["v2x2ssd_b200", "chunk_increment_b200", "state_passing_b200", "chunk_scan_b200",
           "scanprep_b200", "cconv1d_b200", "cconv1d_update_b200", "mixer_decode_step_b200", "gate_skip_b200"]
