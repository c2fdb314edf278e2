"""Access to the unmodified reference package for the drop-in tests.

The reference (``slinoss``) is a Python package; it is installed once, outside version
control, into ``baseline/_ref`` at the repository root (``pip install --no-deps --target
baseline/_ref <reference checkout>``; ``__graft_entry__.build()`` does it when the
checkout is present).  Tests that need it call ``import_reference()`` and are skipped when
the folder is absent.
"""

from __future__ import annotations

import sys
from pathlib import Path

import pytest

REF_DIR = Path(__file__).resolve().parents[1] / "baseline" / "_ref"


def import_reference():
    """Import ``slinoss`` from ``baseline/_ref`` (skip the calling test when it is not installed)."""
    if not (REF_DIR / "slinoss" / "__init__.py").exists():
        pytest.skip(f"reference package not installed under {REF_DIR}")
    if str(REF_DIR) not in sys.path:
        sys.path.insert(0, str(REF_DIR))
    import slinoss  # noqa: F401

    return slinoss


def use_b200_backends(model) -> int:
    """Point every ``SLinOSSMixer`` inside ``model`` at the four B200 backends, the way the
    reference's own workload builder swaps backends (scripts/perf/_nextchar.py:101-127).
    Returns the number of mixers switched."""
    from slinoss.layers import SLinOSSMixer
    from slinoss.layers.backend import ScanInputs
    from slinoss.layers.state import ScanState

    import slinoss_b200 as sb

    scan = sb.B200ScanBackend(state_cls=ScanState)
    prep = sb.B200ScanPrepBackend(inputs_cls=ScanInputs)
    conv = sb.B200CConv1dBackend()
    dec = sb.B200MixerDecodeBackend(state_cls=ScanState)
    n = 0
    for module in model.modules():
        if isinstance(module, SLinOSSMixer):
            module.backend = scan
            module.scanprep.backend = prep
            module.cconv_backend = conv
            module.decode_backend = dec
            n += 1
    return n


def use_reference_backends(model) -> int:
    from slinoss.layers import SLinOSSMixer
    from slinoss.layers.backend import (ReferenceCConv1dBackend, ReferenceMixerDecodeBackend,
                                        ReferenceScanBackend, ReferenceScanPrepBackend)

    n = 0
    for module in model.modules():
        if isinstance(module, SLinOSSMixer):
            module.backend = ReferenceScanBackend(compute_dtype=None)
            module.scanprep.backend = ReferenceScanPrepBackend()
            module.cconv_backend = ReferenceCConv1dBackend()
            module.decode_backend = ReferenceMixerDecodeBackend()
            n += 1
    return n
