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
    """The package's own helper (every ``SLinOSSMixer`` inside ``model`` -> the four B200 backends)."""
    import slinoss_b200 as sb

    return sb.use_b200_backends(model)


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
