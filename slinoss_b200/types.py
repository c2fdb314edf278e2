"""Value types of the backend boundary.

These mirror the reference's frozen dataclasses field for field
(slinoss/layers/backend.py:16-46 ``ScanPrepInputs`` / ``ScanInputs`` and
slinoss/layers/state.py:36 ``ScanState``) so that the backends in
``slinoss_b200.backends`` accept the reference's own objects (duck typing) and
return objects the reference's ``SLinOSSMixer`` can consume.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass(frozen=True)
class ScanPrepInputs:
    """``value (b,T,H*P)``, ``params (b,T,H*13)``, ``bc (b,T,H,4,N)``."""

    value: torch.Tensor
    params: torch.Tensor
    bc: torch.Tensor


@dataclass(frozen=True)
class ScanInputs:
    """``U (b,H,T,P)``, ``M (b,H,T,2)``, ``K (b,H,T,2,2)``, ``B, C (b,H,T,2N)``."""

    U: torch.Tensor
    M: torch.Tensor
    K: torch.Tensor
    B: torch.Tensor
    C: torch.Tensor


@dataclass
class ScanState:
    """Streaming state: ``state (b,H,P,2N)``, ``b_prev (b,H,2N)``, ``u_prev (b,H,P)``."""

    state: Optional[torch.Tensor] = None
    b_prev: Optional[torch.Tensor] = None
    u_prev: Optional[torch.Tensor] = None

    def detach(self) -> "ScanState":
        return ScanState(*(None if t is None else t.detach()
                           for t in (self.state, self.b_prev, self.u_prev)))

    def clone(self) -> "ScanState":
        return ScanState(*(None if t is None else t.clone()
                           for t in (self.state, self.b_prev, self.u_prev)))
