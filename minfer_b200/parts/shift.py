"""Token shift: what a mixer reads is mixed with what it read at the position before,
    u_p = n_p + (n_{p-1} - n_p) * s        (n_{-1} = 0),
element by element with a learned vector ``s``; ``n`` is the block's normed input before the
shift.  The last ``n`` of a sequence is kept as its state (float32 [width]) so that a step may
go on from anywhere.  The norm and the shift are one kernel (``kernels.api.norm_shift``).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..kernels import api as K
from ..weights.spec import VECTOR, Init, TensorSpec
from .base import Part, StateRequest, StepContext

STATE_NAME = "shift.previous"


class TokenShift(Part):
    capturable = True      # launches kernels only; safe inside a CUDA graph capture

    def libraries(self, dtype: torch.dtype) -> List[str]:
        return ["ops"]

    def __init__(self, size: int, tensor_name: str = "shift", init_std: float = 0.3):
        self.size = int(size)
        self.tensor_name = tensor_name
        self.init_std = float(init_std)
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        return [TensorSpec(f"{prefix}{self.tensor_name}", (self.size,), VECTOR,
                           Init(0.5, self.init_std))]

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        self.weight = weights[f"{prefix}{self.tensor_name}"]

    def export(self, prefix: str) -> Dict[str, torch.Tensor]:
        return {f"{prefix}{self.tensor_name}": self.weight}

    def state_request(self) -> Sequence[StateRequest]:
        return (StateRequest(STATE_NAME, (self.size,), torch.float32),)

    def norm_and_shift(self, norm, h: torch.Tensor, ctx: StepContext,
                       state: Dict[str, torch.Tensor]) -> torch.Tensor:
        """``norm`` must be y = x / rms * w (``Norm.foldable``).  A projection output that is
        still pending (its K splits) is added into ``h`` here: by this kernel where every row
        brings one token, else by the reduction kernel first."""
        fold = norm.foldable()
        if fold is None:
            raise K.KernelError("the token shift is fused with an RMS norm; this norm is another")
        weight, eps, size = fold
        out = torch.empty((h.shape[0], self.size), dtype=ctx.act_dtype, device=h.device)
        pending = ctx.extras.pop("pending", None)
        partial = bias = None
        if pending is not None:
            if ctx.single_token and pending.partial.dim() == 3:
                partial, bias = pending.partial, pending.bias
            else:
                pending.settle(h)
        K.norm_shift(h, weight, self.weight, eps, ctx.positions, ctx.token_row, ctx.cu_seqlens,
                     ctx.slots, state[STATE_NAME], out, multi=not ctx.single_token,
                     partial=partial, bias=bias)
        return out
