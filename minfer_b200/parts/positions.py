"""Learned position vectors: a table row per absolute position, added (unscaled) to the
residual stream right after the embedding."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import api as K
from ..weights.spec import MATRIX, Init, TensorSpec
from .base import ModelPart, StepContext


class LearnedPositions(ModelPart):
    capturable = True      # launches kernels only; safe inside a CUDA graph capture

    def libraries(self, dtype: torch.dtype) -> List[str]:
        return ["ops"]

    def __init__(self, width: int, positions: int, tensor_name: str = "pos",
                 init_std: float = 0.02):
        self.width = int(width)
        self.positions = int(positions)
        self.tensor_name = tensor_name
        self.init_std = float(init_std)
        self.table: Optional[torch.Tensor] = None

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        return [TensorSpec(f"{prefix}{self.tensor_name}", (self.positions, self.width), MATRIX,
                           Init(0.0, self.init_std))]

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        self.table = weights[f"{prefix}{self.tensor_name}"]

    def export(self, prefix: str) -> Dict[str, torch.Tensor]:
        return {f"{prefix}{self.tensor_name}": self.table}

    def forward_inplace(self, h: torch.Tensor, ctx: StepContext) -> None:
        K.add_rows(h, self.table, ctx.positions, ctx.status)

    def embedding_rows(self, ctx: StepContext):
        return self.table, ctx.positions
