"""Parts of role "model" that work on the residual stream or the logits around the blocks:

``EmbeddingNorm``    an RMS norm of the embedding rows as they enter the residual stream
``LogitSoftcap``     logits <- cap * tanh(logits / cap)
``PassInjection``    what a pass of a layer loop adds to the residual stream right before its first
                     layer: the embedding output (every pass but the first) and a learned vector
                     per pass, the rows of a table [passes, width]
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import api as K
from ..weights.spec import MATRIX, VECTOR, Init, TensorSpec
from .base import ModelPart, StepContext


class EmbeddingNorm(ModelPart):
    capturable = True      # launches kernels only; safe inside a CUDA graph capture

    def libraries(self, dtype: torch.dtype) -> List[str]:
        return ["ops"]

    def __init__(self, width: int, eps: float, tensor_name: str = "embed.norm"):
        self.width = int(width)
        self.eps = float(eps)
        self.tensor_name = tensor_name
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        return [TensorSpec(f"{prefix}{self.tensor_name}", (self.width,), VECTOR, Init(1.0, 0.0))]

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        self.weight = weights[f"{prefix}{self.tensor_name}"]

    def export(self, prefix: str) -> Dict[str, torch.Tensor]:
        return {f"{prefix}{self.tensor_name}": self.weight}

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        out = torch.empty_like(x)
        K.rmsnorm(x, self.weight, self.eps, out)
        return out

    def forward_inplace(self, x: torch.Tensor, ctx: StepContext) -> None:
        x.copy_(self.forward(x, ctx))


class LogitSoftcap(ModelPart):
    capturable = True      # launches kernels only; safe inside a CUDA graph capture

    def libraries(self, dtype: torch.dtype) -> List[str]:
        return ["ops"]

    def __init__(self, cap: float):
        if not cap > 0.0:
            raise ValueError(f"a soft cap must be positive, got {cap}")
        self.cap = float(cap)

    def forward_inplace(self, x: torch.Tensor, ctx: StepContext) -> None:
        K.tanh_cap(x, self.cap)


class PassInjection(ModelPart):
    """``add(h, ctx, pass_index, embedding_output)``: h += embedding_output (pass_index > 0, if
    ``add_embedding``) + table[pass_index]."""

    capturable = True      # launches kernels only; safe inside a CUDA graph capture

    def libraries(self, dtype: torch.dtype) -> List[str]:
        return ["ops"]

    def __init__(self, width: int, passes: int, tensor_name: str = "loop.step",
                 add_embedding: bool = True, init_std: float = 0.02):
        self.width = int(width)
        self.passes = int(passes)
        self.tensor_name = tensor_name
        self.add_embedding = bool(add_embedding)
        self.init_std = float(init_std)
        self.table: Optional[torch.Tensor] = None

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        return [TensorSpec(f"{prefix}{self.tensor_name}", (self.passes, self.width), MATRIX,
                           Init(0.0, self.init_std))]

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        self.table = weights[f"{prefix}{self.tensor_name}"]

    def export(self, prefix: str) -> Dict[str, torch.Tensor]:
        return {f"{prefix}{self.tensor_name}": self.table}

    def needs_embedding(self) -> bool:
        return self.add_embedding and self.passes > 1

    def add(self, h: torch.Tensor, ctx: StepContext, pass_index: int,
            embedding_output: Optional[torch.Tensor]) -> None:
        if not 0 <= pass_index < self.passes:
            raise K.KernelError(f"pass {pass_index} is outside the table of {self.passes} passes")
        other = embedding_output if (self.add_embedding and pass_index > 0) else None
        K.add_stream(h, other, self.table[pass_index])
