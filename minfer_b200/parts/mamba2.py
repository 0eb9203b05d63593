"""A selective state-space mixer in the Mamba-2 form (scalar decay per head, state-space
duality), with per-sequence state instead of cached keys.

    [z | x | B | C | dt] = W_in u        inner = heads * head_dim; B, C: groups * n_state each
    (x | B | C) <- silu(conv(x | B | C) + b_conv)      causal, per channel, ``conv`` taps, the
                                                       last tap on the current token
    dt <- softplus(dt + dt_bias)                        (no clamp)
    per head h (group floor(h / (heads / groups))):
        S_t = exp(-exp(A_log_h) dt_t) S_{t-1} + dt_t B_t x_t^T       S: n_state x head_dim
        y_t = S_t^T C_t + D_h x_t
    y <- y * silu(z);  each of ``norm_groups`` equal parts of y divided by its root mean square
    (eps inside the root), times a weight;  out = W_o y

State per sequence (float32, zeroed when a slot is handed out): S of every head and the last
``conv`` - 1 inputs of the convolution.  A step may bring any number of tokens per sequence; the
recurrence walks them in order, so the result does not depend on how a sequence is cut.
Everything between the two products is float32 in both engines.  Tensor names behind ``prefix +
tensor_prefix``: ``in``, ``conv``, ``conv.b``, ``dt_bias``, ``A_log``, ``D``, ``norm``, ``o``.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..kernels import api as K
from ..weights.spec import MATRIX, VECTOR, Init, TensorSpec
from .base import CallBinding, Mixer, StateRequest, StepContext
from .linear import Linear
from .sink_attention import project_out

SSM_STATE = "ssm.state"
CONV_STATE = "ssm.conv"


class Mamba2(Mixer):
    capturable = True      # launches kernels only; safe inside a CUDA graph capture

    def libraries(self, dtype: torch.dtype) -> List[str]:
        return ["ops", "recurrent", "gemm_tc" if dtype == torch.bfloat16 else "gemm_simt"]

    def __init__(self, hidden_size: int, n_heads: int, head_dim: int, n_state: int, groups: int,
                 conv: int, norm_groups: int, norm_eps: float, tensor_prefix: str = "mix.",
                 init_std: float = 0.02):
        if min(n_heads, head_dim, n_state, groups, conv, norm_groups) < 1:
            raise ValueError("mamba2: every size must be at least 1")
        if n_heads % groups != 0:
            raise ValueError(f"mamba2: {n_heads} heads do not divide into {groups} groups")
        if (n_heads * head_dim) % norm_groups != 0:
            raise ValueError(f"mamba2: the inner width {n_heads * head_dim} does not divide into "
                             f"{norm_groups} norm groups")
        if conv > 8 or n_state > 256:
            raise ValueError("mamba2: the kernels take up to 8 taps and a state of up to 256")
        self.hidden_size = int(hidden_size)
        self.n_heads = int(n_heads)
        self.head_dim = int(head_dim)
        self.n_state = int(n_state)
        self.groups = int(groups)
        self.conv = int(conv)
        self.norm_groups = int(norm_groups)
        self.norm_eps = float(norm_eps)
        self.tensor_prefix = tensor_prefix
        self.init_std = float(init_std)
        self.inner = self.n_heads * self.head_dim
        self.channels = self.inner + 2 * self.groups * self.n_state
        self.in_width = 2 * self.inner + 2 * self.groups * self.n_state + self.n_heads
        self.in_proj: Optional[Linear] = None
        self.out: Optional[Linear] = None
        self.w: Dict[str, torch.Tensor] = {}

    # ---- weights ----------------------------------------------------------------------
    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        p = f"{prefix}{self.tensor_prefix}"
        init = Init(0.0, self.init_std)
        return [TensorSpec(f"{p}in", (self.in_width, self.hidden_size), MATRIX, init),
                # small per-channel and per-head tensors are held in float32 (role VECTOR)
                TensorSpec(f"{p}conv", (self.channels, self.conv), VECTOR, Init(0.0, 0.3)),
                TensorSpec(f"{p}conv.b", (self.channels,), VECTOR, Init(0.0, 0.1)),
                TensorSpec(f"{p}dt_bias", (self.n_heads,), VECTOR, Init(-1.0, 0.5)),
                TensorSpec(f"{p}A_log", (self.n_heads,), VECTOR, Init(0.0, 0.5)),
                TensorSpec(f"{p}D", (self.n_heads,), VECTOR, Init(1.0, 0.2)),
                TensorSpec(f"{p}norm", (self.inner,), VECTOR, Init(1.0, 0.0)),
                TensorSpec(f"{p}o", (self.hidden_size, self.inner), MATRIX, init)]

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        p = f"{prefix}{self.tensor_prefix}"
        self.in_proj = Linear(weights[f"{p}in"])
        self.out = Linear(weights[f"{p}o"])
        self.w = {n: weights[f"{p}{n}"] for n in ("conv", "conv.b", "dt_bias", "A_log", "D", "norm")}
        self.accepts_row_scale = self.in_proj.takes_row_scale()

    def export(self, prefix: str) -> Dict[str, torch.Tensor]:
        p = f"{prefix}{self.tensor_prefix}"
        out = {f"{p}in": self.in_proj.weight, f"{p}o": self.out.weight}
        out.update({f"{p}{n}": t for n, t in self.w.items()})
        return out

    # ---- what it keeps per sequence -----------------------------------------------------
    def state_request(self) -> Sequence[StateRequest]:
        return (StateRequest(SSM_STATE, (self.n_heads, self.head_dim, self.n_state), torch.float32),
                StateRequest(CONV_STATE, (self.channels, self.conv - 1), torch.float32))

    # ---- the step -----------------------------------------------------------------------
    def forward_add(self, x: torch.Tensor, ctx: StepContext, binding: CallBinding,
                    residual: torch.Tensor) -> None:
        n, dev = x.shape[0], x.device
        proj = self.in_proj.forward(x, torch.float32, row_scale=ctx.input_scale)
        u = torch.empty((n, self.channels), dtype=torch.float32, device=dev)
        K.conv_silu(proj, self.inner, self.channels, self.w["conv"], self.w["conv.b"],
                    binding.state[CONV_STATE], ctx.token_row, ctx.cu_seqlens, ctx.slots, u,
                    ctx.n_rows, single=ctx.single_token)
        y = torch.empty((n, self.inner), dtype=torch.float32, device=dev)
        K.ssm_scan(u, proj, self.inner + self.channels, self.w["dt_bias"], self.w["A_log"],
                   self.w["D"], binding.state[SSM_STATE], ctx.cu_seqlens, ctx.slots, y, ctx.n_rows,
                   self.n_heads, self.head_dim, self.n_state, self.groups)
        gated = torch.empty((n, self.inner), dtype=ctx.act_dtype, device=dev)
        K.gated_group_norm(y, proj, 0, self.w["norm"], gated, self.norm_groups, self.norm_eps)
        project_out(self.out, gated, ctx, residual)
