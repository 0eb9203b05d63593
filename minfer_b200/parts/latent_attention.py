"""Latent attention as a mixer: keys and values of all heads are products of one small latent
vector per position, which is all the cache keeps.

    q = Wq u, per head [q_p : head_dim | q_r : rot_dim]
    [c' | k_r] = Wdkv u;  c = c' / sqrt(mean(c'^2) + eps) * wc        (latent of ``kv_rank``)
    per head h: k_h = [Wuk_h c | k_r], v_h = Wuv_h c;  q_r and k_r rotated (``position``)
    s_ij = (q_i . k_j) * scale, visible iff 0 <= i - j < window        (``window`` > 0: else causal)
    w_ij = exp(s_ij) / (exp(sink_h) + sum_j' exp(s_ij'))               (``sink``: learned per head)
    out = Wo (concat_h(sum_j w_ij v_j) * sigmoid(Wg u))                (``gate``)

Computed in the absorbed form, which never expands the latent into per-head keys and values:
    q'_h = [Wuk_h^T q_p | q_r]   (kv_rank + rot_dim wide),   key_j = [c_j | k_r_j] shared by all
    heads,   value_j = c_j,   o_h = Wuv_h (sum_j w_ij c_j)
since q_p . (Wuk_h c) = (Wuk_h^T q_p) . c.  The attention is therefore one over a single
key/value head of width kv_rank + rot_dim (``parts.sink_attention.scored_attention``), between
two per-head products (``kernels.api.head_linear``; the second applies the gate).  The value IS
the key: the attention kernels get the same tensor [c | k_r] for both, and the second product
reads the first kv_rank columns of the weighted sum (the rot_dim columns behind them are
computed and ignored: a third more work in P V, for keys and values of one size, which is what
the tensor-memory kernel takes, and for a cache that holds each position's vector once).  With a
window the cache entry is a ring.

One packed product gives q | c' | k_r | gate in float32.  Tensor names behind ``prefix +
tensor_prefix``: ``q``, ``dkv``, ``dkv.norm``, ``uk``, ``uv``, ``sink``, ``g``, ``o``.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.base import PartSpec
from ..kernels import api as K
from ..weights.spec import MATRIX, VECTOR, Init, TensorSpec
from .base import CacheRequest, CallBinding, Mixer, StepContext
from .linear import Linear
from .sink_attention import ScoreSpec, project_out, scored_attention


class LatentAttention(Mixer):
    capturable = True      # launches kernels only; safe inside a CUDA graph capture

    def libraries(self, dtype: torch.dtype) -> List[str]:
        libs = ["ops", "mixer_prep", "attention_sink"]
        libs.append("gemm_tc" if dtype == torch.bfloat16 else "gemm_simt")
        kw = self.kv_rank + self.rot_dim
        if K.sink_attention_tc_supported(dtype, kw, kw):
            libs.append("attention_prefill_tc")
        return libs

    def __init__(self, hidden_size: int, n_heads: int, head_dim: int, rot_dim: int, value_dim: int,
                 kv_rank: int, scale: float, norm_eps: float, window: int = 0, sink: bool = True,
                 gate: bool = True, position: Optional[PartSpec] = None,
                 tensor_prefix: str = "mix.", init_std: float = 0.02):
        from ..registry import build_part
        if min(n_heads, head_dim, value_dim, kv_rank) < 1 or rot_dim < 0 or window < 0:
            raise ValueError("latent attention: sizes must be positive (rot_dim and window may be 0)")
        if kv_rank + rot_dim > 640:
            raise ValueError(f"latent attention: kv_rank + rot_dim = {kv_rank + rot_dim} is not "
                             f"supported: the attention kernels take keys up to 640 wide")
        self.hidden_size = int(hidden_size)
        self.n_heads = int(n_heads)
        self.head_dim = int(head_dim)
        self.rot_dim = int(rot_dim)
        self.value_dim = int(value_dim)
        self.kv_rank = int(kv_rank)
        self.scale = float(scale)
        self.norm_eps = float(norm_eps)
        self.window = int(window)
        self.sink = bool(sink)
        self.gate = bool(gate)
        self.tensor_prefix = tensor_prefix
        self.init_std = float(init_std)
        self.position = build_part("position", position) if position is not None else None
        if self.position is not None and getattr(self.position, "rotary_dim", 0) > self.rot_dim:
            raise ValueError("latent attention: the rotation is wider than the rotated part")
        self.proj: Optional[Linear] = None
        self.out: Optional[Linear] = None
        self.c_norm: Optional[torch.Tensor] = None
        self.sink_logit: Optional[torch.Tensor] = None
        self.uk_t: Optional[torch.Tensor] = None      # [heads, kv_rank, head_dim]: Wuk_h transposed
        self.uv: Optional[torch.Tensor] = None        # [heads, value_dim, kv_rank]
        self._uk: Optional[torch.Tensor] = None       # as the checkpoint holds them
        self._uv: Optional[torch.Tensor] = None

    def _widths(self):
        """Columns of the packed projection: q, latent, rotated key, gate."""
        return (self.n_heads * (self.head_dim + self.rot_dim), self.kv_rank, self.rot_dim,
                self.n_heads * self.value_dim if self.gate else 0)

    # ---- weights ----------------------------------------------------------------------
    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        p = f"{prefix}{self.tensor_prefix}"
        nq, rank, rd, ng = self._widths()
        init = Init(0.0, self.init_std)
        specs = [TensorSpec(f"{p}q", (nq, self.hidden_size), MATRIX, init),
                 TensorSpec(f"{p}dkv", (rank + rd, self.hidden_size), MATRIX, init),
                 TensorSpec(f"{p}dkv.norm", (rank,), VECTOR, Init(1.0, 0.0)),
                 TensorSpec(f"{p}uk", (self.n_heads * self.head_dim, rank), MATRIX, init),
                 TensorSpec(f"{p}uv", (self.n_heads * self.value_dim, rank), MATRIX, init),
                 TensorSpec(f"{p}o", (self.hidden_size, self.n_heads * self.value_dim), MATRIX, init)]
        if self.sink:
            specs.append(TensorSpec(f"{p}sink", (self.n_heads,), VECTOR, Init(0.0, 0.5)))
        if self.gate:
            specs.append(TensorSpec(f"{p}g", (ng, self.hidden_size), MATRIX, init))
        return specs

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        p = f"{prefix}{self.tensor_prefix}"
        parts = [weights[f"{p}q"], weights[f"{p}dkv"]] + ([weights[f"{p}g"]] if self.gate else [])
        if len({t.dtype for t in parts}) != 1:
            parts = [t.to(torch.float32) for t in parts]
        self.proj = Linear(torch.cat(parts, dim=0).contiguous())
        self.out = Linear(weights[f"{p}o"])
        self.c_norm = weights[f"{p}dkv.norm"]
        self.sink_logit = weights[f"{p}sink"] if self.sink else None
        self._uk = weights[f"{p}uk"]
        self.uk_t = self._uk.view(self.n_heads, self.head_dim, self.kv_rank).transpose(1, 2).contiguous()
        self._uv = weights[f"{p}uv"]
        self.uv = self._uv.view(self.n_heads, self.value_dim, self.kv_rank)
        self.accepts_row_scale = self.proj.takes_row_scale()

    def export(self, prefix: str) -> Dict[str, torch.Tensor]:
        p = f"{prefix}{self.tensor_prefix}"
        nq, rank, rd, ng = self._widths()
        w = self.proj.weight
        out = {f"{p}q": w[:nq], f"{p}dkv": w[nq:nq + rank + rd], f"{p}dkv.norm": self.c_norm,
               f"{p}uk": self._uk, f"{p}uv": self._uv,
               f"{p}o": self.out.weight}
        if self.sink:
            out[f"{p}sink"] = self.sink_logit
        if self.gate:
            out[f"{p}g"] = w[nq + rank + rd:]
        return out

    # ---- what it keeps per sequence -----------------------------------------------------
    def cache_request(self) -> Optional[CacheRequest]:
        return CacheRequest(1, self.kv_rank + self.rot_dim, self.window, shared_values=True)

    def scores(self) -> ScoreSpec:
        kw = self.kv_rank + self.rot_dim
        return ScoreSpec(n_heads=self.n_heads, n_kv_heads=1, head_dim=kw, value_dim=kw,
                         scale=self.scale, window=self.window, sink=self.sink,
                         sink_logit=self.sink_logit)

    # ---- the step -----------------------------------------------------------------------
    def forward_add(self, x: torch.Tensor, ctx: StepContext, binding: CallBinding,
                    residual: torch.Tensor) -> None:
        n = x.shape[0]
        nh, hd, rd, vd, rank = self.n_heads, self.head_dim, self.rot_dim, self.value_dim, self.kv_rank
        nq, _, _, _ = self._widths()
        dev, act = x.device, ctx.act_dtype
        cache = binding.cache
        if cache is None:
            raise K.KernelError("the attention mixer was given no cache entry")
        if cache.k.dtype != act:
            raise K.KernelError("the cache and the activations must share one dtype")
        proj = self.proj.forward(x, torch.float32, row_scale=ctx.input_scale)
        inv_freq, rot_dims, style, magnitude = None, 0, 0, 1.0
        if self.position is not None and getattr(self.position, "rotary_dim", 0) > 0:
            inv_freq, rot_dims, style = self.position.tables(dev)
            magnitude = self.position.magnitude()
        kw = rank + rd
        q = torch.empty((n, nh * (hd + rd)), dtype=act, device=dev)
        write = binding.writes_cache
        own_kv = ctx.from_start
        k_step = None
        if own_kv and write:
            k_step = torch.empty((n, 1, kw), dtype=act, device=dev)
            if binding.has_readers:
                ctx.extras[("step_kv", binding.entry)] = (k_step, k_step)
        elif own_kv:
            k_step, _ = ctx.extras[("step_kv", binding.entry)]
        # q: rotated part turned; key: latent normed, rotated part turned; the value is the key
        K.qk_prepare(proj, ctx.positions, ctx.token_row, ctx.seq_end, q,
                     k_step if write else None, None,
                     cache.k if write else None, None,
                     cache.page_table if write else None, cache.table_stride, cache.ring,
                     q_off=0, n_heads=nh, q_width=hd + rd, k_off=nq, n_kv=1, k_width=kw,
                     v_off=0, v_width=rank, v_from_k=True, q_norm=None, k_norm=self.c_norm,
                     eps=self.norm_eps, inv_freq=inv_freq, rot_dims=rot_dims, rot_style=style,
                     rot_magnitude=magnitude, q_rot_off=hd, k_rot_off=rank, status=ctx.status)
        if self.uk_t.dtype != act:
            # (a checkpoint that stores its matrices in 32-bit keeps them so; the per-head products
            # take operands of the activations' type)
            self.uk_t, self.uv = self.uk_t.to(act), self.uv.to(act)
        # q'_h = [Wuk_h^T q_p | q_r]
        q_abs = torch.empty((n, nh * kw), dtype=act, device=dev)
        K.head_linear(q, self.uk_t, q_abs, x_head=hd + rd, x_off=0, y_head=kw, tail=rd, x_tail_off=hd)
        o_lat = torch.empty((n, nh * kw), dtype=act, device=dev)
        scored_attention(self.scores(), q_abs.view(n, nh, kw), k_step, k_step, cache, ctx, o_lat)
        # o_h = Wuv_h (the first kv_rank columns of the weighted sum), times the gate
        o = torch.empty((n, nh * vd), dtype=act, device=dev)
        K.head_linear(o_lat, self.uv, o, x_head=kw, x_off=0, y_head=vd,
                      gate=proj if self.gate else None, gate_off=nq + kw)
        project_out(self.out, o, ctx, residual)
