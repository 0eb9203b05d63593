"""Typed configuration of the Budanex decoder, read from its own config.json keys.

The design: token embedding followed by an RMS norm; pre-norm layers x += mixer(norm(x)),
x += ff(norm(x)) (the second half optional per layer) whose mixer is one of three kinds: grouped
attention with biases, q and k normed over all heads at once, a partial rotation and soft-capped
scores; a Mamba-2 state-space mixer; latent attention with a sliding window, a learned sink per
head, a YaRN-scaled interleaved rotation and an output gate.  A stretch of the layers may run
several times in a row with the same weights (each pass with keys and state of its own), the
embedding output and a learned vector per pass added before each pass.  Dense gated feed-forward
with the tanh form of gelu; final norm, head, soft-capped logits.  config.json keys:

    architecture        "Budanex"
    vocab, width        sizes; norm.eps: eps of every norm; logit_softcap: cap of the logits
    loop                null, or {start, stop, times}: layers start .. stop-1 run `times` times
    layers[i].type      "attention" | "mamba2" | "latent_attention"
    layers[i].mixer     attention: heads, kv_heads, dim, vdim, scale, softcap, rot {base, dims}
                        mamba2: heads, vdim, state, groups, conv, norm_groups
                        latent_attention: heads, dim, rot_dim, vdim, kv_rank, scale, mask {size},
                        rot {base, dims, scaling {factor, original, fast, slow}}
    layers[i].mlp       null, or {kind: "dense", ff}
    max_positions       optional bound on a sequence's length (default 2^20)

Tensor names: ``embed``, ``embed.norm``, ``loop.step``, ``final.norm``, ``head``, and per layer
``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.{gate,up,down}``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple

from .base import (ConfigError, ConfigReader, LayerSpec, ModelPlan, PartSpec, default_schedule,
                   looped_schedule)

ARCHITECTURE = "Budanex"
MIXERS = ("attention", "mamba2", "latent_attention")
FEED_FORWARDS = ("dense",)
DEFAULT_MAX_POSITIONS = 1 << 20


def _rotation(data: Optional[Mapping[str, Any]], where: str, head_width: int,
              style: str) -> Optional[PartSpec]:
    """The ``rot`` object of a mixer as a rotary part (None: no rotation)."""
    if data is None:
        return None
    r = ConfigReader(data, where)
    dims = r.integer("dims", minimum=0)
    if dims == 0:
        return None
    if dims % 2 != 0 or dims > head_width:
        raise ConfigError(f"{where}: dims {dims} must be even and at most {head_width}")
    params = {"head_dim": head_width, "rotary_dim": dims, "theta": r.number("base", positive=True),
              "style": style}
    scaling = data.get("scaling")
    if scaling is not None:
        sr = ConfigReader(scaling, f"{where}.scaling")
        params["scaling"] = {k: sr.number(k, positive=True)
                             for k in ("factor", "original", "fast", "slow")}
    return PartSpec("rotary", params)


def _window(data: Mapping[str, Any], where: str) -> int:
    mask = data.get("mask")
    if mask is None:
        return 0
    return ConfigReader(mask, f"{where}.mask").integer("size", minimum=1)


@dataclass(frozen=True)
class BudanexLayer:
    type: str
    mixer: Mapping[str, Any]        # the mixer's object as config.json gives it (checked)
    mlp_kind: Optional[str]         # None: no feed-forward
    ff: int = 0


@dataclass(frozen=True)
class BudanexConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_softcap: float            # 0: none
    loop: Optional[Tuple[int, int, int]]      # (start, stop, times)
    layers: Tuple[BudanexLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str = "config.json") -> "BudanexConfig":
        r = ConfigReader(data, where)
        raw_layers = data.get("layers")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise ConfigError(f"{where}: key 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw_layers):
            w = f"{where}.layers[{i}]"
            lr = ConfigReader(entry, w)
            kind = lr.string("type")
            if kind not in MIXERS:
                raise ConfigError(f"{w}: unknown mixer type {kind!r} (known: {', '.join(MIXERS)})")
            if not isinstance(entry.get("mixer"), Mapping):
                raise ConfigError(f"{w}: key 'mixer' must be an object")
            mlp = entry.get("mlp")
            mlp_kind, ff = None, 0
            if mlp is not None:
                mr = ConfigReader(mlp, f"{w}.mlp")
                mlp_kind = mr.string("kind")
                if mlp_kind not in FEED_FORWARDS:
                    raise ConfigError(f"{w}.mlp: unknown kind {mlp_kind!r} "
                                      f"(known: {', '.join(FEED_FORWARDS)})")
                ff = mr.integer("ff", minimum=1)
            layers.append(BudanexLayer(kind, dict(entry["mixer"]), mlp_kind, ff))
        loop = None
        if data.get("loop") is not None:
            lo = ConfigReader(data["loop"], f"{where}.loop")
            loop = (lo.integer("start", minimum=0), lo.integer("stop", minimum=1),
                    lo.integer("times", minimum=1))
            if not loop[0] < loop[1] <= len(layers):
                raise ConfigError(f"{where}.loop: layers [{loop[0]}, {loop[1]}) do not lie within "
                                  f"the {len(layers)} layers")
        norm = data.get("norm") or {}
        cfg = cls(
            vocab=r.integer("vocab", minimum=1),
            width=r.integer("width", minimum=1),
            norm_eps=ConfigReader(norm, f"{where}.norm").number("eps", positive=True),
            logit_softcap=r.number("logit_softcap", default=0.0),
            loop=loop,
            layers=tuple(layers),
            max_positions=r.integer("max_positions", default=DEFAULT_MAX_POSITIONS, minimum=1),
            extra={k: v for k, v in data.items()},
        )
        cfg.plan()          # every mixer's keys are read (and refused) here, not at the first step
        return cfg

    @classmethod
    def from_folder(cls, folder: str) -> "BudanexConfig":
        path = os.path.join(folder, "config.json")
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f), where=path)

    def to_dict(self) -> dict:
        layers = [{"type": layer.type, "mixer": dict(layer.mixer),
                   "mlp": None if layer.mlp_kind is None else {"kind": layer.mlp_kind, "ff": layer.ff}}
                  for layer in self.layers]
        out = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "layers": layers,
               "loop": None if self.loop is None else
               {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out

    # ---- lowering to parts ----------------------------------------------------------
    def _mixer(self, i: int, layer: BudanexLayer) -> PartSpec:
        w = f"config.layers[{i}].mixer"
        m = layer.mixer
        r = ConfigReader(m, w)
        common = {"hidden_size": self.width, "norm_eps": self.norm_eps, "tensor_prefix": "mix."}
        if layer.type == "attention":
            heads = r.integer("heads", minimum=1)
            kv = r.integer("kv_heads", default=heads, minimum=1)
            if heads % kv != 0:
                raise ConfigError(f"{w}: heads {heads} is not a multiple of kv_heads {kv}")
            dim = r.integer("dim", minimum=1)
            return PartSpec("qk_norm_attention", dict(
                common, n_heads=heads, n_kv_heads=kv, head_dim=dim,
                value_dim=r.integer("vdim", default=dim, minimum=1), scale=r.number("scale"),
                softcap=r.number("softcap", default=0.0), window=_window(m, w), qk_norm=True,
                bias=True, position=_rotation(m.get("rot"), f"{w}.rot", dim, "neox")))
        if layer.type == "mamba2":
            heads = r.integer("heads", minimum=1)
            groups = r.integer("groups", default=1, minimum=1)
            if heads % groups != 0:
                raise ConfigError(f"{w}: heads {heads} is not a multiple of groups {groups}")
            return PartSpec("mamba2", dict(
                common, n_heads=heads, head_dim=r.integer("vdim", minimum=1),
                n_state=r.integer("state", minimum=1), groups=groups,
                conv=r.integer("conv", minimum=1),
                norm_groups=r.integer("norm_groups", default=1, minimum=1)))
        # latent attention
        rot_dim = r.integer("rot_dim", minimum=0)
        return PartSpec("latent_attention", dict(
            common, n_heads=r.integer("heads", minimum=1), head_dim=r.integer("dim", minimum=1),
            rot_dim=rot_dim, value_dim=r.integer("vdim", minimum=1),
            kv_rank=r.integer("kv_rank", minimum=1), scale=r.number("scale"),
            window=_window(m, w), sink=True, gate=True,
            position=_rotation(m.get("rot"), f"{w}.rot", rot_dim, "interleaved") if rot_dim else None))

    def plan(self) -> ModelPlan:
        norm = PartSpec("rms_norm", {"size": self.width, "eps": self.norm_eps})
        layers = []
        for i, layer in enumerate(self.layers):
            ffn = ffn_norm = None
            if layer.mlp_kind == "dense":
                ffn = PartSpec("gated_mlp", {
                    "hidden_size": self.width, "intermediate_size": layer.ff,
                    "activation": "gelu_tanh", "gate_name": "mlp.gate", "up_name": "mlp.up",
                    "down_name": "mlp.down"})
                ffn_norm = norm.with_params(name="norm2", tensor_name="norm2")
            layers.append(LayerSpec(
                prefix=f"l{i}.",
                block=PartSpec("pre_norm", {}),
                mixer=self._mixer(i, layer),
                mixer_norm=norm.with_params(name="norm1", tensor_name="norm1"),
                feed_forward=ffn,
                feed_forward_norm=ffn_norm,
            ))
        injection = None
        if self.loop is not None:
            schedule = looped_schedule(len(layers), *self.loop)
            injection = PartSpec("pass_injection", {
                "width": self.width, "passes": self.loop[2], "tensor_name": "loop.step",
                "add_embedding": True})
        else:
            schedule = default_schedule(len(layers))
        plan = ModelPlan(
            architecture=ARCHITECTURE,
            vocab_size=self.vocab,
            hidden_size=self.width,
            embedding_name="embed",
            head_name="head",
            final_norm=norm.with_params(name="final.norm", tensor_name="final.norm"),
            final_norm_prefix="",
            layers=layers,
            schedule=schedule,
            max_positions=self.max_positions,
            after_embedding=PartSpec("embedding_norm", {
                "width": self.width, "eps": self.norm_eps, "tensor_name": "embed.norm"}),
            on_logits=(PartSpec("logit_softcap", {"cap": self.logit_softcap})
                       if self.logit_softcap else None),
            pass_injection=injection,
            model_part_prefix="",
        )
        plan.validate()
        return plan
