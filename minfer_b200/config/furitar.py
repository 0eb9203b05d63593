"""Typed configuration of the Furitar decoder, read from its own config.json keys.

The design: token embedding times a constant plus a learned vector per position; pre-norm
layers x += mixer(shift(norm(x))), x += ff(norm(x)) with a token shift in front of every mixer;
the mixer ``attention`` (grouped heads, keys and values of different widths, q and k of unit
root mean square, a logarithmic distance bias, a chunk mask, a softmax with a sink); an
optional dense feed-forward with the xIELU activation; a final norm and a head whose logits are
scaled by a constant.  config.json keys:

    architecture            "Furitar"
    vocab, width, max_positions
    embedding.scale         factor on the embedding rows
    norm.eps                eps of every norm (also of the unit norms of q and k)
    logit_scale             factor on the logits
    layers[i].type          the mixer: "attention"
    layers[i].mixer         heads, kv_heads, dim, vdim, scale, mask.size
    layers[i].mlp           null, or {kind: "dense", ff}

Tensor names: ``embed``, ``pos``, ``final.norm``, ``head``, and per layer ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.shift``, ``l<i>.mix.{q,k,v,o,r1,r2}``, ``l<i>.mlp.{up,down,act}``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple

from .base import (ConfigError, ConfigReader, LayerSpec, ModelPlan, PartSpec, default_schedule)

ARCHITECTURE = "Furitar"
MIXERS = ("attention",)
FEED_FORWARDS = ("dense",)


@dataclass(frozen=True)
class FuritarAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: int              # 0: no chunk mask

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "FuritarAttention":
        r = ConfigReader(data, where)
        heads = r.integer("heads", minimum=1)
        kv_heads = r.integer("kv_heads", default=heads, minimum=1)
        if heads % kv_heads != 0:
            raise ConfigError(f"{where}: heads {heads} is not a multiple of kv_heads {kv_heads}")
        dim = r.integer("dim", minimum=1)
        chunk = 0
        mask = data.get("mask")
        if mask is not None:
            chunk = ConfigReader(mask, f"{where}.mask").integer("size", minimum=1)
        return cls(heads=heads, kv_heads=kv_heads, dim=dim,
                   vdim=r.integer("vdim", default=dim, minimum=1),
                   scale=r.number("scale"), chunk=chunk)

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
             "scale": self.scale}
        if self.chunk:
            d["mask"] = {"size": self.chunk}
        return d


@dataclass(frozen=True)
class FuritarLayer:
    type: str
    mixer: FuritarAttention
    mlp_kind: Optional[str]         # None: no feed-forward
    ff: int = 0


@dataclass(frozen=True)
class FuritarConfig:
    vocab: int
    width: int
    max_positions: int
    embedding_scale: float
    norm_eps: float
    logit_scale: float
    layers: Tuple[FuritarLayer, ...]
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str = "config.json") -> "FuritarConfig":
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
            mixer = FuritarAttention.from_dict(entry["mixer"], f"{w}.mixer")
            mlp = entry.get("mlp")
            mlp_kind, ff = None, 0
            if mlp is not None:
                mr = ConfigReader(mlp, f"{w}.mlp")
                mlp_kind = mr.string("kind")
                if mlp_kind not in FEED_FORWARDS:
                    raise ConfigError(f"{w}.mlp: unknown kind {mlp_kind!r} "
                                      f"(known: {', '.join(FEED_FORWARDS)})")
                ff = mr.integer("ff", minimum=1)
            layers.append(FuritarLayer(kind, mixer, mlp_kind, ff))
        emb = data.get("embedding") or {}
        norm = data.get("norm") or {}
        return cls(
            vocab=r.integer("vocab", minimum=1),
            width=r.integer("width", minimum=1),
            max_positions=r.integer("max_positions", minimum=1),
            embedding_scale=ConfigReader(emb, f"{where}.embedding").number("scale", default=1.0),
            norm_eps=ConfigReader(norm, f"{where}.norm").number("eps", positive=True),
            logit_scale=r.number("logit_scale", default=1.0),
            layers=tuple(layers),
            extra={k: v for k, v in data.items()},
        )

    @classmethod
    def from_folder(cls, folder: str) -> "FuritarConfig":
        path = os.path.join(folder, "config.json")
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f), where=path)

    def to_dict(self) -> dict:
        layers = []
        for layer in self.layers:
            layers.append({
                "type": layer.type, "mixer": layer.mixer.to_dict(),
                "mlp": None if layer.mlp_kind is None else {"kind": layer.mlp_kind, "ff": layer.ff}})
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                "max_positions": self.max_positions, "embedding": {"scale": self.embedding_scale},
                "norm": {"eps": self.norm_eps}, "logit_scale": self.logit_scale, "layers": layers}

    # ---- lowering to parts ----------------------------------------------------------
    def plan(self) -> ModelPlan:
        norm = PartSpec("rms_norm", {"size": self.width, "eps": self.norm_eps})
        layers = []
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            mixer = PartSpec("sink_attention", {
                "hidden_size": self.width, "n_heads": m.heads, "n_kv_heads": m.kv_heads,
                "head_dim": m.dim, "value_dim": m.vdim, "scale": m.scale,
                "norm_eps": self.norm_eps, "chunk": m.chunk, "window": 0, "sink": True,
                "qk_norm": True, "distance_bias": True, "tensor_prefix": "mix.",
            })
            ffn = ffn_norm = None
            if layer.mlp_kind == "dense":
                ffn = PartSpec("dense_mlp", {
                    "hidden_size": self.width, "intermediate_size": layer.ff,
                    "activation": "xielu", "up_name": "mlp.up", "down_name": "mlp.down",
                    "act_name": "mlp.act"})
                ffn_norm = norm.with_params(name="norm2", tensor_name="norm2")
            layers.append(LayerSpec(
                prefix=f"l{i}.",
                block=PartSpec("pre_norm", {
                    "token_shift": {"size": self.width, "tensor_name": "shift"}}),
                mixer=mixer,
                mixer_norm=norm.with_params(name="norm1", tensor_name="norm1"),
                feed_forward=ffn,
                feed_forward_norm=ffn_norm,
            ))
        plan = ModelPlan(
            architecture=ARCHITECTURE,
            vocab_size=self.vocab,
            hidden_size=self.width,
            embedding_name="embed",
            head_name="head",
            # the logit scale rides on the last norm's weight: logits = head (norm(x) w g)
            final_norm=norm.with_params(name="final.norm", tensor_name="final.norm",
                                        gain=self.logit_scale),
            final_norm_prefix="",
            layers=layers,
            schedule=default_schedule(len(layers)),
            max_positions=self.max_positions,
            embedding_scale=self.embedding_scale,
            after_embedding=PartSpec("learned_positions", {
                "width": self.width, "positions": self.max_positions, "tensor_name": "pos"}),
            model_part_prefix="",
        )
        plan.validate()
        return plan
