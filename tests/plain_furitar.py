"""A plain, slow implementation of the Furitar decoder, written from its equations: one
function per mechanism, tensors in, tensors out, no kernels, no cache manager, no code shared
with the library.  Everything runs in the dtype of the weights it is given (float64 in the
tests), on the CPU.

Notation.  A sequence's tokens are t_0 .. t_{n-1}, position p counts from 0.  Width W.

    embedding          x_p = E[t_p] * a + P[p]
    norm               rms(x) = x / sqrt(mean(x^2) + eps);  norm(x, w) = rms(x) * w
    token shift        u_p = h_p + (h_{p-1} - h_p) * s      (h_{-1} = 0; h is the mixer's input
                                                             BEFORE the shift)
    layer              x += mixer(shift(norm(x, w1)));  x += ff(norm(x, w2))   (ff optional)
    attention          q, k, v = Wq u, Wk u, Wv u;  per head q <- rms(q), k <- rms(k)
                       s_ij = (q_i . k_j) * c - r1 * ln(1 + r2 * (i - j))
                       j visible from i  iff  j <= i and floor(i / C) == floor(j / C)
                       w_ij = exp(s_ij) / (1 + sum_j' exp(s_ij'))        (a sink of score 0)
                       o_i = sum_j w_ij v_j;  out = Wo concat_heads(o)
    feed-forward       Wd f(Wu y),  f(z) = sp(a0) z^2 + z/2                      (z > 0)
                                           (1/2 + sp(a1)) (exp(z) - 1 - z) + z/2  (z <= 0)
                       sp = softplus
    output             logits = H norm(x, wf) * g
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * w


def token_shift(h: torch.Tensor, before: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    """``h`` [n, W] the mixer's inputs of consecutive positions, ``before`` [W] the one of the
    position before the first (zeros at the start of a sequence)."""
    prev = torch.cat([before[None, :], h[:-1]], dim=0)
    return h + (prev - h) * s


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.log1p(torch.exp(-x.abs())) + torch.clamp(x, min=0)


def xielu(z: torch.Tensor, a: torch.Tensor) -> torch.Tensor:
    pos = softplus(a[0]) * z * z + 0.5 * z
    neg = (0.5 + softplus(a[1])) * (torch.expm1(torch.clamp(z, max=0)) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def visible(i: int, j: int, chunk: int) -> bool:
    if j > i:
        return False
    return chunk <= 0 or i // chunk == j // chunk


def sink_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_pos: List[int],
                   k_pos: List[int], r1: torch.Tensor, r2: torch.Tensor, scale: float,
                   chunk: int) -> torch.Tensor:
    """q [nq, H, D] (already unit-RMS), k [nk, G, D], v [nk, G, Dv]; returns [nq, H, Dv].
    One (query, head) at a time."""
    nq, n_heads, _ = q.shape
    n_kv = k.shape[1]
    group = n_heads // n_kv
    out = torch.zeros((nq, n_heads, v.shape[-1]), dtype=q.dtype)
    kp = torch.tensor(k_pos, dtype=torch.long)
    for a in range(nq):
        i = q_pos[a]
        rows = [b for b, j in enumerate(k_pos) if visible(i, j, chunk)]
        if not rows:
            continue
        dist = (i - kp[rows]).to(q.dtype)
        for h in range(n_heads):
            g = h // group
            s = (k[rows, g] @ q[a, h]) * scale - r1[h] * torch.log1p(r2[h] * dist)
            m = torch.clamp(s.max(), min=0.0)                 # the sink's score is 0
            e = torch.exp(s - m)
            w = e / (torch.exp(-m) + e.sum())
            out[a, h] = (w[:, None] * v[rows, g]).sum(dim=0)
    return out


class SequenceState:
    """What a sequence keeps between calls: per layer the keys, values and the mixer input of
    its last position; and its length."""

    def __init__(self, n_layers: int):
        self.k: List[Optional[torch.Tensor]] = [None] * n_layers
        self.v: List[Optional[torch.Tensor]] = [None] * n_layers
        self.last_h: List[Optional[torch.Tensor]] = [None] * n_layers
        self.length = 0


def attention_mixer(u: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float,
                    positions: List[int], st: SequenceState, layer: int) -> torch.Tensor:
    heads, kv, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    n = u.shape[0]
    q = (u @ w[p + "q"].T).view(n, heads, d)
    k = (u @ w[p + "k"].T).view(n, kv, d)
    v = (u @ w[p + "v"].T).view(n, kv, dv)
    q, k = rms_unit(q, eps), rms_unit(k, eps)
    if st.k[layer] is not None:
        k = torch.cat([st.k[layer], k], dim=0)
        v = torch.cat([st.v[layer], v], dim=0)
    st.k[layer], st.v[layer] = k, v
    chunk = int((m.get("mask") or {}).get("size", 0))
    o = sink_attention(q, k, v, positions, list(range(k.shape[0])), w[p + "r1"], w[p + "r2"],
                       float(m["scale"]), chunk)
    return o.reshape(n, heads * dv) @ w[p + "o"].T


def dense_ff(y: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return xielu(y @ w[p + "up"].T, w[p + "act"]) @ w[p + "down"].T


def forward(config: dict, w: Dict[str, torch.Tensor], tokens: List[int],
            state: Optional[SequenceState] = None, layer_outputs: Optional[list] = None):
    """Runs ``tokens`` as the next positions of a sequence (``state`` None: a new one).
    Returns (logits [n, vocab], state)."""
    layers = config["layers"]
    eps = float(config["norm"]["eps"])
    st = state if state is not None else SequenceState(len(layers))
    positions = list(range(st.length, st.length + len(tokens)))
    x = w["embed"][tokens] * float(config["embedding"]["scale"]) + w["pos"][positions]
    for i, layer in enumerate(layers):
        p = f"l{i}."
        h = rms_norm(x, w[p + "norm1"], eps)
        before = st.last_h[i] if st.last_h[i] is not None else torch.zeros_like(h[0])
        u = token_shift(h, before, w[p + "shift"])
        st.last_h[i] = h[-1].clone()
        if layer["type"] != "attention":
            raise ValueError(f"unknown mixer {layer['type']!r}")
        x = x + attention_mixer(u, w, p + "mix.", layer["mixer"], eps, positions, st, i)
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"unknown feed-forward {layer['mlp']['kind']!r}")
            x = x + dense_ff(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.")
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    st.length += len(tokens)
    logits = (rms_norm(x, w["final.norm"], eps) @ w["head"].T) * float(config["logit_scale"])
    return logits, st


def load_folder(folder: str, dtype: torch.dtype = torch.float64):
    import json
    import os
    from safetensors import safe_open
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    weights = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name).to(dtype)
    return cfg, weights


def generate_greedy(config: dict, w: Dict[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    logits, st = forward(config, w, list(prompt))
    out = []
    for _ in range(n_new):
        tok = int(torch.argmax(logits[-1]))
        out.append(tok)
        logits, st = forward(config, w, [tok], st)
    return out
