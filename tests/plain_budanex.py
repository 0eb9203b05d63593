"""A plain, slow implementation of the Budanex decoder, written from its equations: one
function per mechanism, tensors in, tensors out, no kernels, no cache manager, no code shared
with the library.  Everything runs in the dtype of the weights it is given (float64 in the
tests), on the CPU, over a whole sequence at once (position p counts from 0).

    norm               rms(x) = x / sqrt(mean(x^2) + eps);  norm(x, w) = rms(x) * w
    embedding          x_p = norm(E[t_p], w_e)                      ("the embedding output" e_p)
    layer              x += mixer(norm(x, w1));  x += ff(norm(x, w2))            (ff optional)
    loop               layers [start, stop) run `times` times with the same weights (each pass
                       with its own keys and state); before pass t: x += e (t > 0), x += L[t]
    attention          q, k, v = Wq u + bq, Wk u + bk, Wv u + bv;  q <- norm(q, wq) over all
                       heads at once, k likewise; first R dims of each head rotated (pairs
                       (i, i + R/2), angle p * base^(-2i/R));
                       s_ij = c * tanh((q_i . k_j) * scale / c);  causal softmax;  Wo
    mamba2             [z | x | B | C | dt] = W_in u;  (x, B, C) <- silu(causal conv + bias);
                       dt <- softplus(dt + dt_bias);  per head S_t = exp(-exp(A_log) dt) S_{t-1}
                       + dt B_t x_t^T;  y_t = S_t^T C_t + D x_t;  y <- y * silu(z);  group rms
                       norm * w;  Wo
    latent attention   q = Wq u (per head [D plain | Rd rotated]);  [c | kr] = Wdkv u,
                       c <- norm(c, wc);  per head k = [Wuk c | kr], v = Wuv c;  interleaved
                       rotation (pairs (2i, 2i+1)) with YaRN-scaled frequencies on the rotated
                       parts;  s_ij = (q_i . k_j) * scale, visible iff 0 <= i - j < window;
                       w_ij = exp(s_ij) / (exp(sink_h) + sum_j' exp(s_ij'));  o *= sigmoid(Wg u);  Wo
    feed-forward       Wd (gelu_tanh(Wg y) * (Wu y))
    output             logits = cap * tanh(H norm(x, wf) / cap)
"""
from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional, Tuple

import torch


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.log1p(torch.exp(-x.abs())) + torch.clamp(x, min=0)


# ---- rotations -------------------------------------------------------------------------------
def plain_frequencies(dims: int, base: float) -> List[float]:
    return [base ** (-2.0 * i / dims) for i in range(dims // 2)]


def yarn_frequencies(dims: int, base: float, scaling: Mapping) -> Tuple[List[float], float]:
    """(frequency per pair, factor on cosine and sine)."""
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def dim_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(scaling["slow"]))), dims - 1)
    out = []
    for i, f in enumerate(plain_frequencies(dims, base)):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: List[int], freqs: List[float], layout: str,
           magnitude: float = 1.0) -> torch.Tensor:
    """``x`` [n, heads, d]: the first 2 * len(freqs) dims of each head are rotated, the rest pass.
    ``layout`` "half": pair (i, i + R/2); "interleaved": pair (2i, 2i + 1)."""
    out = x.clone()
    half = len(freqs)
    for a, p in enumerate(positions):
        for i, f in enumerate(freqs):
            ang = p * f
            c, s = math.cos(ang) * magnitude, math.sin(ang) * magnitude
            i0, i1 = (i, i + half) if layout == "half" else (2 * i, 2 * i + 1)
            u, v = x[a, :, i0], x[a, :, i1]
            out[a, :, i0] = u * c - v * s
            out[a, :, i1] = v * c + u * s
    return out


# ---- mixers ------------------------------------------------------------------------------------
def attention_mixer(u: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping,
                    eps: float) -> torch.Tensor:
    n = u.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = u @ w[p + "q"].T + w[p + "q.b"]
    k = u @ w[p + "k"].T + w[p + "k.b"]
    v = u @ w[p + "v"].T + w[p + "v.b"]
    q = rms_norm(q, w[p + "q.norm"], eps).view(n, H, D)
    k = rms_norm(k, w[p + "k.norm"], eps).view(n, G, D)
    v = v.view(n, G, Dv)
    pos = list(range(n))
    freqs = plain_frequencies(m["rot"]["dims"], float(m["rot"]["base"]))
    q, k = rotate(q, pos, freqs, "half"), rotate(k, pos, freqs, "half")
    cap = float(m["softcap"])
    out = torch.zeros((n, H, Dv), dtype=u.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(n):
            s = (k[:i + 1, g] @ q[i, h]) * float(m["scale"])
            s = cap * torch.tanh(s / cap)
            a = torch.softmax(s, dim=0)
            out[i, h] = a @ v[:i + 1, g]
    return out.reshape(n, H * Dv) @ w[p + "o"].T


def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """``x`` [n, channels], ``taps`` [channels, T] whose last column multiplies the current token."""
    n, ch = x.shape
    T = taps.shape[1]
    padded = torch.cat([torch.zeros((T - 1, ch), dtype=x.dtype), x], dim=0)
    out = bias.expand(n, ch).clone()
    for j in range(T):
        out = out + padded[j:j + n] * taps[:, j]
    return out


def mamba2_mixer(u: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping,
                 eps: float) -> torch.Tensor:
    n = u.shape[0]
    Hh, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = Hh * P
    proj = u @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].view(n, Hh, P)
    B = xbc[:, inner:inner + G * N].view(n, G, N)
    C = xbc[:, inner + G * N:].view(n, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    y = torch.zeros((n, Hh, P), dtype=u.dtype)
    for h in range(Hh):
        g = h // (Hh // G)
        S = torch.zeros((N, P), dtype=u.dtype)
        rate = torch.exp(w[p + "A_log"][h])
        for t in range(n):
            S = torch.exp(-rate * dt[t, h]) * S + dt[t, h] * torch.outer(B[t, g], x[t, h])
            y[t, h] = S.T @ C[t, g] + w[p + "D"][h] * x[t, h]
    y = y.reshape(n, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms_unit(y.view(n, parts, inner // parts), eps).reshape(n, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def latent_attention_mixer(u: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, m: Mapping,
                           eps: float) -> torch.Tensor:
    n = u.shape[0]
    H, D, Rd, Dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (u @ w[p + "q"].T).view(n, H, D + Rd)
    dkv = u @ w[p + "dkv"].T
    c = rms_norm(dkv[:, :rank], w[p + "dkv.norm"], eps)
    kr = dkv[:, rank:].view(n, 1, Rd)
    rot = m["rot"]
    if rot.get("scaling"):
        freqs, mag = yarn_frequencies(rot["dims"], float(rot["base"]), rot["scaling"])
    else:
        freqs, mag = plain_frequencies(rot["dims"], float(rot["base"])), 1.0
    pos = list(range(n))
    kr = rotate(kr, pos, freqs, "interleaved", mag)[:, 0]
    q_plain, q_rot = q[:, :, :D], rotate(q[:, :, D:].contiguous(), pos, freqs, "interleaved", mag)
    k_plain = (c @ w[p + "uk"].T).view(n, H, D)
    v = (c @ w[p + "uv"].T).view(n, H, Dv)
    window = int(m["mask"]["size"]) if m.get("mask") else 0
    out = torch.zeros((n, H, Dv), dtype=u.dtype)
    for h in range(H):
        for i in range(n):
            lo = max(0, i - window + 1) if window > 0 else 0
            s = (k_plain[lo:i + 1, h] @ q_plain[i, h] + kr[lo:i + 1] @ q_rot[i, h]) * float(m["scale"])
            top = torch.maximum(s.max(), w[p + "sink"][h])
            e = torch.exp(s - top)
            out[i, h] = (e @ v[lo:i + 1, h]) / (e.sum() + torch.exp(w[p + "sink"][h] - top))
    gate = torch.sigmoid(u @ w[p + "g"].T)
    return (out.reshape(n, H * Dv) * gate) @ w[p + "o"].T


MIXERS = {"attention": attention_mixer, "mamba2": mamba2_mixer,
          "latent_attention": latent_attention_mixer}


def feed_forward(y: torch.Tensor, w: Mapping[str, torch.Tensor], p: str) -> torch.Tensor:
    return (gelu_tanh(y @ w[p + "gate"].T) * (y @ w[p + "up"].T)) @ w[p + "down"].T


# ---- the model ---------------------------------------------------------------------------------
def run_order(config: Mapping) -> List[Tuple[int, Optional[int]]]:
    """(layer, pass number if this run is the first of a pass of the loop, else None)."""
    n_layers = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(n_layers)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(start)]
    for t in range(times):
        order += [(i, t if i == start else None) for i in range(start, stop)]
    order += [(i, None) for i in range(stop, n_layers)]
    return order


def forward(config: Mapping, weights: Mapping[str, torch.Tensor], tokens: List[int],
            taps: Optional[list] = None) -> torch.Tensor:
    """Logits [n, vocab] of one sequence; ``taps`` (a list) receives the residual stream after
    every layer run."""
    eps = float(config["norm"]["eps"])
    x = rms_norm(weights["embed"][torch.tensor(tokens, dtype=torch.long)], weights["embed.norm"], eps)
    e = x.clone()
    for layer, pass_no in run_order(config):
        if pass_no is not None:
            if pass_no > 0:
                x = x + e
            x = x + weights["loop.step"][pass_no]
        spec = config["layers"][layer]
        p = f"l{layer}."
        x = x + MIXERS[spec["type"]](rms_norm(x, weights[p + "norm1"], eps), weights, p + "mix.",
                                     spec["mixer"], eps)
        if spec.get("mlp") is not None:
            x = x + feed_forward(rms_norm(x, weights[p + "norm2"], eps), weights, p + "mlp.")
        if taps is not None:
            taps.append(x.clone())
    logits = rms_norm(x, weights["final.norm"], eps) @ weights["head"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    return logits


# ---- attention over given queries and keys (for tests of the attention kernels alone) ----------
def scored_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_pos: List[int],
                     scale: float, window: int = 0, softcap: float = 0.0,
                     sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [nq, H, D], k [nk, G, D], v [nk, G, Dv]; key j is at position j; query a at position
    q_pos[a] sees j <= q_pos[a] (and q_pos[a] - j < window if window > 0).  ``sink`` [H]: a score
    in the softmax's denominator without a value.  One (query, head) at a time."""
    nq, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((nq, H, v.shape[-1]), dtype=q.dtype)
    for a in range(nq):
        i = q_pos[a]
        lo = max(0, i - window + 1) if window > 0 else 0
        for h in range(H):
            g = h // (H // G)
            s = (k[lo:i + 1, g] @ q[a, h]) * scale
            if softcap > 0:
                s = softcap * torch.tanh(s / softcap)
            top = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - top)
            den = e.sum() if sink is None else e.sum() + torch.exp(sink[h] - top)
            out[a, h] = (e @ v[lo:i + 1, g]) / den
    return out


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


def generate_greedy(config: Mapping, w: Mapping[str, torch.Tensor], prompt: List[int],
                    n_new: int) -> List[int]:
    ids, out = list(prompt), []
    for _ in range(n_new):
        tok = int(torch.argmax(forward(config, w, ids)[-1]))
        out.append(tok)
        ids.append(tok)
    return out
