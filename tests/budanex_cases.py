"""Small Budanex configurations of the tests, each with sizes of its own, and their folders."""
from __future__ import annotations

import tempfile


def _attention(heads, kv, dim, vdim, scale, softcap, rot_dims, base=10000.0):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale,
                      "softcap": softcap, "rot": {"base": base, "dims": rot_dims}}}


def _mamba(heads, vdim, state, groups, conv, norm_groups):
    return {"type": "mamba2",
            "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                      "norm_groups": norm_groups}}


def _latent(heads, dim, rot_dim, vdim, rank, scale, window, scaling=None, base=50000.0):
    rot = {"base": base, "dims": rot_dim}
    if scaling is not None:
        rot["scaling"] = scaling
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
                      "scale": scale, "mask": {"size": window}, "rot": rot}}


def _with(layer, ff=None):
    out = dict(layer)
    out["mlp"] = None if ff is None else {"kind": "dense", "ff": ff}
    return out


# every mixer once plus a second state-space layer with a feed-forward; the loop covers the first
# three layers and runs three times; windows and conv states shorter than a page
BUD_A = {
    "architecture": "Budanex", "vocab": 97, "width": 64, "norm": {"eps": 1e-6},
    "logit_softcap": 9.0, "loop": {"start": 0, "stop": 3, "times": 3},
    "layers": [_with(_attention(4, 2, 16, 24, 0.3, 20.0, 8), 48),
               _with(_mamba(4, 8, 16, 2, 4, 2)),
               _with(_latent(2, 16, 8, 12, 24, 0.25, 20,
                             {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}), 40),
               _with(_mamba(2, 24, 8, 1, 2, 1), 56)],
}
# no loop, no cap on the logits; a width the tensor-core product does not take; sizes that are
# multiples of nothing; windows of exactly a page and of a page and one; a rotation of the whole
# head; as many key/value heads as heads; as many groups as heads; one tap; a state of 24
BUD_B = {
    "architecture": "Budanex", "vocab": 131, "width": 100, "norm": {"eps": 1e-5}, "loop": None,
    "layers": [_with(_latent(3, 10, 6, 14, 20, 0.4, 64, None), 36),
               _with(_attention(3, 3, 12, 20, 0.5, 5.0, 12), 36),
               _with(_mamba(6, 10, 24, 6, 1, 3), 28),
               _with(_latent(5, 12, 4, 6, 30, 0.3, 65,
                             {"factor": 2.0, "original": 32, "fast": 8.0, "slow": 1.0})),
               _with(_mamba(5, 12, 40, 1, 3, 5))],
}
# sizes the tensor-core kernels take; the loop covers the last two layers (to the very end) and
# runs twice; a window longer than a page that is no multiple of one; more heads on one latent
BUD_C = {
    "architecture": "Budanex", "vocab": 211, "width": 256, "norm": {"eps": 1e-5},
    "logit_softcap": 30.0, "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [_with(_mamba(4, 64, 64, 2, 4, 1), 384),
               _with(_latent(8, 32, 64, 64, 64, 0.2, 100,
                             {"factor": 4.0, "original": 128, "fast": 32.0, "slow": 1.0}), 256),
               _with(_attention(4, 1, 64, 128, 0.125, 40.0, 32, 1000000.0), 256)],
}
# keys and values of one size the tensor-memory kernel takes, in both attention mixers (128 with a
# soft cap; a latent of 48 + 16); one pass of a loop over all layers; a single key/value head
BUD_D = {
    "architecture": "Budanex", "vocab": 173, "width": 128, "norm": {"eps": 1e-6},
    "logit_softcap": 12.0, "loop": {"start": 0, "stop": 3, "times": 1},
    "layers": [_with(_attention(2, 1, 128, 128, 0.09, 15.0, 128, 500000.0), 192),
               _with(_latent(4, 24, 16, 40, 48, 0.18, 150,
                             {"factor": 16.0, "original": 256, "fast": 64.0, "slow": 4.0}, 10000.0)),
               _with(_mamba(2, 32, 64, 1, 4, 2), 160)],
}
CASES = {"A": (BUD_A, 21), "B": (BUD_B, 22), "C": (BUD_C, 23), "D": (BUD_D, 24)}


def make_folder(name: str) -> str:
    """A folder with seeded weights: matrices N(0, 0.08), norm weights 1 + N(0, 0.05), the
    per-head and per-channel vectors around their means."""
    from minfer_b200.model import write_random_model
    cfg, seed = CASES[name]
    folder = tempfile.mkdtemp(prefix=f"minfer_b200_bud{name}_")
    write_random_model(folder, cfg, seed, "bfloat16", norm_std=0.05, weight_std=0.08)
    return folder
