"""Small Furitar configurations of the tests, each with sizes of its own, and their folders."""
from __future__ import annotations

import tempfile


def _att(heads, kv, dim, vdim, scale, chunk=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    return m


def _layer(mixer, ff=None):
    return {"type": "attention", "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


# layers that differ in every size; one without a feed-forward; chunks smaller than a page
FUR_A = {
    "architecture": "Furitar", "vocab": 97, "width": 72, "max_positions": 700,
    "embedding": {"scale": 1.7}, "norm": {"eps": 1e-6}, "logit_scale": 1.25,
    "layers": [_layer(_att(4, 2, 16, 24, 0.3, 10), 56),
               _layer(_att(4, 4, 16, 16, 0.25, 10)),
               _layer(_att(2, 1, 32, 8, 0.2, 33), 40)],
}
# a width the tensor-core product does not take, key and value sizes that are no multiples of
# 8, a chunk of exactly a page, one of a page and one position, one of a single position, and
# a layer without a chunk mask; scales of 1
FUR_B = {
    "architecture": "Furitar", "vocab": 131, "width": 100, "max_positions": 400,
    "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5}, "logit_scale": 1.0,
    "layers": [_layer(_att(6, 3, 20, 12, 0.4, 64), 36),
               _layer(_att(6, 3, 20, 12, 0.4, 65), 36),
               _layer(_att(3, 3, 12, 20, 0.5, 1), 36),
               _layer(_att(2, 1, 24, 40, 0.3), 28)],
}
# the sizes the tensor-core attention kernels take, chunks wider than a page and no multiple
# of one
FUR_C = {
    "architecture": "Furitar", "vocab": 211, "width": 256, "max_positions": 1024,
    "embedding": {"scale": 2.5}, "norm": {"eps": 1e-5}, "logit_scale": 0.75,
    "layers": [_layer(_att(8, 2, 64, 64, 0.2, 200), 384),
               _layer(_att(4, 4, 128, 128, 0.15, 128), 384),
               _layer(_att(16, 1, 64, 128, 0.2, 150), 128)],
}
# sizes that are multiples of nothing: a width the vector kernels do not take, five heads of ten,
# more than 16 query heads on one key/value head, and a last layer without a feed-forward
FUR_D = {
    "architecture": "Furitar", "vocab": 77, "width": 90, "max_positions": 300,
    "embedding": {"scale": 0.5}, "norm": {"eps": 1e-4}, "logit_scale": 2.0,
    "layers": [_layer(_att(5, 5, 10, 6, 0.6, 7), 33),
               _layer(_att(20, 1, 16, 8, 0.3, 50), 18),
               _layer(_att(3, 1, 30, 14, 0.35, 129))],
}
CASES = {"A": (FUR_A, 11), "B": (FUR_B, 12), "C": (FUR_C, 13), "D": (FUR_D, 14)}


def make_folder(name: str) -> str:
    """A folder with seeded weights: matrices N(0, 0.08), norm weights 1 + N(0, 0.05), the
    per-head and per-channel vectors around their means."""
    from minfer_b200.model import write_random_model
    cfg, seed = CASES[name]
    folder = tempfile.mkdtemp(prefix=f"minfer_b200_fur{name}_")
    write_random_model(folder, cfg, seed, "bfloat16", norm_std=0.05, weight_std=0.08)
    return folder
