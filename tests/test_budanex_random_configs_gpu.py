"""Random Budanex configurations (sizes, order of layers, windows, loops, constants drawn from a
seed): the engine against the plain implementation, whole prompts, a batch of two, the last tokens
one by one and portions of a random size, in both precisions."""
import random
import tempfile

import pytest
import torch

import plain_budanex as P
from helpers import logits_err, random_ids

pytestmark = pytest.mark.gpu


def divisors(n): return [d for d in range(1, n + 1) if n % d == 0]

def make(rng):
    """A configuration drawn from ``rng``: 1 to 6 layers of any kind, sizes that are multiples of
    nothing, a loop anywhere (or none), with or without a cap on the logits."""
    width = rng.choice([40, 48, 64, 96, 100, 128, 160, 192, 256, 320])
    n_layers = rng.randint(1, 6)
    layers = []
    for _ in range(n_layers):
        kind = rng.choice(["attention", "mamba2", "latent_attention"])
        if kind == "attention":
            heads = rng.choice([1, 2, 3, 4, 6, 8]); kv = rng.choice(divisors(heads))
            dim = rng.choice([8, 16, 24, 32, 48, 64, 96, 128]); vdim = rng.choice([dim, dim, 8, 16, 32, 64, 128])
            rd = rng.choice([dim, 2 * rng.randint(1, dim // 2)])
            m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": rng.choice([dim ** -0.5, 0.125, 0.3]),
                 "softcap": rng.choice([5.0, 20.0, 50.0]), "rot": {"base": rng.choice([1e4, 2e4, 1e6]), "dims": rd}}
        elif kind == "mamba2":
            heads = rng.choice([1, 2, 3, 4, 6, 8, 12]); vdim = rng.choice([4, 8, 12, 16, 32, 64])
            inner = heads * vdim
            m = {"heads": heads, "vdim": vdim, "state": rng.choice([4, 6, 8, 16, 24, 32, 64, 128]),
                 "groups": rng.choice(divisors(heads)), "conv": rng.randint(1, 5), "norm_groups": rng.choice([g for g in divisors(inner) if g <= 8])}
        else:
            rot_dim = 2 * rng.randint(1, 32)
            m = {"heads": rng.choice([1, 2, 3, 4, 5, 8, 16, 20]), "dim": rng.choice([8, 16, 20, 32, 64]), "rot_dim": rot_dim,
                 "vdim": rng.choice([8, 12, 32, 64]), "kv_rank": rng.choice([8, 24, 32, 48, 64, 96, 100, 128 - rot_dim if rot_dim < 120 else 8, 160]),
                 "scale": rng.choice([0.125, 0.2, 0.08]), "mask": {"size": rng.choice([1, 2, 7, 63, 64, 65, 100, 136, 200, 300])},
                 "rot": {"base": rng.choice([1e4, 5e5]), "dims": rot_dim}}
            if rng.random() < 0.7:
                m["rot"]["scaling"] = {"factor": rng.choice([2.0, 4.0, 8.0]), "original": rng.choice([64, 512, 4096]),
                                       "fast": rng.choice([16.0, 32.0]), "slow": rng.choice([1.0, 2.0])}
        mlp = None if rng.random() < 0.4 else {"kind": "dense", "ff": rng.choice([24, 40, 64, 136, 320])}
        layers.append({"type": kind, "mixer": m, "mlp": mlp})
    loop = None
    if rng.random() < 0.7:
        a = rng.randint(0, n_layers - 1); b = rng.randint(a + 1, n_layers)
        loop = {"start": a, "stop": b, "times": rng.randint(1, 3)}
    cfg = {"architecture": "Budanex", "vocab": rng.randint(50, 700), "width": width, "norm": {"eps": rng.choice([1e-5, 1e-6])},
           "loop": loop, "layers": layers}
    if rng.random() < 0.8:
        cfg["logit_softcap"] = rng.choice([15.0, 30.0, 8.0])
    return cfg


@pytest.mark.parametrize("seed", [3, 17, 58, 114, 207, 351, 388, 399])
def test_random_configuration(seed):
    from minfer_b200.engine.step import Engine
    from minfer_b200.model import Model, write_random_model
    rng = random.Random(seed)
    cfg = make(rng)
    folder = tempfile.mkdtemp(prefix="minfer_b200_budr_")
    write_random_model(folder, cfg, seed, "bfloat16", norm_std=0.05, weight_std=0.08)
    c, w = P.load_folder(folder)
    n = rng.choice([1, 5, 37, 70, 130, 210])
    ids = random_ids(n, cfg["vocab"], seed)
    ids2 = random_ids(rng.randint(1, 60), cfg["vocab"], seed + 1000)
    want, want2 = P.forward(c, w, ids), P.forward(c, w, ids2)
    cut = max(1, n - rng.randint(1, 24))
    portion = rng.choice([2, 3, 50, 64, 170])
    for dtype in ("float32", "bfloat16"):
        eng = Engine(Model.from_folder(folder, dtype, "cuda:0"), max_tokens=2048)
        s = eng.acquire()
        got = eng.step([s], [ids], [list(range(n))])
        eng.release(s)
        err, bound = logits_err(got, want, dtype)
        assert err < bound, ("whole", dtype, err, bound)
        a, b = eng.acquire(), eng.acquire()
        out = eng.step([a, b], [ids[:cut], ids2], [list(range(cut)), list(range(len(ids2)))])
        err, bound = logits_err(out[cut:], want2, dtype)
        assert err < bound, ("second of a batch", dtype, err, bound)
        eng.release(b)
        rows = [out[:cut]] + [eng.step([a], [[ids[t]]], [[0]]) for t in range(cut, n)]
        eng.release(a)
        err, bound = logits_err(torch.cat(rows), want, dtype)
        assert err < bound, ("one by one", dtype, err, bound)
        s = eng.acquire()
        rows = []
        for lo in range(0, n, portion):
            part = ids[lo:lo + portion]
            rows.append(eng.step([s], [part], [list(range(len(part)))]))
        eng.release(s)
        err, bound = logits_err(torch.cat(rows), want, dtype)
        assert err < bound, ("portions", dtype, err, bound)
        eng.check_status()
        eng.cache.check_canaries()
