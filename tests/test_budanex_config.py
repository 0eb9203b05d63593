"""The Budanex configuration reader and its lowering to a plan (no GPU)."""
import copy
import math

import pytest
import torch

import plain_budanex as P
from budanex_cases import BUD_A, BUD_B, BUD_C
from minfer_b200.config.base import ConfigError, looped_schedule
from minfer_b200.model import Model
from minfer_b200.registry import read_config


def test_reads_every_size_and_constant():
    cfg = read_config(BUD_A)
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.logit_softcap) == (97, 64, 1e-6, 9.0)
    assert cfg.loop == (0, 3, 3)
    plan = cfg.plan()
    kinds = [layer.mixer.kind for layer in plan.layers]
    assert kinds == ["qk_norm_attention", "mamba2", "latent_attention", "mamba2"]
    att = plan.layers[0].mixer.params
    assert (att["n_heads"], att["n_kv_heads"], att["head_dim"], att["value_dim"]) == (4, 2, 16, 24)
    assert att["softcap"] == 20.0 and att["scale"] == 0.3
    assert att["position"].params["rotary_dim"] == 8 and att["position"].params["style"] == "neox"
    lat = plan.layers[2].mixer.params
    assert (lat["kv_rank"], lat["rot_dim"], lat["window"]) == (24, 8, 20)
    assert lat["position"].params["style"] == "interleaved"
    assert lat["position"].params["scaling"]["factor"] == 8.0
    mam = plan.layers[1].mixer.params
    assert (mam["n_state"], mam["groups"], mam["conv"], mam["norm_groups"]) == (16, 2, 4, 2)
    assert plan.layers[1].feed_forward is None and plan.layers[3].feed_forward is not None
    assert plan.layers[0].feed_forward.params["activation"] == "gelu_tanh"
    assert plan.on_logits.params["cap"] == 9.0
    assert cfg.to_dict()["layers"][2]["mixer"]["mask"] == {"size": 20}
    assert read_config(cfg.to_dict()) == cfg


def test_run_order_of_a_loop():
    plan = read_config(BUD_A).plan()
    assert [(c.layer, c.pass_start) for c in plan.schedule] == \
        [(0, 0), (1, None), (2, None), (0, 1), (1, None), (2, None), (0, 2), (1, None), (2, None),
         (3, None)]
    assert sorted(c.cache for c in plan.schedule) == list(range(10))      # an entry of its own each
    assert [(l, p) for l, p in P.run_order(BUD_A)] == [(c.layer, c.pass_start) for c in plan.schedule]
    plan_c = read_config(BUD_C).plan()
    assert [(c.layer, c.pass_start) for c in plan_c.schedule] == \
        [(0, None), (1, 0), (2, None), (1, 1), (2, None)]
    plan_b = read_config(BUD_B).plan()
    assert plan_b.pass_injection is None and plan_b.on_logits is None
    assert [c.layer for c in plan_b.schedule] == [0, 1, 2, 3, 4]
    with pytest.raises(ConfigError):
        looped_schedule(4, 2, 5, 2)


def test_tensor_names_and_shapes():
    cfg = read_config(BUD_A)
    specs = {s.name: tuple(s.shape) for s in Model(cfg.plan(), "float32", cfg).tensor_specs()}
    assert specs["embed"] == (97, 64) and specs["embed.norm"] == (64,) and specs["head"] == (97, 64)
    assert specs["loop.step"] == (3, 64) and specs["final.norm"] == (64,)
    assert specs["l0.mix.q"] == (64, 64) and specs["l0.mix.k.b"] == (32,) and specs["l0.mix.v"] == (48, 64)
    assert specs["l0.mix.q.norm"] == (64,) and specs["l0.mix.k.norm"] == (32,)
    assert specs["l0.mix.o"] == (64, 96) and specs["l0.mlp.gate"] == (48, 64)
    assert specs["l1.mix.in"] == (2 * 32 + 2 * 2 * 16 + 4, 64) and specs["l1.mix.conv"] == (32 + 64, 4)
    assert specs["l1.mix.A_log"] == (4,) and specs["l1.mix.norm"] == (32,) and "l1.norm2" not in specs
    assert specs["l2.mix.q"] == (2 * 24, 64) and specs["l2.mix.dkv"] == (32, 64)
    assert specs["l2.mix.uk"] == (32, 24) and specs["l2.mix.uv"] == (24, 24) and specs["l2.mix.sink"] == (2,)
    assert specs["l2.mix.g"] == (24, 64) and specs["l2.mix.o"] == (64, 24)
    assert "loop.step" not in {s.name for s in Model(read_config(BUD_B).plan(), "float32").tensor_specs()}


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown mixer"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][1]["mixer"].update(groups=3), "multiple"),
    (lambda c: c["layers"][2]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].pop("slow"), "slow"),
    (lambda c: c["layers"][0].update(mlp={"kind": "sparse", "ff": 8}), "unknown kind"),
])
def test_refusals(change, text):
    bad = copy.deepcopy(BUD_A)
    change(bad)
    with pytest.raises((ConfigError, ValueError)) as e:
        read_config(bad)
    assert text in str(e.value)


def test_scaled_frequencies_follow_the_plain_ones():
    from minfer_b200.parts.rotary import Rotary
    for dims, base, sc in ((8, 50000.0, {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}),
                           (64, 1e6, {"factor": 4.0, "original": 128, "fast": 32.0, "slow": 1.0}),
                           (4, 100.0, {"factor": 2.0, "original": 32, "fast": 8.0, "slow": 1.0})):
        rot = Rotary(dims, dims, base, style="interleaved", scaling=sc)
        want, mag = P.yarn_frequencies(dims, base, sc)
        assert torch.allclose(rot.inverse_frequencies(), torch.tensor(want, dtype=torch.float64),
                              rtol=1e-14, atol=0)
        assert math.isclose(rot.magnitude(), mag, rel_tol=1e-15)
    plain = Rotary(16, 8, 1e4)
    assert plain.magnitude() == 1.0
    assert torch.allclose(plain.inverse_frequencies(),
                          torch.tensor(P.plain_frequencies(8, 1e4), dtype=torch.float64), rtol=1e-14)


def test_parts_export_what_they_loaded():
    """Every tensor the model asks for comes back from ``export_state_dict`` under its name and
    in its shape (packed projections as views), for all three configurations."""
    for config in (BUD_A, BUD_B, BUD_C):
        cfg = read_config(config)
        model = Model(cfg.plan(), "float32", cfg)
        weights = {s.name: torch.randn(s.shape, dtype=torch.float32) for s in model.tensor_specs()}
        model.bind(weights, "cpu")
        out = model.export_state_dict()
        assert set(out) == set(weights)
        for name, t in weights.items():
            assert torch.equal(out[name], t), name
