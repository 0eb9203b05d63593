"""The Furitar configuration reader, its plan and tensor names, and the plain implementation's
own consistency (no GPU)."""
import copy

import pytest
import torch

import minfer_b200.models  # noqa: F401  (registers the shipped architectures)
import plain_furitar as P
from furitar_cases import FUR_A, FUR_B


def _plan(cfg):
    from minfer_b200.registry import plan_from_config
    return plan_from_config(cfg)


def test_registry_picks_the_architecture_by_its_single_name():
    from minfer_b200.config.furitar import FuritarConfig
    from minfer_b200.registry import read_config
    c = read_config(FUR_A)
    assert isinstance(c, FuritarConfig)
    assert c.layers[0].mixer.chunk == 10 and c.layers[1].mlp_kind is None
    assert c.layers[2].mixer.kv_heads == 1 and c.layers[2].mixer.vdim == 8
    assert read_config(c.to_dict()) == c


def test_tensor_names_and_shapes():
    from minfer_b200.model import Model
    from minfer_b200.registry import read_config
    c = read_config(FUR_A)
    specs = {s.name: tuple(s.shape) for s in Model(c.plan(), "float32", c).tensor_specs()}
    assert specs["embed"] == (97, 72) and specs["pos"] == (700, 72) and specs["head"] == (97, 72)
    assert specs["final.norm"] == (72,)
    assert specs["l0.mix.q"] == (64, 72) and specs["l0.mix.k"] == (32, 72)
    assert specs["l0.mix.v"] == (48, 72) and specs["l0.mix.o"] == (72, 96)
    assert specs["l0.mix.r1"] == (4,) and specs["l0.shift"] == (72,) and specs["l0.mlp.act"] == (2,)
    assert specs["l0.mlp.up"] == (56, 72) and specs["l0.mlp.down"] == (72, 56)
    assert "l1.mlp.up" not in specs and "l1.norm2" not in specs and "l1.norm1" in specs
    assert specs["l2.mix.v"] == (8, 72)


def test_plan_carries_every_constant():
    plan = _plan(FUR_B)
    assert plan.embedding_scale == 1.0 and plan.max_positions == 400
    assert plan.final_norm.params["gain"] == 1.0
    m = plan.layers[1].mixer.params
    assert (m["chunk"], m["head_dim"], m["value_dim"], m["scale"]) == (65, 20, 12, 0.4)
    assert plan.layers[3].mixer.params["chunk"] == 0
    assert _plan(FUR_A).final_norm.params["gain"] == 1.25


@pytest.mark.parametrize("damage, word", [
    (lambda c: c["layers"][0].update(type="conv"), "mixer type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "kind"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"].pop("dim"), "dim"),
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_bad_configurations_are_refused_by_name(damage, word):
    from minfer_b200.config.base import ConfigError
    from minfer_b200.registry import read_config
    cfg = copy.deepcopy(FUR_A)
    damage(cfg)
    with pytest.raises(ConfigError) as e:
        read_config(cfg)
    assert word in str(e.value)


def _random_weights(cfg, seed=0):
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    w = {"embed": r(cfg["vocab"], W), "pos": r(cfg["max_positions"], W) * 0.3,
         "final.norm": 1 + 0.1 * r(W), "head": r(cfg["vocab"], W) * 0.3}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        w[p + "norm1"], w[p + "shift"] = 1 + 0.1 * r(W), 0.5 + 0.3 * r(W)
        w[p + "mix.q"], w[p + "mix.k"] = r(m["heads"] * m["dim"], W) * 0.2, r(m["kv_heads"] * m["dim"], W) * 0.2
        w[p + "mix.v"] = r(m["kv_heads"] * m["vdim"], W) * 0.2
        w[p + "mix.o"] = r(W, m["heads"] * m["vdim"]) * 0.2
        w[p + "mix.r1"], w[p + "mix.r2"] = 0.5 + 0.2 * r(m["heads"]), 0.6 + 0.1 * r(m["heads"])
        if layer["mlp"] is not None:
            w[p + "norm2"] = 1 + 0.1 * r(W)
            w[p + "mlp.up"], w[p + "mlp.down"] = r(layer["mlp"]["ff"], W) * 0.2, r(W, layer["mlp"]["ff"]) * 0.2
            w[p + "mlp.act"] = r(2)
    return w


def test_plain_whole_equals_plain_in_pieces():
    w = _random_weights(FUR_A)
    ids = torch.randint(0, 97, (45,), generator=torch.Generator().manual_seed(5)).tolist()
    whole, _ = P.forward(FUR_A, w, ids)
    st, rows = None, []
    for lo, hi in ((0, 9), (9, 10), (10, 11), (11, 31), (31, 45)):
        logits, st = P.forward(FUR_A, w, ids[lo:hi], st)
        rows.append(logits)
    assert torch.allclose(torch.cat(rows), whole, rtol=0, atol=1e-10)


def test_plain_mechanisms_by_hand():
    # a chunk of 4: position 5 sees 4 and 5 only
    assert [j for j in range(8) if P.visible(5, j, 4)] == [4, 5]
    assert [j for j in range(8) if P.visible(5, j, 0)] == [0, 1, 2, 3, 4, 5]
    # one key of score 0: the sink takes half the weight
    q = torch.zeros(1, 1, 2, dtype=torch.float64)
    k = torch.ones(1, 1, 2, dtype=torch.float64)
    v = torch.tensor([[[2.0, 4.0, 6.0]]], dtype=torch.float64)
    z = torch.zeros(1, dtype=torch.float64)
    o = P.sink_attention(q, k, v, [0], [0], z, z, 1.0, 0)
    assert torch.allclose(o[0, 0], torch.tensor([1.0, 2.0, 3.0], dtype=torch.float64))
    # the shift with s = 1 hands over the row before; with s = 0 nothing
    h = torch.arange(6, dtype=torch.float64).view(3, 2)
    before = torch.tensor([9.0, 9.0], dtype=torch.float64)
    assert torch.equal(P.token_shift(h, before, torch.ones(2, dtype=torch.float64))[0], before)
    assert torch.equal(P.token_shift(h, before, torch.zeros(2, dtype=torch.float64)), h)
    # xIELU is continuous at 0 and has slope 1/2 there
    a = torch.tensor([0.3, -0.2], dtype=torch.float64)
    e = 1e-6
    zs = torch.tensor([-e, 0.0, e], dtype=torch.float64)
    y = P.xielu(zs, a)
    assert abs(float(y[1])) < 1e-12 and abs(float((y[2] - y[0]) / (2 * e)) - 0.5) < 1e-5


def test_command_line_writes_and_describes_a_random_model(tmp_path, capsys):
    """``random`` writes a folder from a configuration file; ``--info`` reads it back."""
    import json
    from minfer_b200 import cli
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(FUR_B))
    folder = tmp_path / "model"
    assert cli.main(["random", str(cfg_path), str(folder), "--seed", "3"]) == 0
    capsys.readouterr()
    assert cli.main(["--info", str(folder)]) == 0
    text = capsys.readouterr().out
    assert "architecture: Furitar" in text and "embed" in text
    cfg, w = P.load_folder(str(folder))
    assert cfg["architecture"] == "Furitar" and w["l3.mix.v"].shape == (40, 100)
    assert "l0.norm2" in w and w["pos"].shape == (400, 100)
