"""Dibizen without a GPU: config.json -> typed configuration -> model as data, the tensors it declares, the cache layout
(one page group for a layer and the layers that read its keys, one state slot per recurrent layer), and the plain
restatement's own properties (prefixes, the choice among groups, identity outputs, the temperature's steps)."""

from __future__ import annotations

import copy
import math

import pytest
import torch

import plain_dibizen as pd
from tokenmill_b200.config.dibizen_config import DibizenConfig
from tokenmill_b200.config.model_config import ConfigError
from tokenmill_b200.models.dibizen import dibizen_spec
from tokenmill_b200.parts.model import DecoderModel
from tokenmill_b200.weights import named_config
from tokenmill_b200.weights.random_init import random_tensors


def _model(name_or_raw):
    raw = named_config(name_or_raw) if isinstance(name_or_raw, str) else name_or_raw
    cfg = DibizenConfig.from_dict(raw)
    return cfg, DecoderModel(dibizen_spec(cfg), torch.float32, torch.device("cpu"))


def _set(raw, path, value=None, delete=False):
    bad = copy.deepcopy(raw)
    d = bad
    for k in path[:-1]:
        d = d[k]
    if delete:
        del d[path[-1]]
    else:
        d[path[-1]] = value
    return bad


def test_config_reads_every_size_and_refuses_what_the_design_lacks():
    raw = named_config("dibizen-tiny-a")
    cfg = DibizenConfig.from_dict(raw)
    assert (cfg.vocab, cfg.width, cfg.streams, cfg.eps, cfg.max_positions, cfg.logit_softcap) == (173, 48, 3, 1e-5, 300, 8.0)
    assert [l.type for l in cfg.layers] == ["attention", "mamba1", "lightning", "attention"]
    assert cfg.layers[1].mlp is None and cfg.layers[3].mixer["kv_from"] == 0 and cfg.hyper_connections
    for path, value in ((("layers", 0, "type"), "retention"), (("layers", 0, "mlp", "kind"), "dense"),
                        (("layers", 0, "mixer", "heads"), 5), (("layers", 0, "mixer", "window"), 7),
                        (("layers", 3, "mixer", "kv_from"), 3), (("layers", 3, "mixer", "kv_from"), 1),
                        (("layers", 3, "mixer", "dim"), 16), (("layers", 2, "mixer", "decay"), [0.5, 0.9]),
                        (("layers", 1, "mixer", "conv"), 0), (("layers", 0, "mlp", "router", "groups", "count"), 3),
                        (("layers", 0, "mlp", "router", "groups", "keep"), 5), (("layers", 0, "mlp", "router", "top"), 5),
                        (("layers", 0, "mixer", "q_temp", "every"), 0), (("norm", "eps"), 0.0), (("logit_softcap",), -1.0)):
        with pytest.raises(ConfigError):
            DibizenConfig.from_dict(_set(raw, path, value))
    for path in (("vocab",), ("max_positions",), ("layers", 0, "mixer", "scale"), ("layers", 1, "mixer", "dt_rank"),
                 ("layers", 2, "mixer", "vdim"), ("layers", 0, "mlp", "expert")):
        with pytest.raises(ConfigError):
            DibizenConfig.from_dict(_set(raw, path, delete=True))


def test_optional_keys_may_be_absent():
    raw = named_config("dibizen-tiny-a")
    bare = _set(_set(_set(raw, ("layers", 0, "mixer", "q_temp"), delete=True), ("logit_softcap",), delete=True),
                ("layers", 0, "mlp", "router", "groups"), delete=True)
    cfg = DibizenConfig.from_dict(bare)
    spec = dibizen_spec(cfg)
    assert spec.logit_softcap == 0.0 and spec.layers[0].mixer.params["q_temp"] is None
    assert spec.layers[0].feed_forward.params["groups"] == 1 and spec.layers[3].mixer.params["q_temp"] == (0.7, 16)
    # no ``streams``: one plain stream, and no read and write weights among the tensors
    plain = _set(named_config("dibizen-tiny-b"), ("streams",), delete=True)
    _, model = _model(plain)
    names = {w.name for w in model.weight_specs()}
    assert not any(".hc" in n for n in names) and "l0.norm1.alpha" in names
    _, learned = _model("dibizen-tiny-b")
    assert {w.name: tuple(w.shape) for w in learned.weight_specs()}["l0.hc1.mix"] == (1, 1)


def test_spec_declares_the_tensors_by_name():
    _, model = _model("dibizen-tiny-a")
    names = {w.name: tuple(w.shape) for w in model.weight_specs()}
    assert names["embed"] == (173, 48) and names["pos"] == (300, 48) and names["head"] == (173, 48)
    assert names["final.norm"] == (48,) and names["final.norm.b"] == (48,) and names["final.norm.alpha"] == ()
    assert names["l0.norm1.alpha"] == () and names["l0.hc1.in"] == (3,) and names["l0.hc2.mix"] == (3, 3)
    assert names["l0.mix.q"] == (48, 48) and names["l0.mix.k"] == (24, 48) and names["l0.mix.v"] == (40, 48)
    assert names["l0.mix.g"] == (80, 48) and names["l0.mix.o"] == (48, 80)
    assert names["l3.mix.q"] == (48, 48) and "l3.mix.k" not in names and "l3.mix.v" not in names and names["l3.mix.g"] == (80, 48)
    assert names["l1.mix.in"] == (144, 48) and names["l1.mix.conv"] == (72, 3) and names["l1.mix.conv.b"] == (72,)
    assert names["l1.mix.x"] == (5 + 24, 72) and names["l1.mix.dt"] == (72, 5) and names["l1.mix.A_log"] == (72, 12)
    assert names["l1.mix.D"] == (72,) and names["l1.mix.o"] == (48, 72)
    assert "l1.norm2" not in names and "l1.hc2.in" not in names and "l1.mlp.router" not in names
    assert names["l2.mix.q"] == (30, 48) and names["l2.mix.v"] == (42, 48) and names["l2.mix.norm"] == (42,)
    assert names["l0.mlp.router"] == (8, 48) and names["l0.mlp.correction"] == (8,) and names["l0.mlp.e5.up"] == (24, 48)
    assert "l0.mlp.e6.up" not in names and names["l3.mlp.router"] == (4, 48) and names["l2.mlp.e4.down"] == (48, 16)


def test_cache_layout_shared_pages_and_state_slots():
    _, model = _model("dibizen-tiny-a")
    layout = model.cache_layout()
    assert [(g.need.head_dim, g.need.window, g.need.planes, g.entries) for g in layout.groups] == [(2 * (12 + 20), None, 1, [0])]
    assert layout.entry_group[3] == layout.entry_group[0] and set(layout.entry_group) == {0, 3}
    assert layout.entry_state[1].shape == ((3 - 1) * 72 + 72 * 12,) and layout.entry_state[2].shape == (3 * 14 * 16,)       # 10 rows padded to 16
    assert set(layout.entry_state) == {1, 2} and not layout.block_state
    _, c = _model("dibizen-tiny-c")
    layout = c.cache_layout()
    assert len(layout.groups) == 1 and layout.groups[0].entries == [1]
    assert layout.entry_group[2] == layout.entry_group[1] == layout.entry_group[4]


def test_plain_prefixes_do_not_depend_on_what_follows():
    cfg, model = _model("dibizen-tiny-c")
    raw = named_config("dibizen-tiny-c")
    w = {k: v.float() for k, v in random_tensors(model, 5, torch.bfloat16).items()}
    toks = [(7 * i + 3) % cfg.vocab for i in range(60)]
    layers = []
    full = pd.forward(raw, w, toks, layers_out=layers)
    assert len(layers) == 5 and layers[0].shape == (60, cfg.width)
    assert (full[:33] - pd.forward(raw, w, toks[:33])).abs().max() < 1e-9
    assert float(full.abs().max()) <= 30.0          # the cap


def test_plain_choice_among_groups_with_identity_outputs():
    """Six outputs in three groups of two, the last two without tensors. The correction moves the choice, not the weights;
    an output outside the kept groups is never chosen, also when every choice score inside them is negative."""
    torch.manual_seed(0)
    W = {"r.router": torch.zeros(6, 4, dtype=torch.float64), "r.correction": torch.tensor([0.0, 0.0, -5.0, -5.1, -9.0, -9.0]).double()}
    h = torch.randn(3, 4, dtype=torch.float64)
    r = {"experts": 4, "identity": 2, "top": 2, "groups": {"count": 3, "keep": 1}}
    idx, w = pd.route(h, W, "r.", r)
    assert idx.tolist() == [[0, 1]] * 3 and torch.allclose(w, torch.full_like(w, 0.5))
    W["r.correction"] = torch.tensor([-9.0, -9.0, -5.0, -5.1, -5.05, -7.0]).double()
    idx, w = pd.route(h, W, "r.", r)
    assert idx.tolist() == [[2, 3]] * 3             # the group of the best single output, both of its members
    r["groups"]["keep"] = 2
    idx, w = pd.route(h, W, "r.", r)
    assert idx.tolist() == [[2, 4]] * 3             # two groups kept: the best two outputs among their four
    for e in range(4):
        W[f"r.e{e}.up"], W[f"r.e{e}.down"] = torch.randn(5, 4).double(), torch.randn(4, 5).double()
    out = pd.experts(h, W, "r.", {"router": r})
    y2 = (torch.relu(h @ W["r.e2.up"].T) ** 2) @ W["r.e2.down"].T
    assert torch.allclose(out, 0.5 * y2 + 0.5 * h)  # output 4 hands the input on


def test_plain_temperature_steps_and_streams():
    t = pd.query_temperature(torch.tensor([0, 14, 15, 30, 31, 47]), 0.7, 16)
    want = [1.0, 1.0, 1 + 0.7 * math.log(2), 1 + 0.7 * math.log(2), 1 + 0.7 * math.log(3), 1 + 0.7 * math.log(4)]
    assert torch.allclose(t, torch.tensor(want).double())
    x = [torch.ones(2, 3).double(), 2 * torch.ones(2, 3).double()]
    mix = torch.tensor([[1.0, 10.0], [100.0, 1000.0]]).double()         # [from, to]
    new = pd.stream_write(x, torch.ones(2, 3).double(), mix, torch.tensor([0.5, 0.25]).double())
    assert float(new[0][0, 0]) == 1 + 200 + 0.5 and float(new[1][0, 0]) == 10 + 2000 + 0.25
    assert float(pd.stream_read(x, torch.tensor([3.0, 5.0]).double())[0, 0]) == 13.0
