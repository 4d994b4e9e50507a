"""Gofezen without a GPU: config.json -> typed configuration -> model as data, the tensors it declares, the cache layout
(one page group per shape of attention rows, one state slot per layer holding the convolutions' carried inputs and the
memories), and the plain restatement's own properties (prefixes, the window's edge, the delta rule's two forms, the
forget gate, experts weighted on their input)."""

from __future__ import annotations

import copy

import pytest
import torch

import plain_gofezen as pg
from tokenmill_b200.config.gofezen_config import GofezenConfig
from tokenmill_b200.config.model_config import ConfigError
from tokenmill_b200.kernels import ops
from tokenmill_b200.models.gofezen import gofezen_spec
from tokenmill_b200.parts.model import DecoderModel
from tokenmill_b200.weights import named_config
from tokenmill_b200.weights.random_init import random_tensors


def _model(name_or_raw):
    raw = named_config(name_or_raw) if isinstance(name_or_raw, str) else name_or_raw
    cfg = GofezenConfig.from_dict(raw)
    return cfg, DecoderModel(gofezen_spec(cfg), torch.float32, torch.device("cpu"))


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
    raw = named_config("gofezen-tiny-a")
    cfg, _ = _model(raw)
    assert (cfg.vocab, cfg.width, cfg.max_positions, cfg.eps) == (173, 48, 300, 1e-6)
    assert (cfg.embedding_scale, cfg.logit_scale, cfg.logit_softcap) == (6.9, 0.7, 8.0)
    assert [l.type for l in cfg.layers] == ["parallel", "hgrn2", "hgrn2", "parallel"]
    assert cfg.layers[0].mixer["left"]["mask"]["size"] == 24 and cfg.layers[3].mixer["right"]["conv"] == 1
    assert cfg.layers[2].mlp is None and cfg.layers[1].mlp == {"kind": "dense", "ff": 64}
    for path, value in ((["layers", 0, "type"], "attention"), (["layers", 0, "mixer", "left", "heads"], 5),
                        (["layers", 0, "mixer", "right", "kv_heads"], 3), (["layers", 0, "mixer", "left", "rot"], {"dims": 4}),
                        (["layers", 0, "mixer", "left", "mask", "keep_first"], 2), (["layers", 1, "mixer", "kv_heads"], 1),
                        (["layers", 0, "mlp", "router", "top"], 7), (["layers", 0, "mlp", "kind"], "glu"),
                        (["layers", 1, "mlp", "ff"], 0), (["norm", "eps"], 0.0), (["logit_softcap"], -1.0), (["layers"], [])):
        with pytest.raises(ConfigError):
            GofezenConfig.from_dict(_set(raw, path, value))
    for path in (["vocab"], ["norm"], ["max_positions"], ["layers", 0, "mixer", "left", "scale"],
                 ["layers", 0, "mixer", "right", "dim"], ["layers", 1, "mixer", "vdim"], ["layers", 0, "mlp", "expert"]):
        with pytest.raises(ConfigError):
            GofezenConfig.from_dict(_set(raw, path, delete=True))


def test_optional_keys_may_be_absent():
    raw = named_config("gofezen-tiny-a")
    for path in (["embedding"], ["logit_scale"], ["logit_softcap"], ["layers", 0, "mixer", "left_scale"],
                 ["layers", 0, "mlp", "shared"], ["layers", 3, "mixer", "left", "conv"], ["layers", 3, "mixer", "left", "mask"],
                 ["layers", 0, "mixer", "right", "conv"]):
        raw = _set(raw, path, delete=True)
    cfg, model = _model(raw)
    names = {w.name for w in model.weight_specs()}
    assert not any(n.startswith("l3.mix.left.") and n.endswith(".conv") for n in names) and "l0.mix.left.q.conv" in names
    assert "l0.mix.right.q.conv" not in names and "l3.mix.right.q.conv" in names
    assert [g.need.window for g in model.cache_layout().groups] == [24, None]
    assert (cfg.embedding_scale, cfg.logit_scale, cfg.logit_softcap) == (1.0, 1.0, 0.0)
    spec = model.spec
    assert spec.layers[0].mixer.params["left_scale"] == 1.0 and spec.layers[0].mixer.params["right_scale"] == 0.8
    names = {w.name for w in model.weight_specs()}
    assert "l0.mlp.router" in names and not any(n.startswith("l0.mlp.shared") for n in names)


def test_spec_declares_the_tensors_by_name():
    _, model = _model("gofezen-tiny-a")
    shapes = {w.name: tuple(w.shape) for w in model.weight_specs()}
    for name, shape in {"embed": (173, 48), "pos": (300, 48), "head": (173, 48), "final.norm": (48,), "l0.norm1": (48,),
                        "l0.mix.left.q": (48, 48), "l0.mix.left.k.b": (24,), "l0.mix.left.v": (40, 48),
                        "l0.mix.left.v.conv": (40, 3), "l0.mix.left.talk": (4, 4), "l0.mix.left.o": (48, 80),
                        "l0.mix.right.q": (32, 48), "l0.mix.right.k.conv": (32, 4), "l0.mix.right.v": (48, 48),
                        "l0.mix.right.b": (4, 48), "l0.mix.right.a": (4, 48), "l0.mix.right.A_log": (4,),
                        "l0.mix.right.dt_bias": (4,), "l0.mix.right.norm": (12,), "l0.mix.right.g": (48, 48),
                        "l0.mix.right.o": (48, 48), "l0.mlp.router": (6, 48), "l0.mlp.e5.down": (48, 24),
                        "l0.mlp.shared.gate": (16, 48), "l0.mlp.shared.sg": (1, 48), "l1.mix.q": (30, 48),
                        "l1.mix.f.b": (30,), "l1.mix.lower": (30,), "l1.mix.v": (42, 48), "l1.mix.norm": (14,),
                        "l1.mix.o": (48, 42), "l1.mlp.gate": (64, 48), "l1.mlp.down": (48, 64),
                        "l3.mix.right.v.conv": (84, 1)}.items():
        assert shapes[name] == shape, name
    assert not any(n.startswith(("l2.mlp", "l0.norm2", "l3.mlp.shared")) for n in shapes)
    tensors = random_tensors(model, seed=1, store_dtype=torch.bfloat16)
    low = tensors["l1.mix.lower"].float()
    assert float(low.min()) >= 0.0 and float(low.max()) < 1.0


def test_cache_layout_pages_and_state_slots():
    _, model = _model("gofezen-tiny-a")
    layout = model.cache_layout()
    # two attention layers of unlike rows and windows: two page groups; every layer keeps state
    assert [(g.need.head_dim, g.need.window, g.entries) for g in layout.groups] == [(2 * 12 + 2 * 20, 24, [0]),
                                                                                    (3 * 8 + 3 * 8, 37, [3])]
    assert sorted(layout.entry_state) == [0, 1, 2, 3]
    left = 2 * (48 + 24 + 40)                               # two carried rows of q, k, v
    right = -(-3 * (32 + 32 + 48) // 4) * 4 + ops.gated_memory_state_floats(4, 16, 12)
    assert layout.entry_state[0].shape == (-(-left // 4) * 4 + right,)
    assert layout.entry_state[1].shape == (ops.gated_memory_state_floats(3, 10, 14),)
    # one tap on the right of the last layer: nothing carried there
    assert layout.entry_state[3].shape == (1 * (48 + 24 + 24) + ops.gated_memory_state_floats(3, 20, 28),)


def _weights(name, seed=1):
    raw = named_config(name)
    _, model = _model(raw)
    w = {k: v.float() for k, v in random_tensors(model, seed=seed, store_dtype=torch.bfloat16).items()}
    for k in w:             # lively: matrices of order 1 / sqrt(inputs)
        if w[k].dim() == 2 and not k.endswith((".conv", ".talk")) and k not in ("embed", "pos"):
            w[k] = w[k] * (16.0 / w[k].shape[1] ** 0.5)
    return raw, w


def test_plain_prefixes_do_not_depend_on_what_follows():
    raw, w = _weights("gofezen-tiny-a")
    toks = [(7 * i + 3) % 173 for i in range(40)]
    full = pg.forward(raw, w, toks)
    assert torch.allclose(pg.forward(raw, w, toks[:17]), full[:17], atol=1e-9)
    changed = list(toks)
    changed[30] = (changed[30] + 1) % 173
    other = pg.forward(raw, w, changed)
    assert torch.allclose(other[:30], full[:30], atol=1e-9) and not torch.allclose(other[30:], full[30:], atol=1e-6)


def test_plain_window_edge_and_talking_heads():
    torch.manual_seed(0)
    T, H, G, d = 12, 4, 2, 6
    q, k = torch.randn(T, H, d, dtype=pg.F64), torch.randn(T, G, d, dtype=pg.F64)
    A = pg.window_softmax_weights(q, k, 0.4, 5)
    assert torch.allclose(A.sum(-1), torch.ones(H, T, dtype=pg.F64))
    assert float(A[:, 9, :5].abs().max()) == 0.0 and float(A[:, 9, 5].min()) > 0.0      # 9 sees 5 .. 9
    assert float(A[:, 3, 4:].abs().max()) == 0.0
    talk = torch.randn(H, H, dtype=pg.F64)
    B = pg.talking_heads(A, talk)
    assert torch.allclose(B[1], sum(talk[1, g] * A[g] for g in range(H)))
    assert torch.allclose(pg.talking_heads(A, torch.eye(H, dtype=pg.F64)), A)


def test_plain_delta_rule_equals_its_matrix_form():
    """S <- g S; S <- S + beta k (v - S^T k)^T is S <- g (I - beta k k^T) S + beta k v^T."""
    torch.manual_seed(1)
    T, H, d, dv = 9, 2, 5, 3
    q, k, v = (torch.randn(T, H, n, dtype=pg.F64) for n in (d, d, dv))
    k = pg.unit(k)
    beta, g = torch.rand(T, H, dtype=pg.F64), torch.rand(T, H, dtype=pg.F64)
    out = pg.delta_rule(q, k, v, beta, g)
    S = torch.zeros(H, d, dv, dtype=pg.F64)
    for t in range(T):
        for h in range(H):
            kk = k[t, h]
            S[h] = g[t, h] * (torch.eye(d, dtype=pg.F64) - beta[t, h] * torch.outer(kk, kk)) @ S[h] + \
                beta[t, h] * torch.outer(kk, v[t, h])
            assert torch.allclose(out[t, h], S[h].T @ q[t, h], atol=1e-12)
    # beta = 1 and g = 1: what is read back with the key just written is the value itself
    one = torch.ones(T, H, dtype=pg.F64)
    back = pg.delta_rule(k, k, v, one, one)
    assert torch.allclose(back, v * (k * k).sum(-1, keepdim=True), atol=1e-9)


def test_plain_forget_gate_bounds_and_experts_on_scaled_input():
    torch.manual_seed(2)
    T, H, d, dv = 7, 2, 4, 3
    q, v = torch.randn(T, H, d, dtype=pg.F64), torch.randn(T, H, dv, dtype=pg.F64)
    ones = torch.ones(T, H, d, dtype=pg.F64)
    assert float(pg.forget_gate_memory(q, ones, v).abs().max()) == 0.0                  # f = 1: nothing is ever written
    last = pg.forget_gate_memory(q, 0 * ones, v)                                        # f = 0: only the current token
    assert torch.allclose(last, v * q.sum(-1, keepdim=True))
    Hd, F, E = 6, 5, 4
    W = {"m.router": torch.randn(E, Hd, dtype=pg.F64)}
    for e in range(E):
        W[f"m.e{e}.gate"], W[f"m.e{e}.up"], W[f"m.e{e}.down"] = (torch.randn(F, Hd, dtype=pg.F64), torch.randn(F, Hd, dtype=pg.F64),
                                                                    torch.randn(Hd, F, dtype=pg.F64))
    h = torch.randn(3, Hd, dtype=pg.F64)
    f = {"router": {"experts": E, "top": 2}}
    out = pg.routed_experts(h, W, "m.", f)
    s = torch.sigmoid(h @ W["m.router"].T)
    for t in range(3):
        best = sorted(range(E), key=lambda e: -float(s[t, e]))[:2]
        ref = sum(pg.glu((s[t, e] * h[t])[None], W, f"m.e{e}.")[0] for e in best)
        assert torch.allclose(out[t], ref, atol=1e-12)
        # the weight on the input is not the weight on the output
        assert not torch.allclose(out[t], sum(s[t, e] * pg.glu(h[t][None], W, f"m.e{e}.")[0] for e in best), atol=1e-6)
