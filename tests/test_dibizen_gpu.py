"""Dibizen on the GPU against the plain restatement (tests/plain_dibizen.py, float64 on the CPU).

Small configurations of its own (three named ones and a few made on the spot, differing in every size: one, two, three
and four residual streams, one key head / several / one per query head, dim != vdim, with and without a query
temperature, a logit cap, groups or identity outputs, 1 to 5 convolution taps, a step-size rank of 1, layers that read
another layer's keys once and twice, layers without feed-forward) and random weights. Mechanisms alone (kernels against
the plain functions), then the whole model through the trace replay under every cut (whole, tail decoded one by one,
portions down to two tokens, mixed batches over a pool with no spare page and as many state slots as live requests),
far keys, temperature steps and carried state made visible by sharpened weights, long decoding, and greedy generation
through the engine's own entry point.
"""

from __future__ import annotations

import copy
import io
import json
import random
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_dibizen as pd
from replay_util import (check_against_plain, make_requests, mixed_steps, portion_steps, run_trace, tail_decode_steps,
                         whole_steps)

pytestmark = pytest.mark.gpu

SIZES = ["dibizen-tiny-a", "dibizen-tiny-b", "dibizen-tiny-c"]
LENGTHS = [70, 133, 45, 200, 96, 61]
DEV = "cuda:0"


def _read(folder):
    from safetensors import safe_open
    w = {}
    with safe_open(str(Path(folder) / "model.safetensors"), "pt") as f:
        for k in f.keys():
            w[k] = f.get_tensor(k).float()
    return json.loads((Path(folder) / "config.json").read_text()), w


def _write(folder, config, tensors):
    from safetensors.torch import save_file
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config))
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder


def _logits(cfg, w, toks):
    return pd.forward(cfg, w, toks).float()


def _lively(folder):
    """The random writer draws matrices for wide layers; at these widths the activations would stay far below one and
    every tanh, softmax and router would work in its linear range. Scale the tensors so that they do not: embedding rows
    of order one, matrices of order 1 / sqrt(inputs), logits of order one."""
    cfg, w = _read(folder)
    for k in list(w):
        if k in ("embed", "pos"):
            w[k] = w[k] * (40.0 if k == "embed" else 20.0)
        elif w[k].dim() == 2 and ".hc" not in k and not k.endswith((".router", ".conv", ".dt", ".A_log")):
            w[k] = w[k] * (0.8 / (0.05 if k != "head" else 0.02) / w[k].shape[1] ** 0.5)
    return _write(Path(folder), cfg, w)


@pytest.fixture(scope="session")
def dibizen_dirs(tmp_path_factory):
    from tokenmill_b200.weights import named_config, write_random_model
    return {n: _lively(write_random_model(tmp_path_factory.mktemp(n.replace("-", "_")), named_config(n), seed=3 + i))
            for i, n in enumerate(SIZES)}


@pytest.fixture(scope="session")
def plain_memo():
    return {}


def _plain(folder, reqs, memo):
    cfg, w = None, None
    out = {}
    for rid, toks in reqs.items():
        key = (str(folder), tuple(toks))
        if key not in memo:
            if cfg is None:
                cfg, w = _read(folder)
            memo[key] = _logits(cfg, w, toks)
        out[rid] = memo[key]
    return out


def _check(steps, outputs, reqs, plain, dtype):
    """float32: every row within 2e-4 of the largest logit. bfloat16: a router score computed from rounded inputs may
    choose another expert where two nearly tie, which moves that token's logits (and, through keys and states, later
    ones) by any amount in models this small; so up to eight rows in a hundred may lie outside 3 %. (The 32-bit run, where
    every row is held, is the exact test; this one shows that the bfloat16 kernels compute the same thing.)"""
    if dtype == "float32":
        return check_against_plain(steps, outputs, reqs, plain, dtype)
    fed = {rid: 0 for rid in reqs}
    over = total = 0
    for s in steps:
        row = 0
        for e in s["entries"]:
            for wpos in e["want"]:
                ref = plain[e["id"]][fed[e["id"]] + wpos]
                diff = float((torch.from_numpy(outputs[s["step"]][row]) - ref).abs().max())
                over += diff > 3e-2 * float(ref.abs().max())
                total += 1
                row += 1
            fed[e["id"]] += len(e["tokens"])
    assert over <= 0.08 * total, f"{over} of {total} rows differ by more than bfloat16 rounding"


def _steps(mode, reqs):
    if mode == "whole":
        return whole_steps(reqs)
    if mode == "tail":
        return tail_decode_steps(reqs)
    if mode == "portions":
        return portion_steps(reqs, seed=5)
    return mixed_steps(reqs, seed=7)


def _t(a, dtype=np.int32):
    return torch.as_tensor(np.asarray(a, dtype=dtype), device=DEV)


def _step_arrays(q_lens, slots):
    cu = np.zeros(len(q_lens) + 1, dtype=np.int32)
    cu[1:] = np.cumsum(q_lens)
    return _t(cu), _t(np.repeat(np.arange(len(q_lens)), q_lens)), _t(slots)


def _close(got, ref, dtype, what=""):
    tol = (2e-5 if dtype == torch.float32 else 1.2e-2) * max(1.0, float(ref.abs().max()))
    worst = float((got.detach().cpu().double() - ref.double()).abs().max())
    assert worst <= tol, (what, worst, tol)


# --- mechanisms alone -------------------------------------------------------------------------------------------

@pytest.mark.parametrize("streams,width", [(1, 52), (2, 52), (3, 52), (4, 52), (5, 52), (2, 50), (4, 1030), (6, 37)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_stream_norm_kernel(dtype, streams, width):
    """Start from embedding rows and position vectors, take in a result of two pieces through a mix, read through the
    read weights, and at the end norm the plain sum of a few rows without touching the residual. Up to four streams of a
    width that is a multiple of four take four numbers per access; the rest one."""
    from tokenmill_b200.kernels import ops
    torch.manual_seed(streams)
    T, H, S = 9, width, streams
    table, pos = torch.randn(30, H).to(dtype), torch.randn(40, H).to(dtype)
    ids, positions = torch.randint(0, 30, (T,)), torch.randint(0, 40, (T,))
    w, b, alpha = 1 + 0.1 * torch.randn(H), 0.1 * torch.randn(H), torch.tensor([0.7])
    in_w, out_w, mix = torch.randn(S), torch.randn(S), torch.randn(S, S)
    resid = torch.full((T, S * H), 7.0, device=DEV)
    out = torch.empty(T, H, dtype=dtype, device=DEV)
    g = lambda x: x.to(DEV)
    ops.stream_norm(resid, S, out, kind="dyt", weight=g(w), bias=g(b), alpha=g(alpha), ids=g(ids).int(), table=g(table),
                    positions=g(positions).int(), pos_table=g(pos), in_w=g(in_w))
    x0 = table[ids].double() + pos[positions].double()
    xs = [x0.clone() for _ in range(S)]
    _close(resid.view(T, S, H)[:, S - 1], xs[-1], torch.float32, "start")
    _close(out.float(), pd.dynamic_tanh(pd.stream_read(xs, in_w.double()), w.double(), b.double(), 0.7), dtype, "first read")
    y1, y2, rs = torch.randn(T, H).to(dtype), torch.randn(T, H).to(dtype), torch.rand(T, 3)
    ops.stream_norm(resid, S, out, kind="dyt", weight=g(w), bias=g(b), alpha=g(alpha), branch=g(y1), branch2=g(y2),
                    row_scale=g(rs)[:, 1], mix=g(mix), out_w=g(out_w), in_w=g(in_w))
    xs = pd.stream_write(xs, y1.double() + rs[:, 1:2].double() * y2.double(), mix.double(), out_w.double())
    for s in range(S):
        _close(resid.view(T, S, H)[:, s], xs[s], torch.float32, f"stream {s}")
    _close(out.float(), pd.dynamic_tanh(pd.stream_read(xs, in_w.double()), w.double(), b.double(), 0.7), dtype, "second read")
    before = resid.clone()
    rows = torch.tensor([5, 0, 8])
    last = torch.empty(3, H, dtype=dtype, device=DEV)
    ops.stream_norm(resid, S, last, kind="dyt", weight=g(w), bias=g(b), alpha=g(alpha), branch=g(y2), mix=g(mix), out_w=g(out_w),
                    rows=g(rows).int())
    xs = pd.stream_write(xs, y2.double(), mix.double(), out_w.double())
    _close(last.float(), pd.dynamic_tanh(sum(xs), w.double(), b.double(), 0.7)[rows], dtype, "last")
    assert torch.equal(before, resid)
    rms = torch.empty(3, H, dtype=dtype, device=DEV)
    ops.stream_norm(resid, S, rms, kind="rms", weight=g(w), eps=1e-5, branch=g(y2), mix=g(mix), out_w=g(out_w), rows=g(rows).int())
    _close(rms.float(), (pd.rms(sum(xs), 1e-5) * w.double())[rows], dtype, "rms")


@pytest.mark.parametrize("inner,N,rank,taps", [(72, 12, 5, 3), (100, 20, 7, 2), (96, 80, 1, 5), (40, 200, 4, 4), (33, 1, 2, 1)])
@pytest.mark.parametrize("slice_len", [0, 5, 16])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_convolution_and_selective_scan_under_cuts(dtype, inner, N, rank, taps, slice_len):
    """Two requests (slots 2 and 0 of 4) fed in steps of unequal sizes, single tokens among them: the convolution's
    carried inputs and the scan's states against the plain functions over the whole sequences. With a slice length the
    scan runs its three passes over time slices (one request's last slice short, the other's slices fewer)."""
    from tokenmill_b200.kernels import ops
    torch.manual_seed(inner)
    n = 45
    q = lambda x: x.to(dtype).float()
    w_conv, b_conv = 0.4 * torch.randn(inner, taps), 0.1 * torch.randn(inner)
    w_x = q(0.15 * torch.randn(rank + 2 * N, inner))
    w_dt, b_dt = 0.4 * torch.randn(inner, rank), torch.randn(inner) - 1
    A_log, D = 0.5 * torch.randn(inner, N) - 1, 1 + 0.2 * torch.randn(inner)
    seqs = [q(torch.randn(n, 3 + 2 * inner)), q(torch.randn(n, 3 + 2 * inner))]
    want = []
    for s in seqs:
        p = s.double()[:, 3:]
        x = q(pd.silu(pd.causal_conv(p[:, :inner], w_conv.double(), b_conv.double()))).double()   # (the engine rounds x here)
        dbc = x @ w_x.double().T
        dt = torch.nn.functional.softplus(dbc[:, :rank] @ w_dt.double().T + b_dt.double())
        y = pd.selective_scan(x, dt, -torch.exp(A_log.double()), dbc[:, rank:rank + N], dbc[:, rank + N:], D.double())
        want.append(y * pd.silu(p[:, inner:]))
    conv_len = (taps - 1) * inner
    state = torch.zeros(4, conv_len + inner * N + 6, device=DEV)
    g = lambda x: x.to(DEV)
    fed = [0, 0]
    for na, nb in ((1, 17), (20, 1), (3, 1), (1, 4), (20, 22)):      # (walks of fewer than four tokens compute their step sizes another way)
        rows = torch.cat([seqs[0][fed[0]:fed[0] + na], seqs[1][fed[1]:fed[1] + nb]]).to(dtype).to(DEV)[:, 3:].contiguous()
        cu, seq_of, slots = _step_arrays([na, nb], [2, 0])
        xc = torch.empty(na + nb, inner, dtype=dtype, device=DEV)
        ops.conv_silu_state(rows, 0, inner, g(w_conv), g(b_conv), state, cu, seq_of, slots, xc)
        dbc = ops.linear32(xc, g(w_x).to(dtype))
        out = torch.empty(na + nb, inner, dtype=dtype, device=DEV)
        sliced = {}
        if slice_len:
            slices = -(-max(na, nb) // slice_len)
            sliced = dict(max_q_len=max(na, nb), slice_len=slice_len,
                          slice_S=torch.full((2 * slices * inner * N,), float("nan"), device=DEV),
                          slice_dt=torch.full((2 * slices * inner,), float("nan"), device=DEV))
        ops.selective_scan(xc, rows, inner, dbc, g(w_dt), g(b_dt), g(A_log), g(D), state, conv_len, cu, slots, out,
                           n_seqs=2, rank=rank, N=N, **sliced)
        ref = torch.cat([want[0][fed[0]:fed[0] + na], want[1][fed[1]:fed[1] + nb]])
        _close(out.float(), ref, dtype, (fed, na, nb))
        fed = [fed[0] + na, fed[1] + nb]
    assert float(state[1].abs().max()) == 0.0 and float(state[3].abs().max()) == 0.0
    assert float(state[:, conv_len + inner * N:].abs().max()) == 0.0


@pytest.mark.parametrize("slice_len", [0, 5, 16])
@pytest.mark.parametrize("heads,d,dv", [(3, 10, 14), (1, 40, 72), (2, 64, 130), (2, 200, 24), (5, 1, 3), (2, 300, 8)])
def test_decay_memory_kernel_under_cuts(heads, d, dv, slice_len):
    """Per head S <- decay S + k v^T, o = S^T q, with silu on q, k and v, from strided 32-bit rows; slots 1 and 3 of 4.
    With a slice length the three passes over time slices run instead of one walk."""
    from tokenmill_b200.kernels import ops
    torch.manual_seed(d)
    n = 40
    P = 2 * heads * d + heads * dv
    col = {"q": 0, "k": heads * d, "v": 2 * heads * d}
    decay = torch.tensor([0.999, 0.5, 0.9, 0.97, 1.0][:heads])
    seqs = [torch.randn(n, P + 5), torch.randn(n, P + 5)]
    want = []
    for s in seqs:
        p = pd.silu(s.double()[:, 5:])
        want.append(pd.decay_memory(p[:, :heads * d].view(n, heads, d), p[:, col["k"]:col["v"]].view(n, heads, d),
                                    p[:, col["v"]:].reshape(n, heads, dv), [float(a) for a in decay]).reshape(n, heads * dv))
    floats = ops.decay_memory_state_floats(heads, d, dv)
    state = torch.zeros(4, 8 + floats, device=DEV)
    fed = [0, 0]
    for na, nb in ((1, 17), (20, 1), (2, 1), (17, 21)):
        rows = torch.cat([seqs[0][fed[0]:fed[0] + na], seqs[1][fed[1]:fed[1] + nb]]).to(DEV)
        cu, _, slots = _step_arrays([na, nb], [1, 3])
        y = torch.empty(na + nb, heads * dv, device=DEV)
        sliced = {}
        if slice_len:
            slices = -(-max(na, nb) // slice_len)
            sliced = dict(max_q_len=max(na, nb), slice_len=slice_len,
                          slice_S=torch.full((2 * slices * floats,), float("nan"), device=DEV))
        ops.decay_memory(rows[:, 5:], q_col=col["q"], k_col=col["k"], v_col=col["v"], activation="silu", decay=decay.to(DEV),
                         state=state, state_off=8, cu_q=cu, state_slots=slots, y=y, n_seqs=2, heads=heads, dim=d, vdim=dv,
                         **sliced)
        ref = torch.cat([want[0][fed[0]:fed[0] + na], want[1][fed[1]:fed[1] + nb]])
        _close(y, ref, torch.float32, (fed, na, nb))
        fed = [fed[0] + na, fed[1] + nb]
    assert float(state[0].abs().max()) == 0.0 and float(state[:, :8].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dv", [(1, 600), (2, 512), (1, 1030)])
def test_norm_and_gate_over_wide_heads(heads, dv, dtype):
    """Heads normed together are one head of many numbers: a block per row then, with a sum over its warps."""
    from tokenmill_b200.kernels import ops
    torch.manual_seed(dv)
    n = 9
    y, wide, w = torch.randn(n, heads * dv) * 4, torch.randn(n, heads * dv + 4), torch.randn(heads * dv)
    out = ops.head_norm_gate(y.to(DEV), wide.to(DEV)[:, 4:], w.to(DEV), 1e-5, heads,
                             torch.empty(n, heads * dv, dtype=dtype, device=DEV))
    yd = y.double().view(n, heads, dv)
    ref = (yd / (yd.pow(2).mean(-1, keepdim=True) + 1e-5).sqrt()).reshape(n, -1) * w.double() * torch.sigmoid(wide.double()[:, 4:])
    _close(out.float(), ref, dtype, (heads, dv))


@pytest.mark.parametrize("experts,identity,top,groups,keep", [(6, 2, 2, 4, 2), (5, 1, 3, 2, 2), (4, 0, 1, 1, 1), (8, 0, 2, 4, 1),
                                                              (2, 2, 1, 2, 1), (13, 3, 4, 8, 3), (3, 0, 3, 1, 1)])
def test_choice_among_groups_kernel(experts, identity, top, groups, keep):
    """The router's choice against the plain one: same outputs chosen, same weights; a correction far below zero makes
    every choice score negative (an output outside the kept groups must still lose to them)."""
    from tokenmill_b200.kernels import ops
    torch.manual_seed(experts)
    n, T = experts + identity, 200
    for shift in (0.0, -3.0):
        logits = 2 * torch.randn(T, n)
        corr = 0.3 * torch.randn(n) + shift
        r = {"experts": experts, "identity": identity, "top": top, "groups": {"count": groups, "keep": keep}}
        W = {"r.router": torch.eye(n).double(), "r.correction": corr.double()}
        idx, w = pd.route(logits.double(), W, "r.", r)
        got_idx, got_w, dense, id_w = ops.moe_choose(logits.to(DEV), corr.to(DEV), top, groups, keep, identity)
        ref_dense = torch.zeros(T, n, dtype=torch.float64).scatter_(1, idx, w)
        assert torch.equal(got_idx.cpu().long().sort(1).values, idx.sort(1).values)
        _close(dense, ref_dense, torch.float32, "dense weights")
        _close(torch.zeros(T, n, device=DEV).scatter_(1, got_idx.long(), got_w), ref_dense, torch.float32, "chosen weights")
        _close(id_w, ref_dense[:, experts:].sum(1), torch.float32, "identity weight")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_experts_part_against_plain(dtype):
    """The feed-forward part as the block calls it: the experts' weighted sum and the identity outputs' share."""
    from tokenmill_b200.parts.routed import ChoiceRoutedExperts
    torch.manual_seed(2)
    H, F, E, ident = 40, 24, 5, 3
    part = ChoiceRoutedExperts(hidden_size=H, expert_size=F, num_experts=E, top=3, identity=ident, groups=4, keep=2,
                               dtype=dtype, device=torch.device(DEV))
    q = lambda x: x.to(torch.bfloat16).double()
    W = {"m.router": q(0.5 * torch.randn(E + ident, H)), "m.correction": q(0.1 * torch.randn(E + ident))}
    for e in range(E):
        W[f"m.e{e}.up"], W[f"m.e{e}.down"] = q(0.2 * torch.randn(F, H)), q(0.2 * torch.randn(H, F))
    part.bind({s.name: W["m." + s.name].to(torch.float32 if s.dtype == "float32" else dtype).to(DEV) for s in part.weight_specs()})
    h = q(torch.randn(50, H))
    f = {"router": {"experts": E, "identity": ident, "top": 3, "groups": {"count": 4, "keep": 2}}}
    _close(part.forward(h.to(dtype).to(DEV)).float(), pd.experts(h, W, "m.", f), dtype)


def test_softcap_kernel():
    from tokenmill_b200.kernels import ops
    x = torch.linspace(-90, 90, 1001)
    _close(ops.softcap_(x.to(DEV).clone(), 30.0), 30.0 * torch.tanh(x.double() / 30.0), torch.float32)


# --- the whole model under every cut ----------------------------------------------------------------------------

@pytest.mark.parametrize("size", SIZES)
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_against_plain(dibizen_dirs, plain_memo, size, mode, dtype, tmp_path):
    folder = dibizen_dirs[size]
    vocab = json.loads((folder / "config.json").read_text())["vocab"]
    reqs = make_requests(vocab, LENGTHS, seed=11)
    steps, max_tokens = _steps(mode, reqs)
    outputs = run_trace(folder, dtype, steps, max_tokens, tmp_path / "out")
    _check(steps, outputs, reqs, _plain(folder, reqs, plain_memo), dtype)


@pytest.mark.parametrize("page", [8, 32])
def test_replay_at_other_page_sizes(dibizen_dirs, plain_memo, page, tmp_path):
    folder = dibizen_dirs["dibizen-tiny-a"]
    reqs = make_requests(173, LENGTHS, seed=13)
    steps, max_tokens = mixed_steps(reqs, seed=9)
    outputs = run_trace(folder, "float32", steps, max_tokens, tmp_path / "out", page_size=page)
    check_against_plain(steps, outputs, reqs, _plain(folder, reqs, plain_memo), "float32")


def test_cuts_do_not_move_the_logits_in_float32(dibizen_dirs, tmp_path):
    """Whole prompts against mixed batches of portions and single tokens: every sum walks keys and tokens in the same
    order whatever the cut, so in 32-bit the rows agree to a few units in the last place."""
    folder = dibizen_dirs["dibizen-tiny-a"]
    reqs = make_requests(173, LENGTHS, seed=21)
    rows = {}
    for mode in ("whole", "mixed", "portions"):
        steps, max_tokens = _steps(mode, reqs)
        outputs = run_trace(folder, "float32", steps, max_tokens, tmp_path / mode)
        fed = {r: 0 for r in reqs}
        for s in steps:
            row = 0
            for e in s["entries"]:
                for wpos in e["want"]:
                    rows.setdefault(mode, {})[(e["id"], fed[e["id"]] + wpos)] = outputs[s["step"]][row]
                    row += 1
                fed[e["id"]] += len(e["tokens"])
    scale = max(float(np.abs(v).max()) for v in rows["whole"].values())
    for mode in ("mixed", "portions"):
        worst = max(float(np.abs(rows[mode][k] - rows["whole"][k]).max()) for k in rows["whole"])
        assert worst <= 4e-6 * scale, (mode, worst)


# --- faults that random weights would hide ----------------------------------------------------------------------

def _sharpen(src, dst, *, attention=1.0, slow=False, edit=None):
    """A copy of a model whose attention is sharp (query weights scaled up, so that single keys carry the softmax and a
    lost or doubled key, a wrong temperature step or another layer's keys show) and, with ``slow``, whose recurrent
    layers forget slowly (decays close to one, small step sizes: a lost or stale state shows hundreds of tokens later)."""
    cfg, w = _read(src)
    for i, layer in enumerate(cfg["layers"]):
        if layer["type"] == "attention":
            w[f"l{i}.mix.q"] = w[f"l{i}.mix.q"] * attention
        if slow and layer["type"] == "lightning":
            layer["mixer"]["decay"] = [1.0 - 0.004 / (j + 1) for j in range(layer["mixer"]["heads"])]
        if slow and layer["type"] == "mamba1":
            w[f"l{i}.mix.A_log"] = torch.full_like(w[f"l{i}.mix.A_log"], -4.0)
            w[f"l{i}.mix.dt.b"] = torch.full_like(w[f"l{i}.mix.dt.b"], -2.0)
    if edit is not None:
        edit(cfg, w)
    w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}          # what the file will hold
    return _write(dst, cfg, w), cfg, w


def test_temperature_steps_far_keys_and_borrowed_keys(dibizen_dirs, tmp_path):
    """Sharp attention over 230 and 150 tokens with a temperature that steps every 16 positions. On the plain model,
    an interval one longer or shorter, a layer reading its OWN keys' layer wrongly (the borrowed keys swapped for
    zeros), or a dropped first key each move many rows by far more than the tolerance; the engine agrees with the true
    one in prompts, in decoded tokens (60 of them, across two steps of the temperature) and across page borders."""
    folder, cfg, w = _sharpen(dibizen_dirs["dibizen-tiny-a"], tmp_path / "sharp", attention=6.0)
    reqs = make_requests(cfg["vocab"], [230, 150], seed=31)
    plain = {r: _logits(cfg, w, t) for r, t in reqs.items()}
    tol = 2e-4 * float(plain["r0"].abs().max())
    for d in (-1, 1):
        other = copy.deepcopy(cfg)
        for layer in other["layers"]:
            if layer["type"] == "attention":
                layer["mixer"]["q_temp"]["every"] += d
        moved = ((_logits(other, w, reqs["r0"]) - plain["r0"]).abs().amax(dim=1) > 10 * tol).float()[40:].mean()
        assert moved > 0.3, (d, float(moved))
    own = copy.deepcopy(cfg)
    del own["layers"][3]["mixer"]["kv_from"]
    w_own = dict(w)
    w_own["l3.mix.k"], w_own["l3.mix.v"] = torch.zeros_like(w["l0.mix.k"]), torch.zeros_like(w["l0.mix.v"])
    assert ((_logits(own, w_own, reqs["r0"]) - plain["r0"]).abs().amax(dim=1) > 10 * tol).float().mean() > 0.5
    changed = list(reqs["r0"])
    changed[0] = (changed[0] + 1) % cfg["vocab"]
    assert (_logits(cfg, w, changed)[-1] - plain["r0"][-1]).abs().max() > 10 * tol       # the first key is still read
    for mode in ("whole", "tail", "portions", "mixed"):
        steps, max_tokens = _steps(mode, reqs) if mode != "tail" else tail_decode_steps(reqs, tail=60)
        outputs = run_trace(folder, "float32", steps, max_tokens, tmp_path / mode)
        check_against_plain(steps, outputs, reqs, plain, "float32")


@pytest.mark.parametrize("size", ["dibizen-tiny-b", "dibizen-tiny-c"])
def test_an_old_state_shows(dibizen_dirs, size, tmp_path):
    """Recurrent layers that forget slowly: changing the second token of a 340-token request still moves its last logits
    (checked on the plain model), so state carried over many steps, long decoding (120 tokens) and slots are looked at."""
    folder, cfg, w = _sharpen(dibizen_dirs[size], tmp_path / "slow", attention=3.0, slow=True)
    reqs = make_requests(cfg["vocab"], [340, 310], seed=41)
    plain = {r: _logits(cfg, w, t) for r, t in reqs.items()}
    tol = 2e-4 * float(plain["r0"].abs().max())
    changed = list(reqs["r0"])
    changed[1] = (changed[1] + 1) % cfg["vocab"]
    assert (_logits(cfg, w, changed)[-1] - plain["r0"][-1]).abs().max() > 10 * tol
    for mode in ("whole", "tail", "mixed"):
        steps, max_tokens = tail_decode_steps(reqs, tail=120) if mode == "tail" else _steps(mode, reqs) if mode == "whole" \
            else mixed_steps(reqs, seed=3)
        outputs = run_trace(folder, "float32", steps, max_tokens, tmp_path / mode)
        check_against_plain(steps, outputs, reqs, plain, "float32")


def test_identity_outputs_and_groups_decide(dibizen_dirs, tmp_path):
    """One group of four kept, two outputs chosen: both come from the best group, which the plain model with the groups
    ignored gets wrong at many rows; the engine agrees with the true one. (A correction far below zero: every choice
    score is negative, and an output outside the kept group still loses.)"""
    def edit(cfg, w):
        cfg["layers"][0]["mlp"]["router"]["groups"]["keep"] = 1
        for i, layer in enumerate(cfg["layers"]):
            if layer.get("mlp") is not None:
                w[f"l{i}.mlp.correction"] = w[f"l{i}.mlp.correction"] - 2.0
    folder, cfg, w = _sharpen(dibizen_dirs["dibizen-tiny-a"], tmp_path / "neg", edit=edit)
    reqs = make_requests(cfg["vocab"], [90, 64], seed=43)
    plain = {r: _logits(cfg, w, t) for r, t in reqs.items()}
    tol = 2e-4 * float(plain["r0"].abs().max())
    flat = copy.deepcopy(cfg)
    for layer in flat["layers"]:
        if layer.get("mlp") is not None and layer["mlp"]["router"].get("groups"):
            del layer["mlp"]["router"]["groups"]
    assert ((_logits(flat, w, reqs["r0"]) - plain["r0"]).abs().amax(dim=1) > 10 * tol).float().mean() > 0.3
    for mode in ("whole", "mixed"):
        steps, max_tokens = _steps(mode, reqs)
        check_against_plain(steps, run_trace(folder, "float32", steps, max_tokens, tmp_path / mode), reqs, plain, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_of_unlike_sizes(dtype, tmp_path):
    """Layers that share no size, in another order: two attention owners with different heads (two page groups), each
    read by a later layer; four streams; a step-size rank of 1 and a single tap; one state per channel; groups of one
    output; prompts of 300 and 270 tokens whole and in mixed batches, then decoded."""
    from tokenmill_b200.weights import write_random_model
    from tokenmill_b200.weights.random_init import (dibizen_attention as A, dibizen_config, dibizen_lightning as L,
                                                    dibizen_mamba as M, dibizen_moe as E)
    a1 = dict(heads=10, kv_heads=5, dim=12, vdim=20, scale=0.25, q_temp=(0.3, 7))
    a2 = dict(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.125)
    cfg = dibizen_config(vocab=157, width=72, streams=4, eps=1e-6, max_positions=320, logit_softcap=12.0, layers=[
        ("lightning", L(heads=1, dim=96, vdim=16, decay=[0.98]), E(experts=4, top=2, ff=40, identity=0, groups=(4, 2))),
        ("attention", A(**a1), None),
        ("attention", A(**a2), E(experts=3, top=1, ff=88, identity=1, groups=(1, 1))),
        ("mamba1", M(inner=50, state=1, dt_rank=1, conv=1), E(experts=1, top=2, ff=16, identity=1)),
        ("attention", A(**a2, kv_from=2), None),
        ("attention", A(**a1, kv_from=1), E(experts=9, top=4, ff=8, identity=3, groups=(6, 3))),
        ("mamba1", M(inner=144, state=24, dt_rank=9, conv=4), None)])
    folder = _lively(write_random_model(tmp_path / "m", cfg, seed=12))
    _, w = _read(folder)
    reqs = make_requests(157, [300, 270], seed=71)
    plain = {r: _logits(cfg, w, t) for r, t in reqs.items()}
    for mode in ("whole", "tail", "mixed"):
        steps, max_tokens = _steps(mode, reqs)
        _check(steps, run_trace(folder, dtype, steps, max_tokens, tmp_path / mode), reqs, plain, dtype)


def test_slots_and_pages_used_again_start_clean(dibizen_dirs, plain_memo, tmp_path):
    """Nine requests through a pool for two live ones with two state slots: every slot and page is used several times,
    and a request that follows a long one on its slot gets the same logits as alone."""
    folder = dibizen_dirs["dibizen-tiny-a"]
    reqs = make_requests(173, [90, 30, 64, 12, 100, 5, 77, 48, 33], seed=51)
    steps, max_tokens = mixed_steps(reqs, seed=2, max_live=2)
    from tokenmill_b200.engine.trace import run
    out_dir = tmp_path / "out"
    stdin = io.StringIO("".join(json.dumps(s) + "\n" for s in steps))
    assert run(str(folder), "float32", str(out_dir), max_tokens, stdin=stdin, stdout=io.StringIO(), state_slots=2) == 0
    outputs = {s["step"]: np.fromfile(out_dir / f"{s['step']}.f32", dtype="<f4").reshape(-1, 173) for s in steps}
    check_against_plain(steps, outputs, reqs, _plain(folder, reqs, plain_memo), "float32")


def test_first_tokens_and_single_token_requests(dibizen_dirs, plain_memo, tmp_path):
    """Requests of one, two and three tokens (shorter than the convolution's carried inputs), fed whole and token by
    token, beside each other."""
    folder = dibizen_dirs["dibizen-tiny-c"]       # five taps
    reqs = make_requests(210, [1, 2, 3, 4, 6], seed=61)
    plain = _plain(folder, reqs, plain_memo)
    whole = [{"step": 0, "entries": [{"id": r, "tokens": t, "want": list(range(len(t)))} for r, t in list(reqs.items())[:4]],
              "end": list(reqs)[:4]}]
    check_against_plain(whole, run_trace(folder, "float32", whole, 256, tmp_path / "w"), reqs, plain, "float32")
    reqs4 = {r: t for r, t in reqs.items() if r != "r0"}
    steps = [{"step": p, "entries": [{"id": r, "tokens": [t[p]], "want": [0]} for r, t in reqs4.items() if p < len(t)],
              "end": [r for r, t in reqs4.items() if p == len(t) - 1]} for p in range(6)]
    check_against_plain(steps, run_trace(folder, "float32", steps, 256, tmp_path / "t"), reqs4, plain, "float32")


# --- through the engine's own entry point -----------------------------------------------------------------------

@pytest.mark.parametrize("size,graphs,chunked,dtype", [
    ("dibizen-tiny-a", False, False, "float32"), ("dibizen-tiny-a", True, True, "float32"),
    ("dibizen-tiny-b", False, True, "bfloat16"), ("dibizen-tiny-c", True, True, "bfloat16")])
def test_greedy_generation_through_the_engine(dibizen_dirs, size, graphs, chunked, dtype):
    """LLMEngine with its scheduler: admission (state slots, one page group that several layers read), chunked prompts
    beside decodes, decode graphs with padded rows, a pool so small that requests are evicted and recomputed. The
    logits behind every generated token equal the plain model's on the request's own history, and the token is their
    arg-max."""
    from tokenmill_b200 import EngineConfig
    from tokenmill_b200.engine import LLMEngine
    from tokenmill_b200.sampling import SamplingParams

    folder = dibizen_dirs[size]
    cfg, w = _read(folder)
    rng = random.Random(5)
    prompts = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (9, 30, 17, 44, 5, 26, 12)]
    owners = [l["mixer"] for l in cfg["layers"] if l["type"] == "attention" and l["mixer"].get("kv_from") is None]
    per_token = sum(a["kv_heads"] * (a["dim"] + a["vdim"]) for a in owners) * (4 if dtype == "float32" else 2)
    eng = LLMEngine(EngineConfig(model=str(folder), dtype=dtype, block_size=8, max_model_len=128, max_num_seqs=4,
                                 kv_cache_mb=(16 * 8 + (8 if graphs else 0) + 1) * per_token / 2 ** 20, watermark=0.0,
                                 cuda_graphs=graphs, cuda_graph_max_batch=4, enable_chunked_prefill=chunked,
                                 max_num_batched_tokens=24 if chunked else 256))
    assert eng.cache.state_slots.num_slots == 4 and len(eng.cache.num_pages) == 1
    rows: dict[str, list] = {}

    def tap(where, logits):
        cpu = logits.float().cpu()
        for (rid, pos), row in zip(where, cpu):
            rows.setdefault(rid, []).append((pos, row.clone()))

    eng.on_logits = tap
    reqs = [eng.add_request(f"t{i}", p, SamplingParams(max_tokens=24, ignore_eos=True)) for i, p in enumerate(prompts)]
    while eng.has_unfinished():
        eng.step()
    eng.drain()
    assert eng.cache.all_free
    if graphs:
        assert eng.runner.stats["graph_steps"] > 0
    compared = over = 0
    for i, (p, r) in enumerate(zip(prompts, reqs)):
        assert len(r.output_ids) == 24
        plain = _logits(cfg, w, p + r.output_ids)
        for pos, row in rows[f"t{i}"]:
            ref = plain[pos]
            diff = float((row - ref).abs().max())
            if dtype == "float32":
                assert diff <= 2e-4 * float(ref.abs().max()), (i, pos)
                assert int(row.argmax()) == r.output_ids[pos - len(p) + 1]
            else:
                over += diff > 3e-2 * float(ref.abs().max())
            compared += 1
    assert compared >= 7 * 24 and over <= 0.08 * compared


def test_generate_command_line_and_trace_runner(dibizen_dirs, tmp_path):
    """The two programs a user starts: ``python -m tokenmill_b200.generate`` on a Dibizen folder, and bin/trace_run."""
    root = Path(__file__).resolve().parents[1]
    folder = dibizen_dirs["dibizen-tiny-b"]
    res = subprocess.run([sys.executable, "-m", "tokenmill_b200.generate", "--model", str(folder), "--prompt-ids", "5,17,3,250",
                          "--max-tokens", "6", "--dtype", "float32", "--max-model-len", "64", "--kv-cache-mb", "1"],
                         cwd=root, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    out = json.loads(res.stdout.strip().splitlines()[-1])
    cfg, w = _read(folder)
    toks = [5, 17, 3, 250]
    for _ in range(6):
        toks.append(int(_logits(cfg, w, toks)[-1].argmax()))
    assert out["output_ids"] == toks[4:]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:7], "want": [0, 6]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[7:8], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[8:10], "want": [1]}], "end": ["a"]}]
    res = subprocess.run([str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", "bfloat16", "--out",
                          str(tmp_path / "o"), "--max-tokens", "64"], input="".join(json.dumps(s) + "\n" for s in steps),
                         cwd=root, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [l for l in res.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not (tmp_path / "o" / "1.f32").exists()
    plain = _logits(cfg, w, toks)
    got = np.fromfile(tmp_path / "o" / "0.f32", dtype="<f4").reshape(2, 300)
    last = np.fromfile(tmp_path / "o" / "2.f32", dtype="<f4").reshape(1, 300)
    for row, pos in ((got[0], 0), (got[1], 6), (last[0], 9)):
        assert np.abs(row - plain[pos].numpy()).max() <= 6e-2 * float(plain[pos].abs().max())
