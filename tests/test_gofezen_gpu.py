"""Gofezen on the GPU against the plain restatement (tests/plain_gofezen.py, float64 on the CPU).

Small configurations of its own (three named ones and a few made on the spot, differing in every size: one key head /
several / one per query head on both sides of a pair, dim != vdim, 1 to 5 convolution taps, windows shorter and longer
than the requests, top 1 to all experts, with and without a shared expert, a cap, scales, layers without feed-forward)
and random weights. Mechanisms alone (kernels against the plain functions), then the whole model through the trace
replay under every cut (whole, tail decoded one by one, portions down to two tokens, mixed batches over a pool with no
spare page and as many state slots as live requests), window edges, far keys and carried state made visible by
sharpened weights, long decoding, and greedy generation through the engine's own entry point.
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

import plain_gofezen as pg
from replay_util import (check_against_plain, make_requests, mixed_steps, portion_steps, run_trace, tail_decode_steps,
                         whole_steps)

pytestmark = pytest.mark.gpu

SIZES = ["gofezen-tiny-a", "gofezen-tiny-b", "gofezen-tiny-c"]
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
    return pg.forward(cfg, w, toks).float()


def _lively(folder):
    """The random writer draws matrices for wide layers; at these widths the activations would stay far below one and
    every softmax, gate and router would work in its linear range. Scale the matrices to order 1 / sqrt(inputs), the
    position vectors to order one."""
    cfg, w = _read(folder)
    for k in list(w):
        if k == "pos":
            w[k] = w[k] * 30.0
        elif k == "embed":
            w[k] = w[k] * (50.0 / cfg["embedding"]["scale"])
        elif w[k].dim() == 2 and not k.endswith((".conv", ".talk", ".router", ".sg")):
            w[k] = w[k] * (0.8 / (0.05 if k != "head" else 0.02) / w[k].shape[1] ** 0.5)
    return _write(Path(folder), cfg, w)


@pytest.fixture(scope="session")
def gofezen_dirs(tmp_path_factory):
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

@pytest.mark.parametrize("channels,taps", [(72, 3), (100, 2), (33, 5), (40, 1), (8, 4), (24, 7), (13, 16)])
@pytest.mark.parametrize("bias,act", [(True, None), (False, "silu")])
def test_short_convolution_carries_its_last_inputs(channels, taps, bias, act):
    """Two requests (slots 2 and 0 of 4) fed in steps of unequal sizes, single tokens and portions shorter than the
    carried inputs among them, from strided 32-bit rows; the carried inputs live 8 floats into the slot."""
    from tokenmill_b200.kernels import ops
    torch.manual_seed(channels)
    n = 45
    w, b = 0.5 * torch.randn(channels, taps), torch.randn(channels) if bias else None
    seqs = [torch.randn(n, channels + 4), torch.randn(n, channels + 4)]
    want = []
    for s in seqs:
        u = s.double()[:, 4:] + (b.double() if bias else 0.0)
        y = pg.causal_conv(u, w.double())
        want.append(pg.silu(y) if act else y)
    state = torch.zeros(4, 8 + (taps - 1) * channels + 3, device=DEV)
    fed = [0, 0]
    for na, nb in ((1, 17), (20, 1), (2, 1), (1, 3), (21, 23)):
        rows = torch.cat([seqs[0][fed[0]:fed[0] + na], seqs[1][fed[1]:fed[1] + nb]]).to(DEV)
        cu, seq_of, slots = _step_arrays([na, nb], [2, 0])
        out = torch.full((na + nb, channels + 2), float("nan"), device=DEV)
        ops.short_conv_state(rows, 4, w.to(DEV), b.to(DEV) if bias else None, state, 8, cu, seq_of, slots, out, out_col0=2,
                             activation=act)
        ref = torch.cat([want[0][fed[0]:fed[0] + na], want[1][fed[1]:fed[1] + nb]])
        _close(out[:, 2:], ref, torch.float32, (fed, na, nb))
        fed = [fed[0] + na, fed[1] + nb]
    assert float(state[1].abs().max()) == 0.0 and float(state[3].abs().max()) == 0.0
    assert float(state[:, :8].abs().max()) == 0.0 and float(state[:, 8 + (taps - 1) * channels:].abs().max()) == 0.0


def _memory_case(rule, heads, qk_heads, d, dv, n, seed):
    """Random rows [5 unused | q | k or f | v], (g, beta) per token and head, and the plain results."""
    torch.manual_seed(seed)
    qk = qk_heads * d
    rows = torch.randn(n, 5 + 2 * qk + heads * dv)
    gb = torch.rand(n, 2 * heads)
    gb[:, :heads] = 1.0 - 0.3 * gb[:, :heads] ** 2                      # decays from 0.7 to 1
    p = rows.double()[:, 5:]
    rep = heads // qk_heads
    if rule == "forget":
        rows[:, 5 + qk:5 + 2 * qk] = torch.rand(n, qk) ** 0.3           # the gates, in (0, 1)
        p = rows.double()[:, 5:]
        ref = pg.forget_gate_memory(p[:, :qk].view(n, heads, d), p[:, qk:2 * qk].view(n, heads, d), p[:, 2 * qk:].view(n, heads, dv))
    else:
        k = pg.unit(p[:, qk:2 * qk].view(n, qk_heads, d))
        rows[:, 5 + qk:5 + 2 * qk] = k.reshape(n, qk).float()
        k = rows.double()[:, 5 + qk:5 + 2 * qk].view(n, qk_heads, d).repeat_interleave(rep, dim=1)
        q = p[:, :qk].view(n, qk_heads, d).repeat_interleave(rep, dim=1)
        v = p[:, 2 * qk:].view(n, heads, dv)
        g, beta = gb.double()[:, :heads], gb.double()[:, heads:]
        if rule == "delta":
            ref = pg.delta_rule(q, k, v, beta, g)
        else:           # a decay per token and a plain write: the delta rule without its correction, written out
            S = torch.zeros(heads, d, dv, dtype=pg.F64)
            ref = torch.zeros(n, heads, dv, dtype=pg.F64)
            for t in range(n):
                for h in range(heads):
                    S[h] = g[t, h] * S[h] + torch.outer(k[t, h], v[t, h])
                    ref[t, h] = S[h].T @ q[t, h]
    return rows, gb, ref.reshape(n, heads * dv)


@pytest.mark.parametrize("slice_len", [0, 5, 16])
@pytest.mark.parametrize("rule,heads,qk_heads,d,dv", [
    ("delta", 4, 2, 16, 12), ("delta", 3, 3, 20, 28), ("delta", 2, 1, 64, 130), ("delta", 1, 1, 200, 24), ("delta", 5, 5, 1, 3),
    ("delta", 2, 2, 130, 8), ("forget", 3, 3, 10, 14), ("forget", 1, 1, 40, 72), ("forget", 2, 2, 70, 16), ("forget", 2, 2, 300, 8),
    ("forget", 4, 4, 1, 1), ("decay", 4, 2, 24, 10)])
def test_gated_memory_kernel_under_cuts(rule, heads, qk_heads, d, dv, slice_len):
    """The three write rules from strided 32-bit rows, two requests in slots 1 and 3 of 4, fed in steps of unequal sizes
    with single tokens among them. With a slice length the three passes over time slices run instead of one walk (one
    request's last slice short, the other's slices fewer); the delta rule's slices carry a full transition matrix."""
    from tokenmill_b200.kernels import ops
    n = 40
    cases = [_memory_case(rule, heads, qk_heads, d, dv, n, seed=d + i) for i in range(2)]
    qk = qk_heads * d
    floats = ops.gated_memory_state_floats(heads, d, dv)
    state = torch.zeros(4, 8 + floats, device=DEV)
    fed = [0, 0]
    for na, nb in ((1, 17), (20, 1), (2, 1), (17, 21)):
        rows = torch.cat([cases[0][0][fed[0]:fed[0] + na], cases[1][0][fed[1]:fed[1] + nb]]).to(DEV)
        gb = torch.cat([cases[0][1][fed[0]:fed[0] + na], cases[1][1][fed[1]:fed[1] + nb]]).to(DEV).contiguous()
        cu, _, slots = _step_arrays([na, nb], [1, 3])
        y = torch.empty(na + nb, heads * dv, device=DEV)
        sliced = {}
        if slice_len:
            slices = -(-max(na, nb) // slice_len)
            sliced = dict(max_q_len=max(na, nb), slice_len=slice_len, slice_S=torch.full(
                (2 * slices * ops.gated_memory_slice_floats(heads, d, dv, rule == "delta"),), float("nan"), device=DEV))
        ops.gated_memory(rows[:, 5:], q_col=0, k_col=qk, v_col=2 * qk, gb=None if rule == "forget" else gb, rule=rule, state=state,
                         state_off=8, cu_q=cu, state_slots=slots, y=y, n_seqs=2, heads=heads, qk_heads=qk_heads, dim=d, vdim=dv,
                         **sliced)
        ref = torch.cat([cases[0][2][fed[0]:fed[0] + na], cases[1][2][fed[1]:fed[1] + nb]])
        _close(y, ref, torch.float32, (fed, na, nb))
        fed = [fed[0] + na, fed[1] + nb]
    assert float(state[0].abs().max()) == 0.0 and float(state[:, :8].abs().max()) == 0.0


def test_delta_and_forget_gate_preparation():
    """Unit vectors per head with the query's scale, the decay and beta from their projections; silu and the bounded
    forget gate in place."""
    from tokenmill_b200.kernels import ops
    torch.manual_seed(4)
    n, G, d, H = 13, 3, 20, 6
    x = torch.randn(n, 3 + 2 * G * d + 7)
    raw = torch.randn(n, 2 * H + 5) * 3
    A_log, dt_bias = torch.randn(H) - 1, torch.randn(H)
    xd, gb = x.to(DEV), torch.empty(n, 2 * H, device=DEV)
    ops.delta_prepare(xd[:, 3:], 0, G * d, G, d, d ** -0.5, 1e-6, raw.to(DEV)[:, 2:], 1, 1 + H, A_log.to(DEV), dt_bias.to(DEV), H, gb)
    q = pg.unit(x.double()[:, 3:3 + G * d].view(n, G, d)) * d ** -0.5
    k = pg.unit(x.double()[:, 3 + G * d:3 + 2 * G * d].view(n, G, d))
    _close(xd[:, 3:3 + G * d], q.reshape(n, -1), torch.float32, "q")
    _close(xd[:, 3 + G * d:3 + 2 * G * d], k.reshape(n, -1), torch.float32, "k")
    assert torch.equal(xd[:, 3 + 2 * G * d:].cpu(), x[:, 3 + 2 * G * d:]) and torch.equal(xd[:, :3].cpu(), x[:, :3])
    r = raw.double()[:, 2:]
    _close(gb[:, H:], torch.sigmoid(r[:, 1:1 + H]), torch.float32, "beta")
    _close(gb[:, :H], torch.exp(-torch.exp(A_log.double()) * pg.softplus(r[:, 1 + H:1 + 2 * H] + dt_bias.double())),
           torch.float32, "decay")
    m = 37
    y = torch.randn(n, 2 + 2 * m + 4) * 2
    low, bias = torch.rand(m), torch.randn(m)
    yd = y.to(DEV)
    ops.forget_gate_prepare(yd[:, 2:], 0, m, m, low.to(DEV), bias.to(DEV))
    _close(yd[:, 2:2 + m], pg.silu(y.double()[:, 2:2 + m]), torch.float32, "silu")
    f = low.double() + (1 - low.double()) * torch.sigmoid(y.double()[:, 2 + m:2 + 2 * m] + bias.double())
    _close(yd[:, 2 + m:2 + 2 * m], f, torch.float32, "forget gate")
    assert torch.equal(yd[:, 2 + 2 * m:].cpu(), y[:, 2 + 2 * m:])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("gate_act", ["silu", "sigmoid", None])
def test_head_norm_with_a_silu_gate_or_none(dtype, gate_act):
    from tokenmill_b200.kernels import ops
    torch.manual_seed(6)
    n, heads, dv = 9, 5, 28
    y, wide, w = torch.randn(n, heads * dv) * 4, torch.randn(n, heads * dv + 4), 1 + 0.1 * torch.randn(dv)
    out = ops.head_norm_gate(y.to(DEV), wide.to(DEV)[:, 4:] if gate_act else None, w.repeat(heads).to(DEV), 1e-5, heads,
                             torch.empty(n, heads * dv, dtype=dtype, device=DEV), gate_act=gate_act or "sigmoid")
    ref = (pg.rms(y.double().view(n, heads, dv), 1e-5) * w.double()).reshape(n, -1)
    z = wide.double()[:, 4:]
    if gate_act:
        ref = ref * (pg.silu(z) if gate_act == "silu" else torch.sigmoid(z))
    _close(out.float(), ref, dtype, gate_act)


def test_weighted_pair_scaled_start_and_logit_scale():
    from tokenmill_b200.kernels import ops
    torch.manual_seed(7)
    for dtype, n in ((torch.float32, 5 * 52), (torch.bfloat16, 7 * 33)):
        a, b = torch.randn(n).to(dtype), torch.randn(n).to(dtype)
        out = ops.weighted_pair(a.to(DEV), b.to(DEV), 1.3, -0.4, torch.empty(n, dtype=dtype, device=DEV))
        _close(out.float(), 1.3 * a.double() - 0.4 * b.double(), dtype)
    T, H = 6, 52
    table, pos = torch.randn(30, H), torch.randn(40, H)
    ids, positions, w = torch.randint(0, 30, (T,)), torch.randint(0, 40, (T,)), 1 + 0.1 * torch.randn(H)
    resid, out = torch.zeros(T, H, device=DEV), torch.empty(T, H, device=DEV)
    ops.stream_norm(resid, 1, out, kind="rms", weight=w.to(DEV), eps=1e-6, ids=ids.to(DEV).int(), table=table.to(DEV),
                    positions=positions.to(DEV).int(), pos_table=pos.to(DEV), table_scale=7.5)
    x = table[ids].double() * 7.5 + pos[positions].double()
    _close(resid, x, torch.float32, "start")
    _close(out, pg.rms(x, 1e-6) * w.double(), torch.float32, "norm")
    y1, y2 = torch.randn(T, H), torch.randn(T, H)
    ops.stream_norm(resid, 1, out, kind="rms", weight=w.to(DEV), eps=1e-6, branch=y1.to(DEV), branch2=y2.to(DEV))
    _close(resid, x + (y1.double() + y2.double()), torch.float32, "two branches")
    z = torch.linspace(-90, 90, 1001)
    _close(ops.softcap_(z.to(DEV).clone(), 30.0, 0.5), 30.0 * torch.tanh(0.5 * z.double() / 30.0), torch.float32)
    _close(ops.softcap_(z.to(DEV).clone(), 0.0, 0.25), 0.25 * z.double(), torch.float32)


@pytest.mark.parametrize("experts,top,shared", [(6, 2, 16), (4, 1, 0), (3, 3, 8), (12, 1, 20), (9, 4, 0)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_experts_weighted_on_their_input(dtype, experts, top, shared):
    """The feed-forward part as the block calls it, and its choice: the same experts as the plain router's, weights the
    sigmoids themselves."""
    from tokenmill_b200.parts.routed import InputScaledExperts
    torch.manual_seed(experts)
    H, F = 40, 24
    part = InputScaledExperts(hidden_size=H, expert_size=F, num_experts=experts, top=top, shared_size=shared, dtype=dtype,
                              device=torch.device(DEV))
    q = lambda x: x.to(torch.bfloat16).double()
    W = {"m.router": q(0.5 * torch.randn(experts, H))}
    for e in range(experts):
        W[f"m.e{e}.gate"], W[f"m.e{e}.up"], W[f"m.e{e}.down"] = (q(0.3 * torch.randn(F, H)), q(0.3 * torch.randn(F, H)),
                                                                    q(0.2 * torch.randn(H, F)))
    if shared:
        W["m.shared.gate"], W["m.shared.up"] = q(0.3 * torch.randn(shared, H)), q(0.3 * torch.randn(shared, H))
        W["m.shared.down"], W["m.shared.sg"] = q(0.2 * torch.randn(H, shared)), q(0.5 * torch.randn(1, H))
    part.bind({s.name: W["m." + s.name].to(torch.float32 if s.dtype == "float32" else dtype).to(DEV) for s in part.weight_specs()})
    h = q(torch.randn(50, H))
    f = {"router": {"experts": experts, "top": top}, "shared": {"ff": shared} if shared else None}
    idx, w, dense, _ = part.route(h.to(dtype).to(DEV))
    s = torch.sigmoid(h @ W["m.router"].T)
    assert torch.equal(idx.cpu().long().sort(1).values, torch.topk(s, top).indices.sort(1).values)
    _close(dense, torch.zeros_like(s).scatter_(1, idx.cpu().long(), s.gather(1, idx.cpu().long())), torch.float32, "weights")
    _close(part.forward(h.to(dtype).to(DEV)).float(), pg.routed_experts(h, W, "m.", f), dtype)


def _attend(dtype, H, G, d, dv, window, q_lens, starts, page=8, sharpen=1.0, tc=False, hot=None, splits=1):
    """Kernel chain (norm per head + cache write, attention with every head's weights on every value head, the mix of the
    heads) over a paged cache filled step by step, against the plain attention over whole sequences. Returns (engine
    output, plain output) for the LAST step's rows."""
    from tokenmill_b200.kernels import ops
    torch.manual_seed(3)
    n_seq = len(q_lens)
    total = [s + q for s, q in zip(starts, q_lens)]
    P = H * d + G * d + G * dv
    proj = [torch.randn(t, P) for t in total]
    talk = torch.randn(H, H) * 0.6 + torch.eye(H)
    scale = 0.3 * sharpen
    if hot is not None:                 # all scores equal; a few keys carry large values, so that seeing one shows
        for p in proj:
            p[:, :H * d] = 0.0
            for j in hot:
                if j < p.shape[0]:
                    p[j, H * d + G * d:] *= 60.0
    pages = sum(-(-t // page) for t in total)
    order = list(range(pages))
    random.Random(0).shuffle(order)                     # pages lie anywhere
    tables, at = [], 0
    for t in total:
        n = -(-t // page)
        tables.append(order[at:at + n])
        at += n
    width = max(len(t) for t in tables)
    bt = _t([t + [0] * (width - len(t)) for t in tables])
    cache = torch.zeros(pages, page, 1, G * (d + dv), dtype=dtype, device=DEV)
    none = torch.zeros((1, 0), device=DEV)
    outs = None
    for phase in (0, 1):                                # first the cached part, then the step under test
        lens = starts if phase == 0 else q_lens
        befores = [0] * n_seq if phase == 0 else starts
        if sum(lens) == 0:
            continue
        rows = torch.cat([proj[s][befores[s]:befores[s] + lens[s]] for s in range(n_seq)]).to(DEV)
        positions = _t(np.concatenate([np.arange(befores[s], befores[s] + lens[s]) for s in range(n_seq)]))
        slots = _t(np.concatenate([[tables[s][p // page] * page + p % page for p in range(befores[s], befores[s] + lens[s])]
                                   for s in range(n_seq)]))
        T = rows.shape[0]
        q = torch.empty(T, H * d, dtype=dtype, device=DEV)
        ops.qk_norm_rope_write(rows, heads=H, kv_heads=G, dim=d, vdim=dv, rot_dims=0, wq=None, wk=None, eps=1e-6,
                               positions=positions, cos=none, sin=none, slot_map=slots, q_out=q,
                               cache=cache.view(-1, G * (d + dv)), gate_out=None, head_norm=True)
        if phase == 1:
            Gq = H // G
            tile = 64 if tc else 32
            per = [-(-n * Gq // tile) for n in lens]
            tile_seq = np.repeat(np.arange(n_seq), per)
            tile_row0 = np.concatenate([np.arange(n) * tile for n in per])
            cu = np.zeros(n_seq + 1, dtype=np.int32)
            cu[1:] = np.cumsum(lens)
            cross = torch.full((T, H * G * dv), float("nan"), device=DEV)
            part = torch.full((int(tile_seq.size) * G * G * splits * 64 * (dv + 2),), float("nan"), device=DEV) if splits > 1 else None
            ops.sink_attention(q, cache, bt, _t(cu), _t(befores), _t(tile_seq), _t(tile_row0), int(tile_seq.size), None, None,
                               heads=H, kv_heads=G, dim=d, vdim=dv, scale=scale, softcap=0.0, window=window, keep_first=0,
                               sink=False, tensor_cores=tc, n_splits=splits, part=part, cross_out=cross)
            outs = ops.talk_mix(cross, talk.to(DEV), torch.empty(T, H * dv, dtype=dtype, device=DEV), H, G, dv)
    ref = []
    for s in range(n_seq):
        p = proj[s].double()
        t = total[s]
        qq = pg.rms(p[:, :H * d].view(t, H, d), 1e-6)
        kk = pg.rms(p[:, H * d:H * d + G * d].view(t, G, d), 1e-6)
        vv = p[:, H * d + G * d:].reshape(t, G, dv)
        if dtype == torch.bfloat16:
            qq, kk, vv = (x.to(torch.bfloat16).double() for x in (qq, kk, vv))
        A = pg.talking_heads(pg.window_softmax_weights(qq, kk, scale, window), talk.double())
        o = torch.stack([A[h] @ vv[:, h // (H // G)] for h in range(H)], dim=1)
        ref.append(o[starts[s]:].reshape(q_lens[s], H * dv))
    return outs.float().cpu().double(), torch.cat(ref)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", [dict(H=6, G=3, d=12, dv=20, window=11), dict(H=4, G=1, d=16, dv=8, window=37),
                                  dict(H=5, G=5, d=10, dv=40, window=500), dict(H=2, G=2, d=34, dv=10, window=1)])
def test_mixed_heads_attention_prompt_portion_and_decoding(dtype, case):
    """Three kinds of request in one step: a prompt from position 0, a portion that continues 61 cached tokens (its
    window lies in other pages than its queries), and single decoded tokens behind 40 and 95."""
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    got, ref = _attend(dtype, q_lens=[50, 23, 1, 1], starts=[0, 61, 40, 95], **case)
    assert (got - ref).abs().max() < tol * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("case", [dict(H=4, G=2, d=32, dv=64, window=70), dict(H=6, G=1, d=64, dv=32, window=13),
                                  dict(H=3, G=3, d=128, dv=128, window=1000), dict(H=8, G=2, d=64, dv=128, window=100)])
def test_mixed_heads_on_the_tensor_core_kernel(case):
    """The mma.sync kernel on the same kind of step (a 200-token prompt; a portion behind 150 cached tokens; single
    tokens), against the plain attention on the rounded q, k, v, against the CUDA-core kernel, and with the key blocks
    dealt out over several blocks and merged."""
    q_lens, starts = [200, 23, 1, 1], [0, 150, 40, 333]
    got, ref = _attend(torch.bfloat16, q_lens=q_lens, starts=starts, tc=True, **case)
    assert (got - ref).abs().max() < 3e-2 * max(1.0, float(ref.abs().max()))
    slow, _ = _attend(torch.bfloat16, q_lens=q_lens, starts=starts, tc=False, **case)
    assert (got - slow).abs().max() < 3e-2 * max(1.0, float(ref.abs().max()))
    for splits in (2, 3, 8):
        cut, _ = _attend(torch.bfloat16, q_lens=q_lens, starts=starts, tc=True, splits=splits, **case)
        assert (cut - ref).abs().max() < 3e-2 * max(1.0, float(ref.abs().max())), splits


@pytest.mark.parametrize("tc", [False, True])
def test_window_edges_with_hot_keys(tc):
    """All scores equal and a few keys with values sixty times the others': a row that sees such a key one position
    too early or too late is off by far more than rounding. Hot keys sit where rows of the step have their window's
    first key and the key before it, and at the borders of the kernels' key blocks, in a prompt and in decoded tokens."""
    case = dict(H=4, G=2, d=64, dv=32)
    hot = [5, 6, 31, 32, 63, 64, 100, 128, 129, 140]
    kw = dict(q_lens=[230, 1, 1, 1], starts=[0, 133, 134, 209], hot=hot, tc=tc, splits=3 if tc else 1, **case)
    got, ref = _attend(torch.bfloat16, window=70, **kw)
    assert (got - ref).abs().max() < 3e-2 * float(ref.abs().max())
    for dw in (1, -1):
        _, other = _attend(torch.bfloat16, window=70 + dw, **kw)
        rows = (other - ref).abs().amax(dim=1) > 6e-2 * float(ref.abs().max())
        assert int(rows[:230].sum()) >= 5 and bool(rows[230:].any()), dw


def test_window_edges_with_sharp_queries():
    """Scores scaled up so that single keys carry the softmax: the plain result with the window one off differs visibly;
    the kernel agrees with the true one, in a prompt and in decoded tokens."""
    case = dict(H=4, G=2, d=16, dv=12)
    got, ref = _attend(torch.float32, q_lens=[90, 1, 1], starts=[0, 33, 77], window=13, sharpen=12.0, **case)
    assert (got - ref).abs().max() < 2e-5 * max(1.0, float(ref.abs().max()))
    for dw in (1, -1):
        _, other = _attend(torch.float32, q_lens=[90, 1, 1], starts=[0, 33, 77], window=13 + dw, sharpen=12.0, **case)
        assert ((other - ref).abs().amax(dim=1) > 1e-3).float()[20:].mean() > 0.3, dw


# --- the whole model under every cut ----------------------------------------------------------------------------

@pytest.mark.parametrize("size", SIZES)
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_against_plain(gofezen_dirs, plain_memo, size, mode, dtype, tmp_path):
    folder = gofezen_dirs[size]
    vocab = json.loads((folder / "config.json").read_text())["vocab"]
    reqs = make_requests(vocab, LENGTHS, seed=11)
    steps, max_tokens = _steps(mode, reqs)
    outputs = run_trace(folder, dtype, steps, max_tokens, tmp_path / "out")
    _check(steps, outputs, reqs, _plain(folder, reqs, plain_memo), dtype)


@pytest.mark.parametrize("page", [8, 32])
def test_replay_at_other_page_sizes(gofezen_dirs, plain_memo, page, tmp_path):
    folder = gofezen_dirs["gofezen-tiny-a"]
    reqs = make_requests(173, LENGTHS, seed=13)
    steps, max_tokens = mixed_steps(reqs, seed=9)
    outputs = run_trace(folder, "float32", steps, max_tokens, tmp_path / "out", page_size=page)
    check_against_plain(steps, outputs, reqs, _plain(folder, reqs, plain_memo), "float32")


def test_cuts_do_not_move_the_logits_in_float32(gofezen_dirs, tmp_path):
    """Whole prompts against mixed batches of portions and single tokens: every sum walks keys and tokens in the same
    order whatever the cut, so in 32-bit the rows agree to a few units in the last place."""
    folder = gofezen_dirs["gofezen-tiny-a"]
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
        assert worst <= 6e-6 * scale, (mode, worst)


# --- faults that random weights would hide ----------------------------------------------------------------------

def _sharpen(src, dst, *, attention=1.0, slow=False, edit=None):
    """A copy of a model whose attention is sharp (its score scale multiplied, so that single keys carry the softmax and a
    lost or doubled key or a window one off shows) and, with ``slow``, whose memories forget slowly (decays and forget
    gates close to one: a lost or stale state shows hundreds of tokens later)."""
    cfg, w = _read(src)
    for i, layer in enumerate(cfg["layers"]):
        if layer["type"] == "parallel":
            layer["mixer"]["left"]["scale"] *= attention
            if slow:
                w[f"l{i}.mix.right.A_log"] = torch.full_like(w[f"l{i}.mix.right.A_log"], -5.0)
                w[f"l{i}.mix.right.dt_bias"] = torch.full_like(w[f"l{i}.mix.right.dt_bias"], -2.0)
        elif slow:
            w[f"l{i}.mix.lower"] = torch.full_like(w[f"l{i}.mix.lower"], 0.992)
    if edit is not None:
        edit(cfg, w)
    w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}          # what the file will hold
    return _write(dst, cfg, w), cfg, w


def test_window_edge_in_prompts_and_in_decoding(gofezen_dirs, tmp_path):
    """Sharp attention over 230 and 150 tokens with windows of 24 and 37. On the plain model a window one longer or
    shorter moves many rows by far more than the tolerance; the engine agrees with the true one in prompts, in decoded
    tokens (60 of them, so that the window passes over decoded tokens) and across page borders."""
    folder, cfg, w = _sharpen(gofezen_dirs["gofezen-tiny-a"], tmp_path / "sharp", attention=25.0)
    reqs = make_requests(cfg["vocab"], [230, 150], seed=31)
    plain = {r: _logits(cfg, w, t) for r, t in reqs.items()}
    tol = 2e-4 * float(plain["r0"].abs().max())
    for d in (-1, 1):
        other = copy.deepcopy(cfg)
        for layer in other["layers"]:
            if layer["type"] == "parallel":
                layer["mixer"]["left"]["mask"]["size"] += d
        moved = ((_logits(other, w, reqs["r0"]) - plain["r0"]).abs().amax(dim=1) > 10 * tol).float()[40:].mean()
        assert moved > 0.3, (d, float(moved))
    for mode in ("whole", "tail", "portions", "mixed"):
        steps, max_tokens = _steps(mode, reqs) if mode != "tail" else tail_decode_steps(reqs, tail=60)
        outputs = run_trace(folder, "float32", steps, max_tokens, tmp_path / mode)
        check_against_plain(steps, outputs, reqs, plain, "float32")


@pytest.mark.parametrize("size", ["gofezen-tiny-b", "gofezen-tiny-c"])
def test_an_old_state_shows(gofezen_dirs, size, tmp_path):
    """Memories that forget slowly: changing the second token of a 340-token request still moves its last logits
    (checked on the plain model), so state carried over many steps, the time slices of long portions, long decoding (120
    tokens) and slots are looked at."""
    folder, cfg, w = _sharpen(gofezen_dirs[size], tmp_path / "slow", slow=True)
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


def test_the_weight_is_on_the_input_and_the_heads_are_mixed(gofezen_dirs, tmp_path):
    """Two things a plain model computed otherwise gets wrong at most rows, and the engine gets right: experts run on the
    weighted input (not weighted afterwards), and the heads' softmax weights are mixed (a mix of the identity is not the
    same model)."""
    folder = gofezen_dirs["gofezen-tiny-a"]
    cfg, w = _read(folder)
    reqs = make_requests(cfg["vocab"], [90, 64], seed=43)
    plain = {r: _logits(cfg, w, t) for r, t in reqs.items()}
    tol = 2e-4 * float(plain["r0"].abs().max())
    plain_talk = dict(w)
    for k in w:
        if k.endswith(".talk"):
            plain_talk[k] = torch.eye(w[k].shape[0])
    assert ((_logits(cfg, plain_talk, reqs["r0"]) - plain["r0"]).abs().amax(dim=1) > 10 * tol).float().mean() > 0.5
    real = pg.routed_experts
    try:
        def after(h, W, p, f):          # the weight on the output instead
            out = torch.zeros_like(h)
            s = torch.sigmoid(h @ W[p + "router"].T)
            for t in range(h.shape[0]):
                for e in torch.topk(s[t], f["router"]["top"]).indices.tolist():
                    out[t] += s[t, e] * pg.glu(h[t][None], W, f"{p}e{e}.")[0]
            if f.get("shared"):
                out = out + torch.sigmoid(h @ W[p + "shared.sg"].T) * pg.glu(h, W, p + "shared.")
            return out
        pg.routed_experts = after
        wrong = _logits(cfg, w, reqs["r0"])
    finally:
        pg.routed_experts = real
    assert ((wrong - plain["r0"]).abs().amax(dim=1) > 10 * tol).float().mean() > 0.5
    for mode in ("whole", "mixed"):
        steps, max_tokens = _steps(mode, reqs)
        check_against_plain(steps, run_trace(folder, "float32", steps, max_tokens, tmp_path / mode), reqs, plain, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_of_unlike_sizes(dtype, tmp_path):
    """Layers that share no size, in another order: three pairs with different heads (three page groups), memories wider
    than a warp's rows, one tap and five taps, a single expert, top = all experts, one head; prompts of 300 and 270
    tokens (beyond the slice threshold) whole and in mixed batches, then decoded."""
    from tokenmill_b200.weights import write_random_model
    from tokenmill_b200.weights.random_init import gofezen_config, gofezen_hgrn2 as R, gofezen_moe as E, gofezen_pair as P
    cfg = gofezen_config(vocab=157, width=72, eps=1e-5, max_positions=320, embedding_scale=3.0, logit_scale=1.5, logit_softcap=12.0, layers=[
        ("hgrn2", R(heads=1, dim=96, vdim=16), E(experts=4, top=4, ff=40, shared=8)),
        ("parallel", P(heads=10, kv_heads=5, dim=12, vdim=20, scale=0.25, conv=1, window=50, r_heads=1, r_qk_heads=1, r_dim=36,
                       r_vdim=72, r_conv=5, left_scale=0.5, right_scale=2.0), None),
        ("parallel", P(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.125, conv=5, window=129, r_heads=6, r_qk_heads=2, r_dim=24,
                       r_vdim=12, r_conv=2), E(experts=1, top=1, ff=88)),
        ("hgrn2", R(heads=6, dim=12, vdim=12), {"kind": "dense", "ff": 100}),
        ("parallel", P(heads=2, kv_heads=2, dim=24, vdim=36, scale=0.2, conv=3, window=300, r_heads=2, r_qk_heads=2, r_dim=130,
                       r_vdim=16, r_conv=3), E(experts=9, top=3, ff=8, shared=40))])
    folder = _lively(write_random_model(tmp_path / "m", cfg, seed=12))
    _, w = _read(folder)
    reqs = make_requests(157, [300, 270], seed=71)
    plain = {r: _logits(cfg, w, t) for r, t in reqs.items()}
    for mode in ("whole", "tail", "mixed"):
        steps, max_tokens = _steps(mode, reqs)
        _check(steps, run_trace(folder, dtype, steps, max_tokens, tmp_path / mode), reqs, plain, dtype)


@pytest.mark.parametrize("kind", ["memories", "pairs"])
def test_models_of_one_kind_of_layer(kind, tmp_path):
    """Only forget-gate memories (no pages at all, one layer without a feed-forward) and only pairs (two page groups),
    with seven taps in one layer, and in the other no mask (every earlier key) and no convolution on either side: mixed
    batches against the plain model."""
    from tokenmill_b200.weights import write_random_model
    from tokenmill_b200.weights.random_init import gofezen_config, gofezen_hgrn2 as R, gofezen_moe as E, gofezen_pair as P
    if kind == "memories":
        layers = [("hgrn2", R(heads=2, dim=20, vdim=12), E(experts=3, top=2, ff=16)), ("hgrn2", R(heads=4, dim=8, vdim=16), None),
                  ("hgrn2", R(heads=1, dim=33, vdim=40), {"kind": "dense", "ff": 48})]
    else:
        layers = [("parallel", P(heads=2, kv_heads=1, dim=20, vdim=12, scale=0.3, conv=7, window=17, r_heads=2, r_qk_heads=1, r_dim=12,
                                 r_vdim=20, r_conv=7), None),
                  ("parallel", P(heads=3, kv_heads=3, dim=8, vdim=8, scale=0.4, conv=2, window=64, r_heads=4, r_qk_heads=4, r_dim=8,
                                 r_vdim=10, r_conv=2, left_scale=0.7), E(experts=2, top=1, ff=24, shared=16))]
        del layers[1][1]["left"]["mask"], layers[1][1]["left"]["conv"], layers[1][1]["right"]["conv"]
    cfg = gofezen_config(vocab=131, width=40, max_positions=260, embedding_scale=5.0, logit_softcap=0.0, layers=layers)
    folder = _lively(write_random_model(tmp_path / "m", cfg, seed=21))
    _, w = _read(folder)
    reqs = make_requests(131, [120, 75, 33, 90], seed=81)
    plain = {r: _logits(cfg, w, t) for r, t in reqs.items()}
    for mode in ("whole", "mixed"):
        steps, max_tokens = _steps(mode, reqs)
        check_against_plain(steps, run_trace(folder, "float32", steps, max_tokens, tmp_path / mode), reqs, plain, "float32")


def test_slots_and_pages_used_again_start_clean(gofezen_dirs, plain_memo, tmp_path):
    """Nine requests through a pool for two live ones with two state slots: every slot and page is used several times,
    and a request that follows a long one on its slot gets the same logits as alone."""
    folder = gofezen_dirs["gofezen-tiny-a"]
    reqs = make_requests(173, [90, 30, 64, 12, 100, 5, 77, 48, 33], seed=51)
    steps, max_tokens = mixed_steps(reqs, seed=2, max_live=2)
    from tokenmill_b200.engine.trace import run
    out_dir = tmp_path / "out"
    stdin = io.StringIO("".join(json.dumps(s) + "\n" for s in steps))
    assert run(str(folder), "float32", str(out_dir), max_tokens, stdin=stdin, stdout=io.StringIO(), state_slots=2) == 0
    outputs = {s["step"]: np.fromfile(out_dir / f"{s['step']}.f32", dtype="<f4").reshape(-1, 173) for s in steps}
    check_against_plain(steps, outputs, reqs, _plain(folder, reqs, plain_memo), "float32")


def test_first_tokens_and_single_token_requests(gofezen_dirs, plain_memo, tmp_path):
    """Requests of one, two and three tokens (shorter than the convolutions' carried inputs), fed whole and token by
    token, beside each other."""
    folder = gofezen_dirs["gofezen-tiny-b"]       # five taps
    reqs = make_requests(300, [1, 2, 3, 4, 6], seed=61)
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
    ("gofezen-tiny-a", False, False, "float32"), ("gofezen-tiny-a", True, True, "float32"),
    ("gofezen-tiny-b", False, True, "bfloat16"), ("gofezen-tiny-c", True, True, "bfloat16")])
def test_greedy_generation_through_the_engine(gofezen_dirs, size, graphs, chunked, dtype):
    """LLMEngine with its scheduler: admission (state slots, page groups), chunked prompts beside decodes, decode graphs
    with padded rows, a pool so small that requests are evicted and recomputed. The logits behind every generated token
    equal the plain model's on the request's own history, and the token is their arg-max. (bfloat16: the rows are the same
    numbers with and without graphs and chunks; up to fifteen in a hundred may lie outside 3 %, where a router's choice
    between two nearly equal scores falls the other way on rounded inputs: with one expert of five chosen in a model
    this small that moves a token's logits by tens of percent. The 32-bit runs hold every row.)"""
    from tokenmill_b200 import EngineConfig
    from tokenmill_b200.engine import LLMEngine
    from tokenmill_b200.sampling import SamplingParams

    folder = gofezen_dirs[size]
    cfg, w = _read(folder)
    rng = random.Random(5)
    prompts = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (9, 30, 17, 44, 5, 26, 12)]
    owners = [l["mixer"]["left"] for l in cfg["layers"] if l["type"] == "parallel"]
    per_token = sum(a["kv_heads"] * (a["dim"] + a["vdim"]) for a in owners) * (4 if dtype == "float32" else 2)
    eng = LLMEngine(EngineConfig(model=str(folder), dtype=dtype, block_size=8, max_model_len=128, max_num_seqs=4,
                                 kv_cache_mb=(16 * 8 + (8 if graphs else 0) + 1) * per_token / 2 ** 20, watermark=0.0,
                                 cuda_graphs=graphs, cuda_graph_max_batch=4, enable_chunked_prefill=chunked,
                                 max_num_batched_tokens=24 if chunked else 256))
    assert eng.cache.state_slots.num_slots == 4
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
    assert compared >= 7 * 24 and over <= 0.15 * compared, (over, compared)


def test_generate_command_line_and_trace_runner(gofezen_dirs, tmp_path):
    """The two programs a user starts: ``python -m tokenmill_b200.generate`` on a Gofezen folder, and bin/trace_run."""
    root = Path(__file__).resolve().parents[1]
    folder = gofezen_dirs["gofezen-tiny-b"]
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
