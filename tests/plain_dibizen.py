"""Dibizen restated plainly: float64 on the CPU, token by token where the design is recurrent, one function per
mechanism. It shares nothing with the engine: tensors are read by name from a dictionary, every sum is written out.

Notation: h is a sublayer's input [T, width]; W["l3.mix.q"] and the like are the checkpoint's tensors (matrices stored
[out, in]); ``m`` is a layer's ``mixer`` entry of config.json, ``f`` its ``mlp`` entry.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def silu(x):
    return x * torch.sigmoid(x)


def dynamic_tanh(x, weight, bias, alpha):
    """tanh(alpha x) w + b: no statistic of the row enters."""
    return torch.tanh(alpha * x) * weight + bias


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def stream_read(streams, w_in):
    """u = sum_s in[s] x_s over the list of streams."""
    return sum(w_in[s] * x for s, x in enumerate(streams))


def stream_write(streams, y, mix, w_out):
    """All streams at once from the old ones: x_t <- sum_s mix[s, t] x_s + out[t] y."""
    n = len(streams)
    return [sum(mix[s, t] * streams[s] for s in range(n)) + w_out[t] * y for t in range(n)]


def query_temperature(positions, coef, every):
    """1 + coef ln(floor((p + 1) / every) + 1)."""
    return 1.0 + coef * torch.log(torch.floor((positions.to(F64) + 1.0) / every) + 1.0)


def causal_attention(q, k, v, scale):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; query head h reads key head h // (H / G); every j <= i is seen."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[-1]), dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            s = (k[: i + 1, g] @ q[i, h]) * scale
            out[i, h] = torch.softmax(s, 0) @ v[: i + 1, g]
    return out


def attention_mixer(h, W, p, m, shared_kv=None):
    """Returns (mixer output, (k, v)); ``shared_kv``: another layer's keys and values, used instead of own ones."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).view(T, H, d)
    if shared_kv is None:
        k, v = (h @ W[p + "k"].T).view(T, G, d), (h @ W[p + "v"].T).view(T, G, dv)
    else:
        k, v = shared_kv
    if m.get("q_temp"):
        q = q * query_temperature(torch.arange(T), m["q_temp"]["coef"], m["q_temp"]["every"])[:, None, None]
    o = causal_attention(q, k, v, m["scale"]).reshape(T, H * dv)
    o = o * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T, (k, v)


def decay_memory(q, k, v, decay):
    """Per head S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, from S = 0. q, k [T, H, d]; v [T, H, dv]."""
    T, H, d = q.shape
    S = torch.zeros((H, d, v.shape[-1]), dtype=q.dtype)
    out = torch.zeros((T, H, v.shape[-1]), dtype=q.dtype)
    for t in range(T):
        for hd in range(H):
            S[hd] = decay[hd] * S[hd] + torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = S[hd].T @ q[t, hd]
    return out


def lightning_mixer(h, W, p, m, eps):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q, k = silu(h @ W[p + "q"].T).view(T, H, d), silu(h @ W[p + "k"].T).view(T, H, d)
    v = silu(h @ W[p + "v"].T).view(T, H, dv)
    o = decay_memory(q, k, v, [float(a) for a in m["decay"]]).reshape(T, H * dv)
    o = rms(o, eps) * W[p + "norm"] * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def causal_conv(x, weight, bias):
    """Per channel: out_t = bias + sum_j weight[:, j] x_(t - taps + 1 + j), zeros before the start."""
    T, taps = x.shape[0], weight.shape[1]
    padded = torch.cat([torch.zeros((taps - 1, x.shape[1]), dtype=x.dtype), x])
    return bias + sum(padded[j:j + T] * weight[:, j] for j in range(taps))


def selective_scan(x, dt, A, B, C, D):
    """x, dt [T, I]; A [I, N]; B, C [T, N]; D [I]. S <- exp(dt A) S + dt x B; y = S C + D x."""
    T, I = x.shape
    S = torch.zeros(A.shape, dtype=x.dtype)
    y = torch.zeros((T, I), dtype=x.dtype)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + D * x[t]
    return y


def mamba_mixer(h, W, p, m):
    I, N, R = m["inner"], m["state"], m["dt_rank"]
    xz = h @ W[p + "in"].T
    x, z = xz[:, :I], xz[:, I:]
    x = silu(causal_conv(x, W[p + "conv"], W[p + "conv.b"]))
    low_b_c = x @ W[p + "x"].T
    dt = torch.nn.functional.softplus(low_b_c[:, :R] @ W[p + "dt"].T + W[p + "dt.b"])
    y = selective_scan(x, dt, -torch.exp(W[p + "A_log"]), low_b_c[:, R:R + N], low_b_c[:, R + N:], W[p + "D"])
    return (y * silu(z)) @ W[p + "o"].T


def route(h, W, p, r):
    """(chosen outputs [T, top], their weights [T, top]) of the router entry r."""
    n = r["experts"] + int(r.get("identity") or 0)
    s = torch.softmax(h @ W[p + "router"].T, -1)
    choice = s + W[p + "correction"]
    g = r.get("groups")
    if g and g["count"] > 1:
        per = n // g["count"]
        best = choice.view(-1, g["count"], per).max(-1).values
        keep = torch.zeros_like(best, dtype=torch.bool)
        for t in range(best.shape[0]):                    # the best groups, lowest number first among equals
            order = sorted(range(g["count"]), key=lambda j: (-float(best[t, j]), j))
            keep[t, order[:g["keep"]]] = True
        choice = choice.masked_fill(~keep.repeat_interleave(per, 1), -math.inf)
    idx = torch.zeros((h.shape[0], r["top"]), dtype=torch.long)
    for t in range(h.shape[0]):
        order = sorted(range(n), key=lambda j: (-float(choice[t, j]), j))
        idx[t] = torch.tensor(order[:r["top"]])
    w = s.gather(1, idx)
    return idx, w / (w.sum(-1, keepdim=True) + 1e-20)


def experts(h, W, p, f):
    r = f["router"]
    idx, w = route(h, W, p, r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(r["top"]):
            e = int(idx[t, j])
            if e >= r["experts"]:
                y = h[t]                                  # an identity output
            else:
                y = (torch.relu(h[t] @ W[f"{p}e{e}.up"].T) ** 2) @ W[f"{p}e{e}.down"].T
            out[t] += w[t, j] * y
    return out


def forward(cfg, W, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence from position 0; ``layers_out`` receives the summed streams after every layer."""
    W = {k: v.to(F64) for k, v in W.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    T, n = tokens.numel(), cfg.get("streams", 1)
    start = W["embed"][tokens] + W["pos"][:T]
    streams = [start.clone() for _ in range(n)]
    kv = {}
    for i, layer in enumerate(cfg["layers"]):
        lp, m = f"l{i}.", layer["mixer"]
        u = stream_read(streams, W[lp + "hc1.in"])
        h = dynamic_tanh(u, W[lp + "norm1"], W[lp + "norm1.b"], W[lp + "norm1.alpha"])
        if layer["type"] == "attention":
            y, kv[i] = attention_mixer(h, W, lp + "mix.", m, kv[m["kv_from"]] if m.get("kv_from") is not None else None)
        elif layer["type"] == "lightning":
            y = lightning_mixer(h, W, lp + "mix.", m, cfg["norm"]["eps"])
        else:
            y = mamba_mixer(h, W, lp + "mix.", m)
        streams = stream_write(streams, y, W[lp + "hc1.mix"], W[lp + "hc1.out"])
        if layer.get("mlp") is not None:
            u = stream_read(streams, W[lp + "hc2.in"])
            h = dynamic_tanh(u, W[lp + "norm2"], W[lp + "norm2.b"], W[lp + "norm2.alpha"])
            streams = stream_write(streams, experts(h, W, lp + "mlp.", layer["mlp"]), W[lp + "hc2.mix"], W[lp + "hc2.out"])
        if layers_out is not None:
            layers_out.append(sum(streams))
    x = dynamic_tanh(sum(streams), W["final.norm"], W["final.norm.b"], W["final.norm.alpha"])
    logits = x @ W["head"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits
