"""Gofezen restated plainly: float64 on the CPU, token by token where the design is recurrent, one function per
mechanism. It shares nothing with the engine: tensors are read by name from a dictionary, every sum is written out.

Notation: h is a layer's normed input [T, width]; W["l3.mix.q"] and the like are the checkpoint's tensors (matrices
stored [out, in]); ``m`` is a layer's ``mixer`` entry of config.json, ``f`` its ``mlp`` entry; p a tensor-name prefix.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def rms(x, eps):
    """x over its root mean square along the last axis, eps under the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def causal_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the first token."""
    T, C = u.shape
    taps = w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            src = t - taps + 1 + j
            if src >= 0:
                y[t] += w[:, j] * u[src]
    return y


def window_softmax_weights(q, k, scale, window):
    """q [T, H, d], k [T, G, d] -> weights [H, T, T]: row i of head h is a softmax over the keys j with
    0 <= i - j < window of (q_i . k_j) * scale, zero elsewhere."""
    T, H, _ = q.shape
    G = k.shape[1]
    A = torch.zeros((H, T, T), dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = max(0, i - window + 1)
            s = (k[lo: i + 1, g] @ q[i, h]) * scale
            A[h, i, lo: i + 1] = torch.softmax(s, 0)
    return A


def talking_heads(A, talk):
    """A [H, T, T], talk [H, H]: head h's new weights are sum_g talk[h, g] A[g]."""
    return torch.einsum("hg,gij->hij", talk, A)


def windowed_attention_mixer(h, W, p, m, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    proj = {}
    for name in ("q", "k", "v"):
        u = h @ W[p + name].T + W[p + name + ".b"]
        proj[name] = causal_conv(u, W[p + name + ".conv"]) if "conv" in m else u
    q = rms(proj["q"].view(T, H, d), eps)
    k = rms(proj["k"].view(T, G, d), eps)
    v = proj["v"].view(T, G, dv)
    window = m["mask"]["size"] if m.get("mask") else T          # no mask: every earlier key
    A = talking_heads(window_softmax_weights(q, k, m["scale"], window), W[p + "talk"])
    out = torch.zeros((T, H, dv), dtype=h.dtype)
    for hd in range(H):
        out[:, hd] = A[hd] @ v[:, hd // (H // G)]
    return out.reshape(T, H * dv) @ W[p + "o"].T


def unit(x):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def delta_rule(q, k, v, beta, g):
    """q, k [T, H, d]; v [T, H, dv]; beta, g [T, H]. Per head from S = 0: S <- g S; u = beta (v - S^T k);
    S <- S + k u^T; o = S^T q."""
    T, H, d = q.shape
    dv = v.shape[-1]
    S = torch.zeros((H, d, dv), dtype=q.dtype)
    out = torch.zeros((T, H, dv), dtype=q.dtype)
    for t in range(T):
        for hd in range(H):
            S[hd] = g[t, hd] * S[hd]
            u = beta[t, hd] * (v[t, hd] - S[hd].T @ k[t, hd])
            S[hd] = S[hd] + torch.outer(k[t, hd], u)
            out[t, hd] = S[hd].T @ q[t, hd]
    return out


def gated_delta_mixer(h, W, p, m, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    conv = (lambda u, name: causal_conv(u, W[p + name + ".conv"])) if "conv" in m else (lambda u, name: u)
    q = silu(conv(h @ W[p + "q"].T, "q")).view(T, G, d)
    k = silu(conv(h @ W[p + "k"].T, "k")).view(T, G, d)
    v = silu(conv(h @ W[p + "v"].T, "v")).view(T, H, dv)
    q = unit(q) * d ** -0.5
    k = unit(k)
    rep = H // G
    q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(h @ W[p + "b"].T)
    decay = torch.exp(-torch.exp(W[p + "A_log"]) * softplus(h @ W[p + "a"].T + W[p + "dt_bias"]))
    o = delta_rule(q, k, v, beta, decay)
    o = rms(o, eps) * W[p + "norm"]
    o = o.reshape(T, H * dv) * silu(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def pair_mixer(h, W, p, m, eps):
    left = windowed_attention_mixer(h, W, p + "left.", m["left"], eps)
    right = gated_delta_mixer(h, W, p + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def forget_gate_memory(q, f, v):
    """q, f [T, H, d]; v [T, H, dv]. Per head from S = 0: S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t."""
    T, H, d = q.shape
    dv = v.shape[-1]
    S = torch.zeros((H, d, dv), dtype=q.dtype)
    out = torch.zeros((T, H, dv), dtype=q.dtype)
    for t in range(T):
        for hd in range(H):
            S[hd] = f[t, hd][:, None] * S[hd] + torch.outer(1.0 - f[t, hd], v[t, hd])
            out[t, hd] = S[hd].T @ q[t, hd]
    return out


def hgrn2_mixer(h, W, p, m, eps):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ W[p + "q"].T).view(T, H, d)
    v = (h @ W[p + "v"].T).view(T, H, dv)
    low = W[p + "lower"]
    f = (low + (1.0 - low) * torch.sigmoid(h @ W[p + "f"].T + W[p + "f.b"])).view(T, H, d)
    o = rms(forget_gate_memory(q, f, v), eps) * W[p + "norm"]
    return o.reshape(T, H * dv) @ W[p + "o"].T


def glu(x, W, p):
    return (silu(x @ W[p + "gate"].T) * (x @ W[p + "up"].T)) @ W[p + "down"].T


def routed_experts(h, W, p, f):
    """Sigmoid scores, the ``top`` largest chosen, each chosen expert run on score * h; a shared expert times
    sigmoid(W_sg h)."""
    E, top = f["router"]["experts"], f["router"]["top"]
    s = torch.sigmoid(h @ W[p + "router"].T)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = torch.topk(s[t], top).indices.tolist()
        for e in chosen:
            out[t] += glu((s[t, e] * h[t])[None], W, f"{p}e{e}.")[0]
    if f.get("shared"):
        out = out + torch.sigmoid(h @ W[p + "shared.sg"].T) * glu(h, W, p + "shared.")
    return out


def feed_forward(h, W, p, f):
    if f is None:
        return torch.zeros_like(h)
    return glu(h, W, p) if f["kind"] == "dense" else routed_experts(h, W, p, f)


def forward(cfg, W, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence from position 0. ``layers_out``: a list that receives the stream after every
    layer."""
    W = {k: v.to(F64) for k, v in W.items()}
    ids = torch.as_tensor(tokens, dtype=torch.long)
    T = ids.numel()
    eps = cfg["norm"]["eps"]
    x = W["embed"][ids] * cfg["embedding"]["scale"] + W["pos"][:T]
    for i, layer in enumerate(cfg["layers"]):
        h = rms(x, eps) * W[f"l{i}.norm1"]
        p = f"l{i}.mix."
        if layer["type"] == "parallel":
            mixed = pair_mixer(h, W, p, layer["mixer"], eps)
        else:
            mixed = hgrn2_mixer(h, W, p, layer["mixer"], eps)
        x = x + (mixed + feed_forward(h, W, f"l{i}.mlp.", layer.get("mlp")))
        if layers_out is not None:
            layers_out.append(x.clone())
    z = (rms(x, eps) * W["final.norm"]) @ W["head"].T * cfg["logit_scale"]
    cap = cfg.get("logit_softcap") or 0.0
    return cap * torch.tanh(z / cap) if cap else z
