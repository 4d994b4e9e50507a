"""Matrix memories whose decay is computed from the token: the gated delta rule, and a memory whose forget gate also
decides what is written (HGRN2).

``GatedDeltaMixer``. From the mixer's input h: q = W_q h and k = W_k h (``num_qk_heads`` x d), v = W_v h (``num_heads`` x
dv), no biases; head h reads q/k head h // (num_heads // num_qk_heads). Each of q, k, v passes a short causal
convolution over time per channel (tensors ``<q>.conv`` [channels, taps], the last tap weighing the current token) and
then silu. q and k become unit vectors per head, x / sqrt(sum x^2 + 1e-6), q also times d^-1/2. Per head
``beta = sigmoid(W_b h)`` and ``g = exp(-exp(A_log) softplus(W_a h + dt_bias))``, and from S = 0
    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
so the read-out sees the current token's write. Each head's o is divided by its root mean square over dv, times a plain
weight (dv numbers, shared by the heads), times silu(W_g h), and projected by W_o.

``ForgetGateMemoryMixer``. q = silu(W_q h) (heads x d), v = W_v h (heads x dv), forget gate per head and row
``f = low + (1 - low) sigmoid(W_f h + b_f)`` with a learned lower bound ``low``; per head from S = 0
    S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T;   o_t = S_t^T q_t
(no key and no other scale). Each head's o is RMS-normed over dv with a plain weight shared by the heads, the heads lie
side by side and W_o projects them.

Decays, gates, unit norms, the memories and the norms are 32-bit in both run dtypes; the projections' products keep
their 32-bit accumulators. Per request a mixer keeps the convolutions' last taps - 1 inputs and S (a column's rows side
by side, [heads, dv, d padded]) in ONE state slot of 32-bit floats, zero for a new request; prompt portions and single
decoded tokens run the same kernels, which walk a request's tokens in order whatever the cut. A step whose longest
portion has ``SLICED_FROM`` tokens runs three passes over time slices instead (csrc/gated_memory.cu): the same sums in
another order. A mixer that runs beside another may be handed its columns of a shared product
(``projection_weight`` / ``forward_projected``).
"""

from __future__ import annotations

import torch

from ..kernels import lib, ops
from ..registry import register_mixer
from .base import LayerCache, StepInputs
from .spec import StateNeed, WeightSpec


SLICED_FROM = 256               # a step whose longest portion has this many tokens runs over time slices
SLICE_LEN = 128
SLICE_SCRATCH_LIMIT = 1 << 29    # bytes of scratch the slices may take; beyond it a step walks each request in one piece


def _slices(step: StepInputs, heads: int, d: int, dv: int, delta: bool, name: str) -> dict:
    """Keyword arguments of ``ops.gated_memory`` for a step that runs over time slices, or none."""
    if step.max_q_len < SLICED_FROM or step.workspace is None:
        return {}
    need = -(-step.max_q_len // SLICE_LEN) * step.n_seqs * ops.gated_memory_slice_floats(heads, d, dv, delta)
    if need * 4 > SLICE_SCRATCH_LIMIT:
        return {}
    return dict(max_q_len=step.max_q_len, slice_len=SLICE_LEN, slice_S=step.workspace.get(name, need, torch.float32))


class GatedDeltaMixer:
    def __init__(self, *, hidden_size: int, num_heads: int, num_qk_heads: int, head_dim: int, value_dim: int, conv_taps: int,
                 eps: float, unit_eps: float = 1e-6, names: dict[str, str] | None = None, dtype: torch.dtype,
                 device: torch.device):
        if num_heads % num_qk_heads:
            raise ValueError(f"heads ({num_heads}) must be a multiple of q/k heads ({num_qk_heads})")
        if head_dim > 512:
            raise ValueError("memories of up to 512 rows per head are built")
        if not 0 <= conv_taps <= 16:
            raise ValueError(f"convolutions of up to 16 taps are built, got {conv_taps}")
        lib.prefer("delta")
        self.hidden_size, self.nh, self.nqk, self.d, self.dv = hidden_size, num_heads, num_qk_heads, head_dim, value_dim
        # conv_taps 0: no convolution and no tensors of it (q, k, v go through silu alone)
        self.has_conv, self.taps = conv_taps > 0, max(int(conv_taps), 1)
        self.eps, self.unit_eps = float(eps), float(unit_eps)
        self.dtype, self.device = dtype, device
        self.names = {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "beta": "b",
                      "a": "a", "A_log": "A_log", "dt_bias": "dt_bias", "g": "g", "norm": "norm", "o": "o", **(names or {})}
        self.qk, self.inner = num_qk_heads * head_dim, num_heads * value_dim
        self.conv_width = 2 * self.qk + self.inner
        # columns of the projection: [q | k | v | beta | a | g]
        self.col = {"q": 0, "k": self.qk, "v": 2 * self.qk, "beta": self.conv_width, "a": self.conv_width + num_heads,
                    "g": self.conv_width + 2 * num_heads}
        self.proj_width = self.conv_width + 2 * num_heads + self.inner
        self.carry = (self.taps - 1) * self.conv_width
        self.memory_off = -(-self.carry // 4) * 4             # the memories start on 16 bytes
        self.w_in = self.w_o = self.w_conv = self.w_norm = self.A_log = self.dt_bias = None
        self._scales: set[float] = set()
        self._scaled: dict[float, torch.Tensor] = {}

    def weight_specs(self) -> list[WeightSpec]:
        n, W, nh = self.names, self.hidden_size, self.nh
        specs = [WeightSpec(n["q"], (self.qk, W), init=("normal", 0.05)), WeightSpec(n["k"], (self.qk, W), init=("normal", 0.05)),
                 WeightSpec(n["v"], (self.inner, W), init=("normal", 0.05))]
        if self.has_conv:
            specs += [WeightSpec(n[f"{x}_conv"], (size, self.taps), dtype="float32", init=("normal", 0.3, 1.0 / self.taps))
                      for x, size in (("q", self.qk), ("k", self.qk), ("v", self.inner))]
        specs += [WeightSpec(n["beta"], (nh, W), init=("normal", 0.05)), WeightSpec(n["a"], (nh, W), init=("normal", 0.05)),
                  WeightSpec(n["A_log"], (nh,), dtype="float32", init=("normal", 0.5, -1.0)),
                  WeightSpec(n["dt_bias"], (nh,), dtype="float32", init=("normal", 0.5)),
                  WeightSpec(n["g"], (self.inner, W), init=("normal", 0.05)),
                  WeightSpec(n["norm"], (self.dv,), dtype="float32", init=("ones_plus_normal", 0.1)),
                  WeightSpec(n["o"], (W, self.inner), init=("normal", 0.05))]
        return specs

    def cache_need(self):
        return None

    def state_need(self) -> StateNeed:
        return StateNeed((self.memory_off + ops.gated_memory_state_floats(self.nh, self.d, self.dv),), "float32")

    def activation_bytes(self, n_tokens: int) -> int:
        elt = 4 if self.dtype == torch.float32 else 2
        return n_tokens * ((self.proj_width + self.conv_width + 2 * self.nh + self.inner) * 4 + (self.inner + self.hidden_size) * elt)

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        n = self.names
        self.w_in = torch.cat([tensors[n[k]] for k in ("q", "k", "v", "beta", "a", "g")], dim=0).contiguous()
        if self.has_conv:
            self.w_conv = torch.cat([tensors[n[f"{x}_conv"]] for x in "qkv"], dim=0).contiguous()
        else:       # one tap that weighs one: the kernel's activation alone
            self.w_conv = torch.ones((self.conv_width, 1), dtype=torch.float32, device=self.device)
        self.w_o, self.A_log, self.dt_bias = tensors[n["o"]], tensors[n["A_log"]], tensors[n["dt_bias"]]
        self.w_norm = tensors[n["norm"]].repeat(self.nh).contiguous()       # the kernel reads one weight per output number
        self._scaled = {s: (self.w_norm * s).contiguous() for s in self._scales}

    def projection_weight(self) -> torch.Tensor:
        """[proj_width, hidden] rows [q; k; v; beta; a; g]: what a shared product multiplies for this mixer."""
        return self.w_in

    @property
    def output_width(self) -> int:
        return self.inner

    def output_weight(self) -> torch.Tensor:
        """[hidden, heads * vdim]: what multiplies the normed and gated heads (``forward_projected(heads_out=)`` leaves them)."""
        return self.w_o

    def use_output_scale(self, scale: float) -> None:
        """Announce, before the weights are bound, a constant that ``forward_projected(out_scale=)`` will be called with:
        the heads' norm weight times it is made when the weights are bound (never inside a step, which a graph may be
        capturing)."""
        self._scales.add(float(scale))

    def _norm_weight(self, scale: float) -> torch.Tensor:
        if scale == 1.0:
            return self.w_norm
        if scale not in self._scaled:
            raise ValueError(f"output scale {scale} was not announced through use_output_scale before the weights were bound")
        return self._scaled[scale]

    def forward(self, x: torch.Tensor, step: StepInputs, cache: LayerCache) -> torch.Tensor:
        return self.forward_projected(ops.linear32(x, self.w_in), step, cache)

    def forward_projected(self, proj: torch.Tensor, step: StepInputs, cache: LayerCache, *,
                          heads_out: torch.Tensor | None = None, out_scale: float = 1.0) -> torch.Tensor | None:
        """``proj`` [T, proj_width] float32 (a view of a wider product is fine). ``heads_out`` [T, heads * vdim] (columns of
        a wider matrix): the normed and gated heads times ``out_scale`` are left there and the output product is the
        caller's."""
        T, dev, c = proj.shape[0], proj.device, self.col
        off = cache.state_off
        qkv = torch.empty((T, self.conv_width), dtype=torch.float32, device=dev)
        ops.short_conv_state(proj, 0, self.w_conv, None, cache.state, off, step.cu_q, step.seq_of_token, step.state_slots, qkv,
                             activation="silu")
        gb = torch.empty((T, 2 * self.nh), dtype=torch.float32, device=dev)
        ops.delta_prepare(qkv, c["q"], c["k"], self.nqk, self.d, self.d ** -0.5, self.unit_eps, proj, c["beta"], c["a"],
                          self.A_log, self.dt_bias, self.nh, gb)
        y = torch.empty((T, self.inner), dtype=torch.float32, device=dev)
        ops.gated_memory(qkv, q_col=c["q"], k_col=c["k"], v_col=c["v"], gb=gb, rule="delta", state=cache.state,
                         state_off=off + self.memory_off, cu_q=step.cu_q, state_slots=step.state_slots, y=y,
                         n_seqs=step.n_seqs, heads=self.nh, qk_heads=self.nqk, dim=self.d, vdim=self.dv,
                         **_slices(step, self.nh, self.d, self.dv, True, "delta_slice_memories"))
        gated = heads_out if heads_out is not None else torch.empty((T, self.inner), dtype=self.dtype, device=dev)
        ops.head_norm_gate(y, proj[:, c["g"]:c["g"] + self.inner], self._norm_weight(out_scale), self.eps, self.nh, gated,
                           gate_act="silu")
        return ops.linear(gated, self.w_o) if heads_out is None else None


class ForgetGateMemoryMixer:
    def __init__(self, *, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, eps: float,
                 names: dict[str, str] | None = None, dtype: torch.dtype, device: torch.device):
        if head_dim > 512:
            raise ValueError("memories of up to 512 rows per head are built")
        lib.prefer("delta")
        self.hidden_size, self.nh, self.d, self.dv, self.eps = hidden_size, num_heads, head_dim, value_dim, float(eps)
        self.dtype, self.device = dtype, device
        self.names = {"q": "q", "f": "f", "f_bias": "f.b", "lower": "lower", "v": "v", "norm": "norm", "o": "o", **(names or {})}
        self.qk, self.inner = num_heads * head_dim, num_heads * value_dim
        self.col = {"q": 0, "f": self.qk, "v": 2 * self.qk}        # columns of the projection
        self.proj_width = 2 * self.qk + self.inner
        self.w_in = self.w_o = self.b_f = self.low = self.w_norm = None

    def weight_specs(self) -> list[WeightSpec]:
        n, W = self.names, self.hidden_size
        return [WeightSpec(n["q"], (self.qk, W), init=("normal", 0.05)), WeightSpec(n["f"], (self.qk, W), init=("normal", 0.05)),
                WeightSpec(n["f_bias"], (self.qk,), dtype="float32", init=("normal", 1.0, 1.0)),
                WeightSpec(n["lower"], (self.qk,), dtype="float32", init=("uniform", 0.0, 0.9)),
                WeightSpec(n["v"], (self.inner, W), init=("normal", 0.05)),
                WeightSpec(n["norm"], (self.dv,), dtype="float32", init=("ones_plus_normal", 0.1)),
                WeightSpec(n["o"], (W, self.inner), init=("normal", 0.05))]

    def cache_need(self):
        return None

    def state_need(self) -> StateNeed:
        return StateNeed((ops.gated_memory_state_floats(self.nh, self.d, self.dv),), "float32")

    def activation_bytes(self, n_tokens: int) -> int:
        elt = 4 if self.dtype == torch.float32 else 2
        return n_tokens * ((self.proj_width + self.inner) * 4 + (self.inner + self.hidden_size) * elt)

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        n = self.names
        self.w_in = torch.cat([tensors[n[k]] for k in ("q", "f", "v")], dim=0).contiguous()
        self.w_o, self.b_f, self.low = tensors[n["o"]], tensors[n["f_bias"]], tensors[n["lower"]]
        self.w_norm = tensors[n["norm"]].repeat(self.nh).contiguous()

    def projection_weight(self) -> torch.Tensor:
        return self.w_in

    def forward(self, x: torch.Tensor, step: StepInputs, cache: LayerCache) -> torch.Tensor:
        return self.forward_projected(ops.linear32(x, self.w_in), step, cache)

    def forward_projected(self, proj: torch.Tensor, step: StepInputs, cache: LayerCache) -> torch.Tensor:
        T, dev, c = proj.shape[0], proj.device, self.col
        ops.forget_gate_prepare(proj, c["q"], c["f"], self.qk, self.low, self.b_f)      # in place: q <- silu, f <- the gate
        y = torch.empty((T, self.inner), dtype=torch.float32, device=dev)
        ops.gated_memory(proj, q_col=c["q"], k_col=c["f"], v_col=c["v"], gb=None, rule="forget", state=cache.state,
                         state_off=cache.state_off, cu_q=step.cu_q, state_slots=step.state_slots, y=y, n_seqs=step.n_seqs,
                         heads=self.nh, qk_heads=self.nh, dim=self.d, vdim=self.dv,
                         **_slices(step, self.nh, self.d, self.dv, False, "forget_slice_memories"))
        normed = torch.empty((T, self.inner), dtype=self.dtype, device=dev)
        ops.head_norm_gate(y, None, self.w_norm, self.eps, self.nh, normed)
        return ops.linear(normed, self.w_o)


register_mixer("gated_delta", GatedDeltaMixer)
register_mixer("forget_gate_memory", ForgetGateMemoryMixer)
