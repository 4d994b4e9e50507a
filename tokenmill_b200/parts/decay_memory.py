"""Linear attention with a constant decay per head (lightning attention): per head a d x dv memory without gates.

From the mixer's input h: ``q = act(W_q h)``, ``k = act(W_k h)`` (heads x d), ``v = act(W_v h)`` (heads x dv), act = silu
by default. Per head, from S = 0:
    S_t = decay_h S_(t-1) + k_t v_t^T          o_t = S_t^T q_t
with one constant ``decay_h`` per head and no other scale. The heads side by side are RMS-normed together (one root mean
square over all heads x dv numbers, a plain weight), multiplied by sigmoid(W_g h), and projected by W_o. The memory, the
products and the norm are 32-bit in both run dtypes; the projections' product keeps its 32-bit accumulator. Per request
the mixer keeps S (a column's rows side by side, [heads, dv, d padded]) in ONE state slot of 32-bit floats, zero for a new request; prompt portions and single
decoded tokens run the same kernel, which walks a request's tokens in order whatever the cut. A step whose longest
portion has ``SLICED_FROM`` tokens runs three passes over time slices instead (the slices' own memories side by side,
then their start memories one after the other, then the slices again with the results): the same sums in another
order.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..registry import register_mixer
from .base import LayerCache, StepInputs
from .spec import StateNeed, WeightSpec


SLICED_FROM = 256               # a step whose longest portion has this many tokens runs over time slices
SLICE_LEN = 128
SLICE_SCRATCH_LIMIT = 1 << 28    # bytes of scratch the slices may take; beyond it a step walks each request in one piece


class DecayMemoryMixer:
    def __init__(self, *, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, decay: list[float], eps: float,
                 activation: str | None = "silu", names: dict[str, str] | None = None, dtype: torch.dtype,
                 device: torch.device):
        if len(decay) != num_heads:
            raise ValueError(f"one decay per head: {num_heads} heads, {len(decay)} decays")
        if head_dim > 512:
            raise ValueError("memories of up to 512 rows per head are built")
        self.hidden_size, self.nh, self.d, self.dv = hidden_size, num_heads, head_dim, value_dim
        self.eps, self.activation = float(eps), activation
        self.dtype, self.device = dtype, device
        self.names = {"q": "q", "k": "k", "v": "v", "g": "g", "norm": "norm", "o": "o", **(names or {})}
        self.qk, self.inner = num_heads * head_dim, num_heads * value_dim
        self.col = {"q": 0, "k": self.qk, "v": 2 * self.qk, "g": 2 * self.qk + self.inner}     # columns of the projection
        self.proj_width = 2 * self.qk + 2 * self.inner
        self.decay = torch.tensor([float(a) for a in decay], dtype=torch.float32, device=device)
        self.w_in = self.w_o = self.g = None

    def weight_specs(self) -> list[WeightSpec]:
        n, W = self.names, self.hidden_size
        return [WeightSpec(n["q"], (self.qk, W), init=("normal", 0.05)), WeightSpec(n["k"], (self.qk, W), init=("normal", 0.05)),
                WeightSpec(n["v"], (self.inner, W), init=("normal", 0.05)),
                WeightSpec(n["g"], (self.inner, W), init=("normal", 0.05)),
                WeightSpec(n["o"], (W, self.inner), init=("normal", 0.05)),
                WeightSpec(n["norm"], (self.inner,), dtype="float32", init=("ones_plus_normal", 0.1))]

    def cache_need(self):
        return None

    def state_need(self) -> StateNeed:
        return StateNeed((ops.decay_memory_state_floats(self.nh, self.d, self.dv),), "float32")

    def activation_bytes(self, n_tokens: int) -> int:
        elt = 4 if self.dtype == torch.float32 else 2
        return n_tokens * ((self.proj_width + self.inner) * 4 + (self.inner + self.hidden_size) * elt)

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        n = self.names
        self.w_in = torch.cat([tensors[n[k]] for k in ("q", "k", "v", "g")], dim=0).contiguous()
        self.w_o, self.g = tensors[n["o"]], tensors[n["norm"]]

    def forward(self, x: torch.Tensor, step: StepInputs, cache: LayerCache) -> torch.Tensor:
        T, dev, c = x.shape[0], x.device, self.col
        proj = ops.linear32(x, self.w_in)                                       # [T, q | k | v | g] float32
        y = torch.empty((T, self.inner), dtype=torch.float32, device=dev)
        sliced = {}
        if step.max_q_len >= SLICED_FROM and step.workspace is not None:
            need = -(-step.max_q_len // SLICE_LEN) * step.n_seqs * ops.decay_memory_state_floats(self.nh, self.d, self.dv)
            if need * 4 <= SLICE_SCRATCH_LIMIT:
                sliced = dict(max_q_len=step.max_q_len, slice_len=SLICE_LEN,
                              slice_S=step.workspace.get("decay_slice_memories", need, torch.float32))
        ops.decay_memory(proj, q_col=c["q"], k_col=c["k"], v_col=c["v"], activation=self.activation, decay=self.decay,
                         state=cache.state, state_off=0, cu_q=step.cu_q, state_slots=step.state_slots, y=y,
                         n_seqs=step.n_seqs, heads=self.nh, dim=self.d, vdim=self.dv, **sliced)
        gated = torch.empty((T, self.inner), dtype=self.dtype, device=dev)
        # one "head" of all the numbers: the heads are normed together
        ops.head_norm_gate(y, proj[:, c["g"]:c["g"] + self.inner], self.g, self.eps, 1, gated)
        return ops.linear(gated, self.w_o)


register_mixer("decay_memory", DecayMemoryMixer)
