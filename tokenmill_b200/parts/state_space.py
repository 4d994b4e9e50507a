"""Selective state-space mixer (the Mamba-2 form: one scalar decay per head and token).

From the mixer's input h: ``W_in h = [z (inner) | x (inner) | B (G N) | C (G N) | dt (heads)]`` with inner =
heads * vdim. x, B and C pass a short causal convolution per channel (bias, silu). Per head (head h reads group
h // (heads / G)), in 32-bit:
    dt = softplus(dt + dt_bias)          S <- exp(-exp(A_log) dt) S + dt B x^T          y = S^T C + D x
then y * silu(z), RMS norm in ``norm_groups`` equal parts (each by its own root mean square) times a weight, W_o.

Per request the mixer keeps, in ONE state slot of 32-bit floats: the last ``taps - 1`` inputs of the convolution
[(taps - 1), channels], then S [heads, vdim, N]. The slot is zero for a new request. Prompt portions and single
decoded tokens run through the same two kernels; the recurrence walks a request's tokens in order whatever the cut.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..registry import register_mixer
from .base import LayerCache, StepInputs
from .spec import StateNeed, WeightSpec


SLICED_FROM = 256       # a step whose longest portion has this many tokens runs the recurrence over time slices
SLICE_LEN = 128
SLICE_SCRATCH_LIMIT = 1 << 28    # bytes of scratch the selective scan's slices may take; beyond it a step walks each
                                 # request in one piece
VECTOR_CONV_FROM = 16   # steps whose longest portion is shorter are mostly rows that own a slot: a thread per channel
                        # (8 decoded tokens at 2,560 channels: 5 us against 14 with eight channels a thread)


class StateSpaceMixer:
    def __init__(self, *, hidden_size: int, num_heads: int, value_dim: int, state_size: int, groups: int, conv_taps: int,
                 norm_groups: int, eps: float, names: dict[str, str] | None = None, dtype: torch.dtype,
                 device: torch.device):
        if num_heads % groups:
            raise ValueError(f"heads ({num_heads}) must be a multiple of groups ({groups})")
        self.hidden_size, self.nh, self.dv, self.N, self.G = hidden_size, num_heads, value_dim, state_size, groups
        self.taps, self.norm_groups, self.eps = conv_taps, norm_groups, float(eps)
        self.inner = num_heads * value_dim
        if self.inner % norm_groups:
            raise ValueError(f"inner size ({self.inner}) must be a multiple of norm_groups ({norm_groups})")
        if not 1 <= conv_taps <= 16 or state_size > 256:
            raise ValueError("convolutions of 1 to 16 taps and states of up to 256 per column are built")
        self.channels = self.inner + 2 * groups * state_size
        self.proj_width = 2 * self.inner + 2 * groups * state_size + num_heads
        self.conv_len = (conv_taps - 1) * self.channels
        self.dtype, self.device = dtype, device
        self.names = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "A_log": "A_log", "D": "D",
                      "norm": "norm", "o": "o", **(names or {})}
        self.w_in = self.w_conv = self.w_conv_t = self.b_conv = self.dt_bias = self.A_log = self.D = self.g = self.w_o = None

    def weight_specs(self) -> list[WeightSpec]:
        n, H = self.names, self.hidden_size
        f32 = dict(dtype="float32")
        return [WeightSpec(n["in"], (self.proj_width, H), init=("normal", 0.05)),
                WeightSpec(n["conv"], (self.channels, self.taps), init=("normal", 0.3), **f32),
                WeightSpec(n["conv_bias"], (self.channels,), init=("normal", 0.1), **f32),
                WeightSpec(n["dt_bias"], (self.nh,), init=("normal", 0.5), **f32),
                WeightSpec(n["A_log"], (self.nh,), init=("normal", 0.5), **f32),
                WeightSpec(n["D"], (self.nh,), init=("ones_plus_normal", 0.2), **f32),
                WeightSpec(n["norm"], (self.inner,), init=("ones_plus_normal", 0.1), **f32),
                WeightSpec(n["o"], (H, self.inner), init=("normal", 0.05))]

    def cache_need(self):
        return None

    def state_need(self) -> StateNeed:
        return StateNeed((self.conv_len + self.nh * self.dv * self.N,), "float32")

    def activation_bytes(self, n_tokens: int) -> int:
        elt = 4 if self.dtype == torch.float32 else 2
        return n_tokens * ((self.proj_width + self.channels + self.inner + self.hidden_size) * elt + self.inner * 4)

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        n = self.names
        self.w_in, self.w_o = tensors[n["in"]], tensors[n["o"]]
        self.w_conv, self.b_conv = tensors[n["conv"]], tensors[n["conv_bias"]]
        self.w_conv_t = self.w_conv.t().contiguous()          # [taps, channels], for the kernel's 16-byte loads
        self.dt_bias, self.A_log, self.D, self.g = tensors[n["dt_bias"]], tensors[n["A_log"]], tensors[n["D"]], tensors[n["norm"]]

    def forward(self, x: torch.Tensor, step: StepInputs, cache: LayerCache) -> torch.Tensor:
        T, dev = x.shape[0], x.device
        proj = ops.linear(x, self.w_in)                                       # [T, z | x | B | C | dt]
        xbc = torch.empty((T, self.channels), dtype=self.dtype, device=dev)
        ops.conv_silu_state(proj, self.inner, self.channels, self.w_conv, self.b_conv, cache.state, step.cu_q,
                            step.seq_of_token, step.state_slots, xbc,
                            weight_t=self.w_conv_t if step.max_q_len >= VECTOR_CONV_FROM else None)
        y = torch.empty((T, self.inner), dtype=torch.float32, device=dev)
        # Long portions: three passes over time slices instead of one walk over the whole portion (kernels/ops.py).
        sliced = {}
        if step.max_q_len >= SLICED_FROM and step.workspace is not None:
            slices = -(-step.max_q_len // SLICE_LEN) * step.n_seqs
            sliced = dict(slice_len=SLICE_LEN,
                          slice_S=step.workspace.get("ssm_slice_states", slices * self.nh * self.dv * self.N, torch.float32),
                          slice_a=step.workspace.get("ssm_slice_decays", slices * self.nh, torch.float32))
        ops.ssm_scan(xbc, proj, self.inner + self.channels, self.A_log, self.dt_bias, self.D, cache.state, self.conv_len,
                     step.cu_q, step.state_slots, y, n_seqs=step.n_seqs, heads=self.nh, vdim=self.dv, N=self.N,
                     groups=self.G, max_q_len=step.max_q_len, **sliced)
        gated = torch.empty((T, self.inner), dtype=self.dtype, device=dev)
        ops.gated_group_norm(y, proj, self.g, self.eps, self.norm_groups, gated)
        return ops.linear(gated, self.w_o)


class SelectiveScanMixer:
    """Selective state-space mixer in its first form (Mamba): a step size per channel and a decay per (channel, state).

    ``W_in h = [x (inner) | z (inner)]``; x passes a causal convolution per channel (bias, silu). ``W_x x = [low (rank) |
    B (N) | C (N)]``, ``dt = softplus(W_dt low + b_dt)`` per channel, ``A = -exp(A_log)`` [inner, N]. Per channel c and
    state n, in 32-bit: ``S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n``, ``y_c = sum_n S[c, n] C_n + D_c x_c``;
    then ``y silu(z)`` and W_o. ``W_x``'s product keeps its 32-bit accumulator and the rank-sized product with W_dt
    happens inside the scan kernel in 32-bit, so nothing that enters the recurrence is rounded on the way.

    Per request the mixer keeps, in ONE state slot of 32-bit floats: the last ``taps - 1`` inputs of the convolution
    [(taps - 1), inner], then S [inner, N]; zero for a new request. The recurrence walks a request's tokens in order
    whatever the cut; a step whose longest portion has ``SLICED_FROM`` tokens runs three passes over time slices instead
    (a slice's decays multiply to exp(A times the sum of its step sizes)): the same sums in another order."""

    def __init__(self, *, hidden_size: int, inner: int, state_size: int, dt_rank: int, conv_taps: int,
                 names: dict[str, str] | None = None, dtype: torch.dtype, device: torch.device):
        if not 1 <= conv_taps <= 16 or state_size > 256:
            raise ValueError("convolutions of 1 to 16 taps and up to 256 states per channel are built")
        self.hidden_size, self.inner, self.N, self.rank, self.taps = hidden_size, inner, state_size, dt_rank, conv_taps
        self.conv_len = (conv_taps - 1) * inner
        self.dtype, self.device = dtype, device
        self.names = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "x": "x", "dt": "dt", "dt_bias": "dt.b",
                      "A_log": "A_log", "D": "D", "o": "o", **(names or {})}
        self.w_in = self.w_conv = self.w_conv_t = self.b_conv = self.w_x = self.w_dt = self.b_dt = self.A_log = self.D = None
        self.w_o = None

    def weight_specs(self) -> list[WeightSpec]:
        n, H, I = self.names, self.hidden_size, self.inner
        f32 = dict(dtype="float32")
        return [WeightSpec(n["in"], (2 * I, H), init=("normal", 0.05)),
                WeightSpec(n["conv"], (I, self.taps), init=("normal", 0.3), **f32),
                WeightSpec(n["conv_bias"], (I,), init=("normal", 0.1), **f32),
                WeightSpec(n["x"], (self.rank + 2 * self.N, I), init=("normal", 0.1)),
                WeightSpec(n["dt"], (I, self.rank), init=("normal", 0.3), **f32),
                WeightSpec(n["dt_bias"], (I,), init=("normal", 0.5, -1.0), **f32),
                WeightSpec(n["A_log"], (I, self.N), init=("normal", 0.5), **f32),
                WeightSpec(n["D"], (I,), init=("ones_plus_normal", 0.2), **f32),
                WeightSpec(n["o"], (H, I), init=("normal", 0.05))]

    def cache_need(self):
        return None

    def state_need(self) -> StateNeed:
        return StateNeed((self.conv_len + self.inner * self.N,), "float32")

    def activation_bytes(self, n_tokens: int) -> int:
        elt = 4 if self.dtype == torch.float32 else 2
        return n_tokens * ((4 * self.inner + self.hidden_size) * elt + (self.rank + 2 * self.N) * 4)

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        n = self.names
        self.w_in, self.w_x, self.w_o = tensors[n["in"]], tensors[n["x"]], tensors[n["o"]]
        self.w_conv, self.b_conv = tensors[n["conv"]], tensors[n["conv_bias"]]
        self.w_conv_t = self.w_conv.t().contiguous()          # [taps, inner], for the kernel's 16-byte loads
        self.w_dt, self.b_dt, self.A_log, self.D = tensors[n["dt"]], tensors[n["dt_bias"]], tensors[n["A_log"]], tensors[n["D"]]

    def forward(self, x: torch.Tensor, step: StepInputs, cache: LayerCache) -> torch.Tensor:
        T, dev = x.shape[0], x.device
        proj = ops.linear(x, self.w_in)                                       # [T, x | z]
        xc = torch.empty((T, self.inner), dtype=self.dtype, device=dev)
        ops.conv_silu_state(proj, 0, self.inner, self.w_conv, self.b_conv, cache.state, step.cu_q, step.seq_of_token,
                            step.state_slots, xc, weight_t=self.w_conv_t if step.max_q_len >= VECTOR_CONV_FROM else None)
        dbc = ops.linear32(xc, self.w_x)                                      # [T, low | B | C] float32
        gated = torch.empty((T, self.inner), dtype=self.dtype, device=dev)
        sliced = {}
        if step.max_q_len >= SLICED_FROM and step.workspace is not None:
            slices = -(-step.max_q_len // SLICE_LEN) * step.n_seqs
            if slices * self.inner * (self.N + 1) * 4 <= SLICE_SCRATCH_LIMIT:
                sliced = dict(max_q_len=step.max_q_len, slice_len=SLICE_LEN,
                              slice_S=step.workspace.get("scan_slice_states", slices * self.inner * self.N, torch.float32),
                              slice_dt=step.workspace.get("scan_slice_steps", slices * self.inner, torch.float32))
        ops.selective_scan(xc, proj, self.inner, dbc, self.w_dt, self.b_dt, self.A_log, self.D, cache.state, self.conv_len,
                           step.cu_q, step.state_slots, gated, n_seqs=step.n_seqs, rank=self.rank, N=self.N, **sliced)
        return ops.linear(gated, self.w_o)


register_mixer("selective_scan", SelectiveScanMixer)
register_mixer("state_space", StateSpaceMixer)
