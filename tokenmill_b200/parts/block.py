"""Pre-norm block: ``x = x + mixer(norm1(x)); x = x + feed_forward(norm2(x))``
(src/infer/model/qwen2.py:13-23).

The residual stream ``x`` is 32-bit. A branch output is not added where it is produced: it is
handed on as ``Pending`` and the next norm adds it while it reads the row anyway (one pass over the
stream instead of two). The embedding gather enters the same way, as the first pending item.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..registry import register_block
from .base import LayerCache, StepInputs


@dataclass
class Pending:
    """What still has to be added to the residual stream: a branch output, a stack of 32-bit partial
    products, or (at the very start) the embedding rows of the token ids."""

    branch: torch.Tensor | None = None
    partials: torch.Tensor | None = None
    ids: torch.Tensor | None = None
    table: torch.Tensor | None = None
    branch2: torch.Tensor | None = None      # a second branch output, and the multiplier of both (blocks whose
    scale: float = 1.0                        # branches read the same stream; norms that take them: RMSNorm32)
    gate: torch.Tensor | None = None         # 32-bit pre-activations of a gate on the branch, and the gate's bias
    gate_bias: torch.Tensor | None = None    # (norms that take them: GatedAddRMSNorm)
    table_scale: float = 1.0                  # multiplier of the embedding rows (norms that read ``table``)
    positions: torch.Tensor | None = None    # a learned vector per position, added to the embedding rows
    pos_table: torch.Tensor | None = None    # (norms that take them: DynamicTanhNorm)
    row_scale: torch.Tensor | None = None    # [T] float32: branch2 enters as row_scale[t] * branch2[t] (the same norms)
    stream_mix: torch.Tensor | None = None   # several residual streams: how the branch enters them, x_t <- sum_s
    stream_out: torch.Tensor | None = None   # mix[s, t] x_s + out[t] y (blocks with hyper-connections set them)

    @classmethod
    def of(cls, y) -> "Pending":
        """A part's output: [T, H] in the activation dtype, or [n, T, H] float32 partial products of a
        matrix product whose K range was cut (the norm that follows adds them up in index order), or None
        when the part has added its output into the stream itself; a ``Pending`` passes through."""
        if y is None:
            return cls()
        if isinstance(y, cls):
            return y
        return cls(partials=y) if y.dim() == 3 else cls(branch=y)

    def kwargs(self) -> dict:
        kw = {"branch": self.branch, "partials": self.partials, "ids": self.ids, "table": self.table}
        if self.row_scale is not None:
            kw.update(branch2=self.branch2, row_scale=self.row_scale)
        elif self.branch2 is not None or self.scale != 1.0:
            kw.update(branch2=self.branch2, scale=self.scale)
        if self.gate is not None:
            kw.update(gate=self.gate, gate_bias=self.gate_bias)
        if self.table_scale != 1.0 and self.table is not None:
            kw.update(table_scale=self.table_scale)
        if self.pos_table is not None and self.table is not None:
            kw.update(positions=self.positions, pos_table=self.pos_table)
        if self.stream_mix is not None:
            kw.update(stream_mix=self.stream_mix, stream_out=self.stream_out)
        return kw


class PreNormBlock:
    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm

    def forward(self, resid: torch.Tensor, pending: Pending, step: StepInputs, cache: LayerCache) -> Pending:
        # A part that says ``adds_to_residual`` is offered the stream: it may add its output there itself (its
        # last product's epilogue) and return None; the norm that follows then has nothing left to add.
        normed = self.mixer_norm.forward(resid, **pending.kwargs())
        offer = {"residual": resid} if getattr(self.mixer, "adds_to_residual", False) else {}
        mixed = Pending.of(self.mixer.forward(normed, step, cache, **offer))
        normed = self.feed_forward_norm.forward(resid, **mixed.kwargs())
        offer = {"residual": resid} if getattr(self.feed_forward, "adds_to_residual", False) else {}
        return Pending.of(self.feed_forward.forward(normed, step, **offer))


    def emit(self, b, resid, pending: dict, cache: LayerCache) -> dict:
        """The block's launches written into a step program (kernels/program.py). ``pending`` holds what the
        first norm still has to add to the stream (``branch``: a workspace buffer, or ``ids`` and ``table``);
        returns the same for the norm that follows the block."""
        T = b.tokens()
        normed = self.mixer_norm.emit(b, resid, n_rows=T, **pending)
        mixed = self.mixer.emit(b, normed, cache)
        normed = self.feed_forward_norm.emit(b, resid, n_rows=T, branch=mixed)
        return {"branch": self.feed_forward.emit(b, normed)}


class ParallelShiftBlock:
    """``x <- x + m * (mixer(shift(norm1(x))) + feed_forward(norm2(x)))``: both branches read the same stream, the
    sum is scaled by ``residual_mult``, and the mixer's input passes a token shift first:
    ``h_t <- h_t + (h_{t-1} - h_t) * mu`` with the learned vector ``mu`` (tensor ``shift`` of the layer), h_{t-1}
    the previous token's h before its own replacement, zeros before a sequence's first token. The last h of every
    request is per-request state of the block (one row of the hidden size in 32-bit), so a prompt may be cut
    anywhere. The feed-forward may be absent. One kernel adds the previous block's two branch outputs to the
    stream and writes both norms; the norms are ``RMSNorm32`` parts."""

    wants_run_context = True

    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm, *, hidden_size: int, residual_mult: float = 1.0,
                 token_shift: bool = True, shift_name: str = "shift", dtype: torch.dtype, device: torch.device):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        self.hidden_size, self.mult, self.shifts, self.shift_name = hidden_size, float(residual_mult), token_shift, shift_name
        self.dtype, self.device = dtype, device
        self.mu: torch.Tensor | None = None

    def weight_specs(self):
        from .spec import WeightSpec
        return [WeightSpec(self.shift_name, (self.hidden_size,), dtype="float32", init=("normal", 0.3, 0.5))] if self.shifts else []

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        if self.shifts:
            self.mu = tensors[self.shift_name]

    def state_need(self):
        from .spec import StateNeed
        return StateNeed((self.hidden_size,), "float32") if self.shifts else None

    def forward(self, resid: torch.Tensor, pending: Pending, step: StepInputs, cache: LayerCache) -> Pending:
        from ..kernels import ops
        if self.feed_forward is not None:
            h, g = self.mixer_norm.forward(resid, pair=self.feed_forward_norm, raw=self.shifts, **pending.kwargs())
        else:
            h, g = self.mixer_norm.forward(resid, raw=self.shifts, **pending.kwargs()), None
        if self.shifts:
            shifted = torch.empty(h.shape, dtype=self.dtype, device=h.device)
            h = ops.token_shift(h, self.mu, cache.block_state, step.cu_q, step.seq_of_token, step.state_slots, shifted)
        mixed = self.mixer.forward(h, step, cache)
        fed = self.feed_forward.forward(g, step) if self.feed_forward is not None else None
        return Pending(branch=mixed, branch2=fed, scale=self.mult)


class ParallelBlock:
    """``x <- x + (mixer(h) + feed_forward(h))`` with ``h = norm(x)``: ONE norm, and both sublayers read its output. Neither
    result is added where it is produced: the next norm takes both as two branches and adds their sum while it reads
    the row (a norm that takes ``branch`` and ``branch2``). The feed-forward may be absent."""

    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm=None):
        if feed_forward_norm is not None:
            raise ValueError("a parallel block has one norm; its feed-forward reads the mixer's")
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, None

    def forward(self, resid: torch.Tensor, pending: Pending, step: StepInputs, cache: LayerCache) -> Pending:
        h = self.mixer_norm.forward(resid, **pending.kwargs())
        mixed = self.mixer.forward(h, step, cache)
        fed = self.feed_forward.forward(h, step) if self.feed_forward is not None else None
        return Pending(branch=mixed, branch2=fed)


class ConvGatedBlock:
    """Pre-norm block with two additions. Each sublayer reads its normed input h through a short causal convolution
    over time, ``h + conv(h)`` with ``conv(h)_t = sum_j w[:, j] h_(t - taps + 1 + j)`` per channel (tensors ``canon1`` and
    ``canon2`` of the layer, [width, taps]); and each sublayer's result enters the stream through a learned gate,
    ``x <- x + sigmoid(W h + b) * sublayer(h + conv(h))`` (``rg1`` / ``rg1.b`` for the mixer, ``rg2`` / ``rg2.b`` for the
    feed-forward), the gate reading h before the convolution. The last ``taps - 1`` inputs of both convolutions are
    per-request state of the block ([2, taps - 1, width] in 32-bit), so a sequence may be cut anywhere. The gate's
    product keeps its 32-bit accumulator; the norm that follows (``GatedAddRMSNorm``) applies the sigmoid and adds the
    gated branch while it reads the row. The feed-forward may be absent."""

    wants_run_context = True

    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm, *, hidden_size: int, taps: int,
                 names: dict[str, str] | None = None, dtype: torch.dtype, device: torch.device):
        if not 1 <= taps <= 16:
            raise ValueError(f"input convolutions of 1 to 16 taps are built, got {taps}")
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        self.hidden_size, self.taps = hidden_size, int(taps)
        self.dtype, self.device = dtype, device
        self.names = {"conv1": "canon1", "conv2": "canon2", "gate1": "rg1", "gate1_bias": "rg1.b", "gate2": "rg2",
                      "gate2_bias": "rg2.b", **(names or {})}
        self.carry = (self.taps - 1) * hidden_size
        self.w_conv: list = [None, None]
        self.w_gate: list = [None, None]
        self.b_gate: list = [None, None]

    def _sides(self) -> list[int]:
        return [1] if self.feed_forward is None else [1, 2]

    def weight_specs(self):
        from .spec import WeightSpec
        H, n, out = self.hidden_size, self.names, []
        for i in self._sides():
            out += [WeightSpec(n[f"conv{i}"], (H, self.taps), dtype="float32", init=("normal", 0.2)),
                    WeightSpec(n[f"gate{i}"], (H, H), init=("normal", 0.05)),
                    WeightSpec(n[f"gate{i}_bias"], (H,), dtype="float32", init=("normal", 0.5))]
        return out

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        for i in self._sides():
            self.w_conv[i - 1] = tensors[self.names[f"conv{i}"]]
            self.w_gate[i - 1] = tensors[self.names[f"gate{i}"]]
            self.b_gate[i - 1] = tensors[self.names[f"gate{i}_bias"]]

    def state_need(self):
        from .spec import StateNeed
        return StateNeed((2 * self.carry,), "float32") if self.taps > 1 else None

    def _read(self, h: torch.Tensor, side: int, step: StepInputs, cache: LayerCache):
        """(gate pre-activations [T, H] float32, h + conv(h)) of one sublayer."""
        from ..kernels import ops
        gate = ops.linear32(h, self.w_gate[side])
        if self.taps == 1:          # one tap: conv(h) = w h, nothing is carried (the kernel never touches the state)
            state = torch.empty((1, 0), dtype=torch.float32, device=h.device)
        else:
            state = cache.block_state[:, side * self.carry:(side + 1) * self.carry]
        return gate, ops.canon_conv(h, self.w_conv[side], state, step.cu_q, step.seq_of_token, step.state_slots,
                                    torch.empty_like(h))

    def forward(self, resid: torch.Tensor, pending: Pending, step: StepInputs, cache: LayerCache) -> Pending:
        h = self.mixer_norm.forward(resid, **pending.kwargs())
        gate, hc = self._read(h, 0, step, cache)
        out = Pending(branch=self.mixer.forward(hc, step, cache), gate=gate, gate_bias=self.b_gate[0])
        if self.feed_forward is None:
            return out
        h = self.feed_forward_norm.forward(resid, **out.kwargs())
        gate, hc = self._read(h, 1, step, cache)
        return Pending(branch=self.feed_forward.forward(hc, step), gate=gate, gate_bias=self.b_gate[1])


class HyperConnectionBlock:
    """Pre-norm block over several residual streams (hyper-connections). A token carries ``streams`` copies x_1 .. x_s of
    the stream, all equal where the model starts. Sublayer q (1: mixer, 2: feed-forward) reads them as
    ``u = sum_s in_q[s] x_s``, runs on ``norm(u)``, and its result y enters all streams at once from the old ones:
    ``x_t <- sum_s mix_q[s, t] x_s + out_q[t] y`` (mix is indexed [from, to]). The tensors are ``hc1.in``, ``hc1.out``,
    ``hc1.mix`` and ``hc2.*`` of the layer, 32-bit. Neither the read nor the write is a pass of its own: the norm in
    front of a sublayer (a norm that takes ``stream_in`` / ``stream_mix`` / ``stream_out``, such as ``DynamicTanhNorm``)
    first takes in the previous sublayer's result and then reads, in one pass over the row. With one stream and
    mix = out = in = 1 this is the plain pre-norm block. The feed-forward may be absent. A feed-forward that can hand
    over its result in two pieces (``forward_parts``: a branch, and a second one with a weight per token) is taken that
    way, so that the sum happens in the same pass."""

    wants_run_context = True

    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm, *, hidden_size: int, streams: int,
                 learned: bool = True, names: dict[str, str] | None = None, dtype: torch.dtype, device: torch.device):
        if streams < 1:
            raise ValueError(f"a block has at least one residual stream, got {streams}")
        if not learned and streams != 1:
            raise ValueError("several residual streams need their learned read and write weights")
        self.learned = bool(learned)     # False: one stream read and written as it is (no tensors): the plain block
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        self.hidden_size, self.streams = hidden_size, int(streams)
        self.dtype, self.device = dtype, device
        self.names = {"in1": "hc1.in", "out1": "hc1.out", "mix1": "hc1.mix", "in2": "hc2.in", "out2": "hc2.out",
                      "mix2": "hc2.mix", **(names or {})}
        self.w_in: list = [None, None]
        self.w_out: list = [None, None]
        self.w_mix: list = [None, None]

    def _sides(self) -> list[int]:
        return [1] if self.feed_forward is None else [1, 2]

    def weight_specs(self):
        from .spec import WeightSpec
        s, n, out = self.streams, self.names, []
        for i in self._sides() if self.learned else []:
            out += [WeightSpec(n[f"in{i}"], (s,), dtype="float32", init=("normal", 0.2, 1.0 / s)),
                    WeightSpec(n[f"out{i}"], (s,), dtype="float32", init=("normal", 0.2, 1.0)),
                    WeightSpec(n[f"mix{i}"], (s, s), dtype="float32", init=("normal", 0.2, 1.0 / s))]
        return out

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        for i in self._sides() if self.learned else []:
            self.w_in[i - 1] = tensors[self.names[f"in{i}"]]
            self.w_out[i - 1] = tensors[self.names[f"out{i}"]]
            self.w_mix[i - 1] = tensors[self.names[f"mix{i}"]]

    def _written(self, y, side: int) -> Pending:
        out = Pending.of(y)
        if out.partials is not None:
            raise NotImplementedError("several residual streams take branch outputs, not partial products")
        out.stream_mix, out.stream_out = self.w_mix[side], self.w_out[side]
        return out

    def forward(self, resid: torch.Tensor, pending: Pending, step: StepInputs, cache: LayerCache) -> Pending:
        h = self.mixer_norm.forward(resid, stream_in=self.w_in[0], **pending.kwargs())
        out = self._written(self.mixer.forward(h, step, cache), 0)
        if self.feed_forward is None:
            return out
        h = self.feed_forward_norm.forward(resid, stream_in=self.w_in[1], **out.kwargs())
        if callable(getattr(self.feed_forward, "forward_parts", None)):
            branch, branch2, row_scale = self.feed_forward.forward_parts(h, step)
            y = Pending(branch=branch, branch2=branch2, row_scale=row_scale) if branch2 is not None else branch
        else:
            y = self.feed_forward.forward(h, step)
        return self._written(y, 1)


register_block("conv_gated", ConvGatedBlock)
register_block("parallel", ParallelBlock)
register_block("hyper_connections", HyperConnectionBlock)
register_block("pre_norm", PreNormBlock)
register_block("parallel_shift", ParallelShiftBlock)
