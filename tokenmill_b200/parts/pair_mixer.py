"""Two mixers side by side: both read the same input. ``combine="norm_mean"``: the result is half the sum of their
outputs, each first RMS-normed over the model width with a plain weight of its own (``<left>.out`` / ``<right>.out``).
``combine="weighted"``: ``left_scale * left + right_scale * right`` with two constants and no tensors of the pair's own.

The two may be any registered mixers; their tensors live under the sub-prefixes ``left`` and ``right``. At most one of
them keeps pages: the pair hands its ``LayerCache`` to both. Both may keep per-request state: a request's slot then
holds the left one's floats followed by the right one's (padded to a multiple of four), and each side finds its share
through ``LayerCache.state_off`` (a side that ignores the offset must be the only one with state, or the left). Mixers
that can take their columns of a shared product (``projection_weight`` / ``forward_projected``) are fed from ONE matrix
product over the concatenated weights, which keeps its 32-bit accumulator. With ``combine="weighted"``, mixers that can
leave what their output projection reads in columns of a shared matrix, times a constant (``output_width`` /
``output_weight()`` / ``forward_projected(..., heads_out=, out_scale=)``), share ONE output product as well:
``[left_scale * a | right_scale * b] [W_o,left | W_o,right]^T`` is the weighted sum, summed in the product's 32-bit
accumulator.
"""

from __future__ import annotations

import dataclasses

import torch

from ..kernels import ops
from ..registry import get_part, register_mixer
from .base import LayerCache, StepInputs, part_activation_bytes
from .spec import PartSpec, StateNeed, WeightSpec


class PairMixer:
    def __init__(self, *, hidden_size: int, eps: float, left: PartSpec, right: PartSpec, names: dict[str, str] | None = None,
                 combine: str = "norm_mean", left_scale: float = 1.0, right_scale: float = 1.0, dtype: torch.dtype,
                 device: torch.device):
        if combine not in ("norm_mean", "weighted"):
            raise ValueError(f"two mixers are combined by norm_mean or weighted, got {combine!r}")
        self.combine, self.scales = combine, (float(left_scale), float(right_scale))
        self.hidden_size, self.eps = hidden_size, float(eps)
        self.dtype, self.device = dtype, device
        self.names = {"left": "left", "right": "right", "left_out": "left.out", "right_out": "right.out", **(names or {})}
        self.sides = [get_part("mixer", s.kind)(dtype=dtype, device=device, **s.params) for s in (left, right)]
        if sum(m.cache_need() is not None for m in self.sides) > 1:
            raise ValueError("of two mixers side by side at most one keeps pages")
        needs = [m.state_need() for m in self.sides]
        if all(n is not None for n in needs) and any(len(n.shape) != 1 or n.dtype != "float32" for n in needs):
            raise ValueError("two states in one slot are both flat runs of 32-bit floats")
        # where each side's state starts in a request's slot
        self.state_offs = (0, -(-needs[0].shape[0] // 4) * 4 if all(n is not None for n in needs) else 0)
        self.shared = all(callable(getattr(m, "forward_projected", None)) for m in self.sides)
        self.joint_out = self.shared and combine == "weighted" and \
            all(callable(getattr(m, "output_weight", None)) for m in self.sides)
        self.w_o = None
        if self.joint_out:
            for m, s in zip(self.sides, self.scales):
                if callable(getattr(m, "use_output_scale", None)):
                    m.use_output_scale(s)
        self.w_out: list = [None, None]
        self.w_in = None

    def sub_parts(self) -> list:
        return list(self.sides)

    def weight_specs(self) -> list[WeightSpec]:
        out = []
        for key, m in zip(("left", "right"), self.sides):
            out += [WeightSpec(f"{self.names[key]}.{w.name}", w.shape, w.dtype, w.init) for w in m.weight_specs()]
        if self.combine == "norm_mean":
            out += [WeightSpec(self.names[k], (self.hidden_size,), dtype="float32", init=("ones_plus_normal", 0.1))
                    for k in ("left_out", "right_out")]
        return out

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        for key, m in zip(("left", "right"), self.sides):
            m.bind({w.name: tensors[f"{self.names[key]}.{w.name}"] for w in m.weight_specs()})
        if self.combine == "norm_mean":
            self.w_out = [tensors[self.names["left_out"]], tensors[self.names["right_out"]]]
        if self.shared:
            self.w_in = torch.cat([m.projection_weight() for m in self.sides], dim=0).contiguous()
        if self.joint_out:
            self.w_o = torch.cat([m.output_weight() for m in self.sides], dim=1).contiguous()

    def cache_need(self):
        return next((n for n in (m.cache_need() for m in self.sides) if n is not None), None)

    def state_need(self):
        needs = [m.state_need() for m in self.sides]
        if all(n is not None for n in needs):
            return StateNeed((self.state_offs[1] + needs[1].shape[0],), "float32")
        return next((n for n in needs if n is not None), None)

    def activation_bytes(self, n_tokens: int) -> int:
        elt = 4 if self.dtype == torch.float32 else 2
        return sum(part_activation_bytes(m, n_tokens, self.hidden_size) for m in self.sides) + 3 * n_tokens * self.hidden_size * elt

    def forward(self, x: torch.Tensor, step: StepInputs, cache: LayerCache) -> torch.Tensor:
        caches = [cache if off == cache.state_off else dataclasses.replace(cache, state_off=cache.state_off + off)
                  for off in self.state_offs]
        if self.joint_out:
            proj = ops.linear32(x, self.w_in)
            split, wide = self.sides[0].proj_width, self.sides[0].output_width
            heads = torch.empty((x.shape[0], wide + self.sides[1].output_width), dtype=self.dtype, device=x.device)
            self.sides[0].forward_projected(proj[:, :split], step, caches[0], heads_out=heads[:, :wide], out_scale=self.scales[0])
            self.sides[1].forward_projected(proj[:, split:], step, caches[1], heads_out=heads[:, wide:], out_scale=self.scales[1])
            return ops.linear(heads, self.w_o)
        if self.shared:
            proj = ops.linear32(x, self.w_in)
            split = self.sides[0].proj_width
            a = self.sides[0].forward_projected(proj[:, :split], step, caches[0])
            b = self.sides[1].forward_projected(proj[:, split:], step, caches[1])
        else:
            a, b = (m.forward(x, step, c) for m, c in zip(self.sides, caches))
        if self.combine == "weighted":
            return ops.weighted_pair(a, b, self.scales[0], self.scales[1], torch.empty_like(a))
        return ops.norm_pair_mean(a, b, self.w_out[0], self.w_out[1], self.eps, torch.empty_like(a))


register_mixer("pair", PairMixer)
