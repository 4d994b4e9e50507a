"""Feed-forward layers beyond SwiGLU: a dense layer with a squared-relu activation, and a mixture of experts.

``SquaredReluFeedForward``: ``W_down relu(W_up h)^2``, no biases.

``RoutedExperts``: E small gated feed-forwards ``W_down (silu(W_gate h) * (W_up h))`` of which each token uses
``top``. Router logits ``W_r h + b`` are 32-bit; the ``top`` largest are chosen and weighted by a softmax over the
chosen logits alone; the output is the weighted sum of the chosen experts' outputs. The experts' gate and up
matrices are held as one matrix [E, 2, F, H] and their down matrices side by side along K as [H, E F]: the
activation kernel writes silu(gate) * up * weight for the chosen experts and exact zeros for the others, so the
second product sums the chosen experts with their weights in its 32-bit accumulator.

``ChoiceRoutedExperts``: E small feed-forwards ``W_down relu(W_up h)^2`` and ``identity`` further router outputs without
tensors, whose result is the input h itself. Scores are a softmax over ALL router outputs; the choice is made by score +
``correction`` (a learned vector that does not enter the weights), among the best ``keep`` of ``groups`` equal groups of
neighbouring outputs (a group's score: its largest choice score); the weights are the chosen scores divided by their sum.

``InputScaledExperts``: E small gated feed-forwards ``W_down (silu(W_gate x) * (W_up x))`` of which each token uses
``top``, chosen by the largest router logits (32-bit). A chosen expert's weight is the sigmoid of its logit, not
renormalized, and it multiplies the expert's INPUT: the output is the sum of expert(w h). Optionally a shared expert of
the same form runs for every token and is added, times sigmoid(W_sg h), one number per token. The products W_gate h
and W_up h of all experts (and of the shared one) run as one matrix product on h itself; the activation kernel forms
silu(w g) * (w u) for the chosen experts and exact zeros for the others, and one down product over [E F + shared]
sums them. The router and the shared expert's gate are one 32-bit product.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..registry import register_feed_forward
from .base import StepInputs
from .spec import WeightSpec


class SquaredReluFeedForward:
    def __init__(self, *, hidden_size: int, intermediate_size: int, names: dict[str, str] | None = None,
                 dtype: torch.dtype, device: torch.device):
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.dtype, self.device = dtype, device
        self.names = {"up": "up", "down": "down", **(names or {})}
        self.w_up = self.w_down = None

    def weight_specs(self) -> list[WeightSpec]:
        H, I = self.hidden_size, self.intermediate_size
        return [WeightSpec(self.names["up"], (I, H), init=("normal", 0.05)),
                WeightSpec(self.names["down"], (H, I), init=("normal", 0.05))]

    def activation_bytes(self, n_tokens: int) -> int:
        return n_tokens * (2 * self.intermediate_size + self.hidden_size) * (4 if self.dtype == torch.float32 else 2)

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.w_up, self.w_down = tensors[self.names["up"]], tensors[self.names["down"]]

    def forward(self, x: torch.Tensor, step: StepInputs | None = None) -> torch.Tensor:
        up = ops.linear(x, self.w_up)
        ops.relu2(up, up)
        return ops.linear(up, self.w_down)


class RoutedExperts:
    def __init__(self, *, hidden_size: int, expert_size: int, num_experts: int, top: int,
                 names: dict[str, str] | None = None, dtype: torch.dtype, device: torch.device):
        if not 1 <= top <= num_experts:
            raise ValueError(f"top ({top}) must lie between 1 and the number of experts ({num_experts})")
        self.hidden_size, self.F, self.E, self.top = hidden_size, expert_size, num_experts, top
        self.dtype, self.device = dtype, device
        # {e} is the expert's number
        self.names = {"router": "router", "router_bias": "router.b", "gate": "e{e}.gate", "up": "e{e}.up",
                      "down": "e{e}.down", **(names or {})}
        self.w_router = self.b_router = self.w_router_low = self.w_gate_up = self.w_down = None

    def weight_specs(self) -> list[WeightSpec]:
        H, F, n = self.hidden_size, self.F, self.names
        specs = []
        for e in range(self.E):
            specs += [WeightSpec(n["gate"].format(e=e), (F, H), init=("normal", 0.05)),
                      WeightSpec(n["up"].format(e=e), (F, H), init=("normal", 0.05)),
                      WeightSpec(n["down"].format(e=e), (H, F), init=("normal", 0.05))]
        specs += [WeightSpec(n["router"], (self.E, H), dtype="float32", init=("normal", 0.3)),
                  WeightSpec(n["router_bias"], (self.E,), dtype="float32", init=("normal", 0.3))]
        return specs

    def activation_bytes(self, n_tokens: int) -> int:
        elt = 4 if self.dtype == torch.float32 else 2
        return n_tokens * ((3 * self.E * self.F + self.hidden_size) * elt + 8 * self.E)

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        n = self.names
        self.w_router, self.b_router = tensors[n["router"]], tensors[n["router_bias"]]
        # bfloat16 runs: a bfloat16 copy of the router for the library product, if it holds the very same values
        low = self.w_router.to(torch.bfloat16)
        self.w_router_low = low if self.dtype == torch.bfloat16 and bool((low.float() == self.w_router).all()) else None
        self.w_gate_up = torch.cat([t for e in range(self.E) for t in (tensors[n["gate"].format(e=e)],
                                                                       tensors[n["up"].format(e=e)])], dim=0).contiguous()
        self.w_down = torch.cat([tensors[n["down"].format(e=e)] for e in range(self.E)], dim=1).contiguous()

    def route(self, x: torch.Tensor):
        """(chosen experts [T, top] int32, their weights [T, top] float32, dense weights [T, E] float32)."""
        return ops.moe_route(x, self.w_router, self.b_router, self.top, self.w_router_low)

    def forward(self, x: torch.Tensor, step: StepInputs | None = None) -> torch.Tensor:
        T = x.shape[0]
        _idx, _w, dense = self.route(x)
        gu = ops.linear(x, self.w_gate_up)                                   # [T, E * 2 * F]
        act = torch.empty((T, self.E * self.F), dtype=self.dtype, device=x.device)
        ops.glu_routed(gu, dense, act, self.E, self.F)
        return ops.linear(act, self.w_down)


class ChoiceRoutedExperts:
    def __init__(self, *, hidden_size: int, expert_size: int, num_experts: int, top: int, identity: int = 0, groups: int = 1,
                 keep: int = 1, names: dict[str, str] | None = None, dtype: torch.dtype, device: torch.device):
        n = num_experts + identity
        if num_experts < 1 or identity < 0:
            raise ValueError("at least one expert with tensors, and no negative count of identity outputs")
        if groups < 1 or n % groups or not 1 <= keep <= groups:
            raise ValueError(f"{n} router outputs do not form {groups} equal groups of which {keep} are kept")
        if not 1 <= top <= keep * (n // groups):
            raise ValueError(f"top ({top}) must lie between 1 and the outputs of the kept groups ({keep * (n // groups)})")
        self.hidden_size, self.F, self.E, self.top, self.identity = hidden_size, expert_size, num_experts, top, identity
        self.n, self.groups, self.keep = n, groups, keep
        self.dtype, self.device = dtype, device
        # {e} is the expert's number
        self.names = {"router": "router", "correction": "correction", "up": "e{e}.up", "down": "e{e}.down", **(names or {})}
        self.w_router = self.w_router_low = self.correction = self.w_up = self.w_down = None

    def weight_specs(self) -> list[WeightSpec]:
        H, F, n = self.hidden_size, self.F, self.names
        specs = []
        for e in range(self.E):
            specs += [WeightSpec(n["up"].format(e=e), (F, H), init=("normal", 0.05)),
                      WeightSpec(n["down"].format(e=e), (H, F), init=("normal", 0.05))]
        specs += [WeightSpec(n["router"], (self.n, H), dtype="float32", init=("normal", 0.3)),
                  WeightSpec(n["correction"], (self.n,), dtype="float32", init=("normal", 0.05))]
        return specs

    def activation_bytes(self, n_tokens: int) -> int:
        elt = 4 if self.dtype == torch.float32 else 2
        return n_tokens * ((2 * self.E * self.F + self.hidden_size) * elt + 12 * self.n)

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        n = self.names
        self.w_router, self.correction = tensors[n["router"]], tensors[n["correction"]]
        # bfloat16 runs: a bfloat16 copy of the router for the library product, if it holds the very same values
        low = self.w_router.to(torch.bfloat16)
        self.w_router_low = low if self.dtype == torch.bfloat16 and bool((low.float() == self.w_router).all()) else None
        self.w_up = torch.cat([tensors[n["up"].format(e=e)] for e in range(self.E)], dim=0).contiguous()       # [E F, H]
        self.w_down = torch.cat([tensors[n["down"].format(e=e)] for e in range(self.E)], dim=1).contiguous()   # [H, E F]

    def route(self, x: torch.Tensor):
        """(chosen outputs [T, top] int32, their weights [T, top], dense weights [T, E + identity], summed weight of the
        chosen identity outputs [T]), all weights float32."""
        logits = ops.router_logits(x, self.w_router, self.w_router_low)
        return ops.moe_choose(logits, self.correction, self.top, self.groups, self.keep, self.identity)

    def forward_parts(self, x: torch.Tensor, step: StepInputs | None = None):
        """(the experts' weighted sum [T, H], x or None, the identity outputs' weight per token or None): the result is
        the first plus the third times the second; a norm that takes two branches adds them in its own pass."""
        T = x.shape[0]
        _idx, _w, dense, id_w = self.route(x)
        up = ops.linear(x, self.w_up)                                            # [T, E * F]
        act = torch.empty((T, self.E * self.F), dtype=self.dtype, device=x.device)
        ops.act_routed(up, dense, act, self.E, self.F)
        out = ops.linear(act, self.w_down)
        return (out, x, id_w) if self.identity else (out, None, None)

    def forward(self, x: torch.Tensor, step: StepInputs | None = None) -> torch.Tensor:
        out, x2, id_w = self.forward_parts(x, step)
        if x2 is None:
            return out
        return ops.add_scaled_rows(out, x2, id_w)


class InputScaledExperts:
    def __init__(self, *, hidden_size: int, expert_size: int, num_experts: int, top: int, shared_size: int = 0,
                 shared_gate: bool = True, names: dict[str, str] | None = None, dtype: torch.dtype, device: torch.device):
        if not 1 <= top <= num_experts:
            raise ValueError(f"top ({top}) must lie between 1 and the number of experts ({num_experts})")
        if shared_size < 0:
            raise ValueError("the shared expert has no negative size")
        self.hidden_size, self.F, self.E, self.top, self.Fs = hidden_size, expert_size, num_experts, top, int(shared_size)
        self.gated = bool(shared_gate) and self.Fs > 0
        self.dtype, self.device = dtype, device
        # {e} is the expert's number
        self.names = {"router": "router", "gate": "e{e}.gate", "up": "e{e}.up", "down": "e{e}.down",
                      "shared_gate": "shared.gate", "shared_up": "shared.up", "shared_down": "shared.down",
                      "shared_weight": "shared.sg", **(names or {})}
        self.w_router = self.w_router_low = self.w_gate_up = self.w_down = None

    def weight_specs(self) -> list[WeightSpec]:
        H, F, n = self.hidden_size, self.F, self.names
        specs = []
        for e in range(self.E):
            specs += [WeightSpec(n["gate"].format(e=e), (F, H), init=("normal", 0.05)),
                      WeightSpec(n["up"].format(e=e), (F, H), init=("normal", 0.05)),
                      WeightSpec(n["down"].format(e=e), (H, F), init=("normal", 0.05))]
        specs.append(WeightSpec(n["router"], (self.E, H), dtype="float32", init=("normal", 0.3)))
        if self.Fs:
            specs += [WeightSpec(n["shared_gate"], (self.Fs, H), init=("normal", 0.05)),
                      WeightSpec(n["shared_up"], (self.Fs, H), init=("normal", 0.05)),
                      WeightSpec(n["shared_down"], (H, self.Fs), init=("normal", 0.05))]
        if self.gated:
            specs.append(WeightSpec(n["shared_weight"], (1, H), dtype="float32", init=("normal", 0.3)))
        return specs

    def activation_bytes(self, n_tokens: int) -> int:
        elt = 4 if self.dtype == torch.float32 else 2
        return n_tokens * ((3 * (self.E * self.F + self.Fs) + self.hidden_size) * elt + 12 * (self.E + 1))

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        n = self.names
        # the router's rows, then the shared expert's gate as one more row: one 32-bit product serves both
        rows = [tensors[n["router"]]] + ([tensors[n["shared_weight"]].reshape(1, -1)] if self.gated else [])
        pad = -(self.E + len(rows) - 1) % 8          # rows of zeros up to a multiple of 8: the library's products of odd
        if pad:                                       # widths run several times slower; nothing reads those columns
            rows.append(torch.zeros((pad, self.hidden_size), dtype=rows[0].dtype, device=rows[0].device))
        self.w_router = torch.cat(rows, dim=0).contiguous()
        low = self.w_router.to(torch.bfloat16)
        self.w_router_low = low if self.dtype == torch.bfloat16 and bool((low.float() == self.w_router).all()) else None
        parts = [t for e in range(self.E) for t in (tensors[n["gate"].format(e=e)], tensors[n["up"].format(e=e)])]
        downs = [tensors[n["down"].format(e=e)] for e in range(self.E)]
        if self.Fs:
            parts += [tensors[n["shared_gate"]], tensors[n["shared_up"]]]
            downs.append(tensors[n["shared_down"]])
        self.w_gate_up = torch.cat(parts, dim=0).contiguous()                # [E * 2 F + 2 Fs, H]
        self.w_down = torch.cat(downs, dim=1).contiguous()                   # [H, E F + Fs]

    def route(self, x: torch.Tensor):
        """(chosen experts [T, top] int32, their weights [T, top], dense weights [T, E] float32, the logits [T, E (+ 1)])."""
        logits = ops.router_logits(x, self.w_router, self.w_router_low)
        return (*ops.moe_topk(logits, self.E, self.top, "sigmoid"), logits)

    def forward(self, x: torch.Tensor, step: StepInputs | None = None) -> torch.Tensor:
        T = x.shape[0]
        _idx, _w, dense, logits = self.route(x)
        gu = ops.linear(x, self.w_gate_up)
        act = torch.empty((T, self.E * self.F + self.Fs), dtype=self.dtype, device=x.device)
        ops.glu_routed_in(gu, dense, act, self.E, self.F, self.Fs, logits[:, self.E] if self.gated else None)
        return ops.linear(act, self.w_down)


register_feed_forward("routed_input_scaled", InputScaledExperts)
register_feed_forward("routed_choice", ChoiceRoutedExperts)
register_feed_forward("relu2", SquaredReluFeedForward)
register_feed_forward("routed_experts", RoutedExperts)
