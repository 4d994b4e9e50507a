"""RMSNorm over the 32-bit residual stream, fused with whatever feeds the stream.

Formula (src/infer/model/layers.py:35-44): ``x32 * rsqrt(mean(x32^2) + eps)`` in 32-bit, cast to the
activation dtype, then multiplied by the weight. The weight is held in float32 (a 16-bit checkpoint
value converts exactly; the product is rounded once to the activation dtype, which equals the
reference's 16-bit multiply).
"""

from __future__ import annotations

import torch

from ..kernels import lib, ops
from ..registry import register_norm
from .spec import WeightSpec


class RMSNorm:
    def __init__(self, *, hidden_size: int, eps: float, dtype: torch.dtype, device: torch.device):
        self.hidden_size = hidden_size
        self.eps = float(eps)
        self.dtype = dtype
        self.device = device
        self.weight: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec("weight", (self.hidden_size,), dtype="float32", init=("ones_plus_normal", 0.02))]

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"]

    def forward(self, resid: torch.Tensor, out: torch.Tensor | None = None, *,
                branch: torch.Tensor | None = None, partials: torch.Tensor | None = None,
                ids: torch.Tensor | None = None, table: torch.Tensor | None = None,
                rows: torch.Tensor | None = None) -> torch.Tensor:
        n = rows.numel() if rows is not None else resid.shape[0]
        if out is None:
            out = torch.empty((n, self.hidden_size), dtype=self.dtype, device=resid.device)
        return ops.add_rmsnorm(resid, self.weight, self.eps, out, branch=branch, partials=partials, ids=ids,
                               table=table, rows=rows)


    def emit(self, b, resid, *, n_rows, out_tag: str = "normed", branch=None, ids=None, table=None, rows=None,
             cond=None):
        """The same launch, written into a step program (kernels/program.py): ``resid`` and ``branch`` are
        workspace buffers, ``ids`` / ``rows`` / ``n_rows`` step parameters. Returns the output buffer."""
        from ..kernels.program import OP_ADD_RMSNORM, Float
        out = b.buffer(out_tag, self.hidden_size * (torch.finfo(self.dtype).bits // 8))
        b.emit(OP_ADD_RMSNORM, [ops.dtype_code(self.dtype), resid, branch, ids, table, rows, self.weight, Float(self.eps), out,
                                n_rows, self.hidden_size], cond=cond)
        return out


class RMSNorm32:
    """RMSNorm whose every product is 32-bit: ``x * rsqrt(mean(x^2) + eps) * (offset + w)``, rounded once. ``offset``
    is 1 for checkpoints that store the weight around zero (it is added when the weight is bound). The stream may
    receive two branch outputs with a common multiplier on the way (``resid += scale * (branch + branch2)``), and
    one pass can serve two norms of the same stream: ``pair`` names the second norm, whose output is returned
    beside this one's; ``raw`` keeps this norm's output in 32-bit (for a token shift that follows)."""

    def __init__(self, *, hidden_size: int, eps: float, offset: float = 0.0, weight_name: str = "weight",
                 dtype: torch.dtype, device: torch.device):
        self.hidden_size, self.eps, self.offset = hidden_size, float(eps), float(offset)
        self.weight_name = weight_name
        self.dtype, self.device = dtype, device
        self.weight: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        init = ("normal", 0.1) if self.offset else ("ones_plus_normal", 0.1)
        return [WeightSpec(self.weight_name, (self.hidden_size,), dtype="float32", init=init)]

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        w = tensors[self.weight_name]
        self.weight = (w + self.offset).contiguous() if self.offset else w

    def forward(self, resid: torch.Tensor, out: torch.Tensor | None = None, *, branch: torch.Tensor | None = None,
                branch2: torch.Tensor | None = None, scale: float = 1.0, partials: torch.Tensor | None = None,
                ids: torch.Tensor | None = None, table: torch.Tensor | None = None, rows: torch.Tensor | None = None,
                pair: "RMSNorm32 | None" = None, raw: bool = False):
        if partials is not None:
            raise NotImplementedError("the 32-bit norm takes branch outputs, not partial products")
        n = rows.numel() if rows is not None else resid.shape[0]
        if out is None:
            out = torch.empty((n, self.hidden_size), dtype=torch.float32 if raw else self.dtype, device=resid.device)
        out2 = None
        if pair is not None:
            if pair.eps != self.eps or pair.hidden_size != self.hidden_size:
                raise ValueError("two norms served by one pass share eps and width")
            out2 = torch.empty((n, self.hidden_size), dtype=self.dtype, device=resid.device)
        ops.add_norm_pair(resid, self.weight, self.eps, out, dtype=self.dtype, w2=pair.weight if pair is not None else None,
                          out2=out2, a=branch, b=branch2, scale=scale, ids=ids, table=table, rows=rows)
        return (out, out2) if pair is not None else out


class GatedAddRMSNorm:
    """RMSNorm (32-bit products, plain weight, one rounding) over a stream that receives the previous branch through a
    learned gate on the way: ``resid += sigmoid(gate + gate_bias) * branch``, the gate's pre-activations arriving as a
    32-bit matrix product. Without a gate the branch is added as it is; at the start the stream is the embedding row
    times ``table_scale`` (multiplied in 32-bit). Also a model's final norm (``rows``)."""

    def __init__(self, *, hidden_size: int, eps: float, weight_name: str = "weight", dtype: torch.dtype,
                 device: torch.device):
        self.hidden_size, self.eps, self.weight_name = hidden_size, float(eps), weight_name
        self.dtype, self.device = dtype, device
        self.weight: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec(self.weight_name, (self.hidden_size,), dtype="float32", init=("ones_plus_normal", 0.1))]

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name]

    def forward(self, resid: torch.Tensor, out: torch.Tensor | None = None, *, branch: torch.Tensor | None = None,
                gate: torch.Tensor | None = None, gate_bias: torch.Tensor | None = None,
                partials: torch.Tensor | None = None, ids: torch.Tensor | None = None, table: torch.Tensor | None = None,
                table_scale: float = 1.0, rows: torch.Tensor | None = None) -> torch.Tensor:
        if partials is not None:
            raise NotImplementedError("the gated norm takes branch outputs, not partial products")
        n = rows.numel() if rows is not None else resid.shape[0]
        if out is None:
            out = torch.empty((n, self.hidden_size), dtype=self.dtype, device=resid.device)
        return ops.gated_add_rmsnorm(resid, self.weight, self.eps, out, branch=branch, gate=gate, gate_bias=gate_bias,
                                     ids=ids, table=table, table_scale=table_scale, rows=rows)


class DynamicTanhNorm:
    """Dynamic Tanh in the place of a norm: ``tanh(alpha * x) * w + b`` with a learned scalar ``alpha``, a weight and a
    bias vector; no mean, no variance, no eps. Tensors: the weight under the part's own name, ``b`` and ``alpha`` beside
    it. 32-bit throughout, one rounding.

    It reads a residual of one or several streams (``streams`` copies of the row side by side, ``resid`` [T, streams * H]):
    on the way it takes in the previous sublayer's result, ``x_t <- sum_s stream_mix[s, t] x_s + stream_out[t] y`` (one
    stream without a mix: ``x += y``), with ``y = branch + row_scale * branch2``; or starts every stream as
    ``table[ids] * table_scale + pos_table[positions]``; then norms ``u = sum_s stream_in[s] x_s`` (no ``stream_in``: the sum of the
    streams, which is what a model's last norm reads). ``kind="rms"`` keeps all of that with an RMS norm (weight only)."""

    def __init__(self, *, hidden_size: int, streams: int = 1, kind: str = "dyt", eps: float = 0.0,
                 names: dict[str, str] | None = None, library: str = "streams", dtype: torch.dtype, device: torch.device):
        if kind not in ops.STREAM_NORMS or not 1 <= streams <= ops.MAX_STREAMS:
            raise ValueError(f"norm kinds {sorted(ops.STREAM_NORMS)} over 1 to {ops.MAX_STREAMS} streams are built, got "
                             f"{kind!r} over {streams}")
        lib.prefer(library)      # the kernel library a model of such norms runs from (kernels/build.py)
        self.hidden_size, self.streams, self.kind, self.eps = hidden_size, int(streams), kind, float(eps)
        self.dtype, self.device = dtype, device
        self.names = {"weight": "", "bias": "b", "alpha": "alpha", **(names or {})}
        self.weight = self.bias = self.alpha = None

    def weight_specs(self) -> list[WeightSpec]:
        n, H = self.names, self.hidden_size
        specs = [WeightSpec(n["weight"], (H,), dtype="float32", init=("ones_plus_normal", 0.1))]
        if self.kind == "dyt":
            specs += [WeightSpec(n["bias"], (H,), dtype="float32", init=("normal", 0.1)),
                      WeightSpec(n["alpha"], (), dtype="float32", init=("normal", 0.05, 0.6))]
        return specs

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.names["weight"]]
        if self.kind == "dyt":
            self.bias, self.alpha = tensors[self.names["bias"]], tensors[self.names["alpha"]].reshape(1)

    def forward(self, resid: torch.Tensor, out: torch.Tensor | None = None, *, branch: torch.Tensor | None = None,
                branch2: torch.Tensor | None = None, row_scale: torch.Tensor | None = None,
                partials: torch.Tensor | None = None, ids: torch.Tensor | None = None, table: torch.Tensor | None = None,
                positions: torch.Tensor | None = None, pos_table: torch.Tensor | None = None,
                rows: torch.Tensor | None = None, stream_mix: torch.Tensor | None = None,
                stream_out: torch.Tensor | None = None, stream_in: torch.Tensor | None = None,
                table_scale: float = 1.0, scale: float = 1.0) -> torch.Tensor:
        if partials is not None:
            raise NotImplementedError("this norm takes branch outputs, not partial products")
        if scale != 1.0:
            raise NotImplementedError("this norm adds branch outputs as they are")
        n = rows.numel() if rows is not None else resid.shape[0]
        if out is None:
            out = torch.empty((n, self.hidden_size), dtype=self.dtype, device=resid.device)
        return ops.stream_norm(resid, self.streams, out, kind=self.kind, weight=self.weight, bias=self.bias, alpha=self.alpha,
                               eps=self.eps, ids=ids, table=table, positions=positions, pos_table=pos_table, branch=branch,
                               branch2=branch2, row_scale=row_scale, mix=stream_mix, out_w=stream_out, in_w=stream_in, rows=rows,
                               table_scale=table_scale)


register_norm("dyt", DynamicTanhNorm)
register_norm("rmsnorm", RMSNorm)
register_norm("rmsnorm_gated", GatedAddRMSNorm)
register_norm("rmsnorm32", RMSNorm32)
