"""Grouped-query attention with the options a windowed design may combine, each a constructor parameter:

* key/query heads of ``head_dim`` and value heads of ``value_dim`` (they may differ);
* an RMS norm over the WHOLE query projection and the whole key projection (all heads at once, plain weights), before
  the rotation (``qk_norm``);
* rotate-half rotation of the first ``rot_dims`` dimensions of each head, tables from a position-encoding part;
* ``score = q . k * scale``, then ``softcap * tanh(score / softcap)`` (``softcap`` 0: none);
* a sliding window that keeps the sequence's first tokens visible: position i sees j <= i when i - j < window or
  j < keep_first (window 0: every key). Kept tokens keep their true positions;
* a softmax with one added to the denominator, p_j = exp(s_j) / (1 + sum exp(s_j)): a sink of score 0 without a
  value (``sink``);
* a per-head output gate sigmoid(W_g h), one number per head, read from the same input as the projections
  (``head_gate``), or a gate of one number per output number, applied to the heads side by side before the output
  projection (``value_gate``);
* a query temperature: q is multiplied by ``1 + coef * ln(floor((p + 1) / every) + 1)`` at position p (``q_temp``);
* no keys and values of its own (``shares_kv``): the layer has no k and v tensors and reads the cache of another
  layer with the same head counts and sizes (the run order's ``cache_of``), with its own queries, mask and gate;
* biases of the q, k and v projections (``bias``: tensors ``<q>.b`` and so on), added to the product's 32-bit result;
* a short causal convolution over time on every channel of q, k and v, directly after the projection (``conv_taps`` >= 1:
  tensors ``<q>.conv`` [channels, taps], the last tap weighing the current token; a request's last taps - 1 projected
  rows are per-request state of the mixer; 0: none);
* ``qk_norm="head"``: every head of q and of k divided by its own root mean square, without weights;
* talking heads (``talk``: tensor [heads, heads]): after the softmax the heads' weights are mixed, weight_h <- sum_g
  talk[h, g] weight_g, and head h applies its mixed weights to the values of its own key/value head. The softmax and the
  product with the values are linear in between, so the kernel applies every head's own weights to the values of each
  value head ([T, heads, kv_heads, vdim] in 32-bit) and a small kernel mixes those results.

Projections q, k, v (and g) are held as one matrix whose product keeps its 32-bit accumulator; one kernel norms,
rotates and writes the token's cache row ``[k | v]`` (a paged cache of one plane whose row holds all key heads, then
all value heads); the attention kernel reads rows back through the block table, so a prompt portion sees its own keys.
A mixer that runs beside others may be handed its columns of a shared product (``projection_weight`` /
``forward_projected``).
"""

from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops
from ..registry import get_part, register_mixer
from .base import LayerCache, StepInputs, StepMetadata, StepShape, part_limit_positions, part_max_positions
from .spec import PagedKVNeed, PartSpec, StateNeed, WeightSpec


SPLIT_BLOCKS = 296      # blocks the tensor-core kernel should have in flight before a tile's keys stop being dealt out
MAX_SPLITS = 8


class SinkWindowAttention:
    def __init__(self, *, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int, scale: float,
                 position: PartSpec | None, rot_dims: int = 0, window: int | None = None, keep_first: int = 0,
                 softcap: float = 0.0, sink: bool = True, qk_norm: bool = True, head_gate: bool = True, eps: float = 1e-6,
                 value_gate: bool = False, q_temp: tuple[float, int] | None = None, shares_kv: bool = False,
                 bias: bool = False, conv_taps: int = 0, talk: bool = False,
                 names: dict[str, str] | None = None, dtype: torch.dtype, device: torch.device):
        if num_heads % num_kv_heads:
            raise ValueError(f"heads ({num_heads}) must be a multiple of kv heads ({num_kv_heads})")
        if value_dim > 256 or head_dim > 512:
            raise ValueError("heads of up to 512 (keys) and 256 (values) are built")
        self.hidden_size, self.nh, self.nkv, self.d, self.dv = hidden_size, num_heads, num_kv_heads, head_dim, value_dim
        self.scale, self.softcap, self.eps = float(scale), float(softcap or 0.0), float(eps)
        self.window, self.keep_first = int(window) if window else 0, int(keep_first or 0)
        if qk_norm not in (True, False, "head"):
            raise ValueError(f"qk_norm is False, True (whole projections, weights) or 'head', got {qk_norm!r}")
        self.head_norm = qk_norm == "head"
        self.bias, self.taps, self.talk = bool(bias), int(conv_taps), bool(talk)
        if not 0 <= self.taps <= 16:
            raise ValueError(f"convolutions of up to 16 taps are built, got {conv_taps}")
        if (self.taps or self.bias) and shares_kv:
            raise ValueError("a layer that reads another layer's keys has no biases and no convolution")
        if (self.talk or self.taps or self.bias) and (head_gate or value_gate):
            raise ValueError("mixed heads, biases and convolved projections are built without an output gate")
        self.sink, self.qk_norm, self.head_gate = bool(sink), qk_norm is True, bool(head_gate)
        self.value_gate, self.shares_kv = bool(value_gate), bool(shares_kv)
        if self.value_gate and self.head_gate:
            raise ValueError("the output gate has one number per head or one per output number, not both")
        if self.shares_kv and self.qk_norm:
            raise ValueError("a layer that reads another layer's keys has no key norm of its own")
        self.q_temp = (float(q_temp[0]), int(q_temp[1])) if q_temp else None
        if self.q_temp is not None and self.q_temp[1] < 1:
            raise ValueError(f"the query temperature's interval must be positive, got {self.q_temp[1]}")
        self.position = get_part("position", position.kind)(**position.params) if position is not None else None
        self.rot_dims = int(rot_dims) if self.position is not None else 0
        if self.rot_dims % 2 or self.rot_dims > head_dim:
            raise ValueError(f"rot_dims ({self.rot_dims}) must be even and at most head_dim ({head_dim})")
        self.dtype, self.device = dtype, device
        self.names = {"q": "q", "k": "k", "v": "v", "q_norm": "q.norm", "k_norm": "k.norm", "g": "g", "o": "o",
                      "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "q_conv": "q.conv", "k_conv": "k.conv",
                      "v_conv": "v.conv", "talk": "talk", **(names or {})}
        self.q_size, self.k_size, self.v_size = num_heads * head_dim, num_kv_heads * head_dim, num_kv_heads * value_dim
        self.gate_cols = num_heads if self.head_gate else num_heads * value_dim if self.value_gate else 0
        self.proj_width = self.q_size + (0 if self.shares_kv else self.k_size + self.v_size) + self.gate_cols
        # bfloat16 with key and value heads of 32, 64 or 128: tensor cores, 64 rows a tile; anything else (and the 32-bit
        # path): the shape-generic kernel on CUDA cores, 32 rows a tile
        self.tensor_cores = ops.sink_attention_tc_ok(dtype, head_dim, value_dim) and self.scale > 0
        self.tile_rows = ops.SINK_TC_TILE_ROWS if self.tensor_cores else ops.SINK_TILE_ROWS
        self.qkv_width = self.q_size + self.k_size + self.v_size
        self.w_in = self.w_o = self.g_q = self.g_k = self.cos = self.sin = None
        self.b_in = self.w_conv = self.w_talk = None

    # --- declarations -----------------------------------------------------------------------------------------

    def weight_specs(self) -> list[WeightSpec]:
        n, W = self.names, self.hidden_size
        specs = [WeightSpec(n["q"], (self.q_size, W), init=("normal", 0.05))]
        if not self.shares_kv:
            specs += [WeightSpec(n["k"], (self.k_size, W), init=("normal", 0.05)),
                      WeightSpec(n["v"], (self.v_size, W), init=("normal", 0.05))]
        if self.qk_norm:
            specs += [WeightSpec(n["q_norm"], (self.q_size,), dtype="float32", init=("ones_plus_normal", 0.1)),
                      WeightSpec(n["k_norm"], (self.k_size,), dtype="float32", init=("ones_plus_normal", 0.1))]
        if self.gate_cols:
            specs.append(WeightSpec(n["g"], (self.gate_cols, W), init=("normal", 0.05)))
        sizes = (("q", self.q_size), ("k", self.k_size), ("v", self.v_size))
        if self.bias:
            specs += [WeightSpec(n[f"{x}_bias"], (size,), dtype="float32", init=("normal", 0.1)) for x, size in sizes]
        if self.taps:
            specs += [WeightSpec(n[f"{x}_conv"], (size, self.taps), dtype="float32", init=("normal", 0.3, 1.0 / self.taps))
                      for x, size in sizes]
        if self.talk:
            specs.append(WeightSpec(n["talk"], (self.nh, self.nh), dtype="float32", init=("normal", 0.3, 1.0 / self.nh)))
        specs.append(WeightSpec(n["o"], (W, self.nh * self.dv), init=("normal", 0.05)))
        return specs

    def cache_need(self) -> PagedKVNeed:
        return PagedKVNeed(1, self.k_size + self.v_size, self.window or None, planes=1,
                           keep_first=self.keep_first if self.window else 0)

    def state_need(self) -> StateNeed | None:
        return StateNeed(((self.taps - 1) * self.qkv_width,), "float32") if self.taps > 1 else None

    def max_positions(self) -> int | None:
        return part_max_positions(self.position) if self.position is not None else None

    def limit_positions(self, n: int) -> None:
        if self.position is not None:
            part_limit_positions(self.position, n)

    def activation_bytes(self, n_tokens: int) -> int:
        elt = 4 if self.dtype == torch.float32 else 2
        return n_tokens * (self.proj_width * 4 + (self.q_size + self.nh * self.dv + self.hidden_size) * elt + self.nh * 4)

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        n = self.names
        rows = [tensors[n["q"]]] + ([] if self.shares_kv else [tensors[n["k"]], tensors[n["v"]]]) + \
            ([tensors[n["g"]]] if self.gate_cols else [])
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_o = tensors[n["o"]]
        if self.qk_norm:
            self.g_q, self.g_k = tensors[n["q_norm"]], tensors[n["k_norm"]]
        if self.bias:
            self.b_in = torch.cat([tensors[n[f"{x}_bias"]] for x in "qkv"]).contiguous()
        if self.taps:
            self.w_conv = torch.cat([tensors[n[f"{x}_conv"]] for x in "qkv"], dim=0).contiguous()
        elif self.bias:
            self.w_conv = torch.ones((self.qkv_width, 1), dtype=torch.float32, device=self.device)
        if self.talk:
            self.w_talk = tensors[n["talk"]].contiguous()
        if self.position is not None:
            self.cos, self.sin = self.position.tables(self.device)
        else:       # no rotation: tables of no columns
            self.cos = self.sin = torch.zeros((1, 0), dtype=torch.float32, device=self.device)

    def projection_weight(self) -> torch.Tensor:
        """[proj_width, hidden] rows [q; k; v; g]: what a shared product multiplies for this mixer."""
        return self.w_in

    @property
    def output_width(self) -> int:
        return self.nh * self.dv

    def output_weight(self) -> torch.Tensor:
        """[hidden, heads * vdim]: what multiplies the heads side by side (``forward_projected(heads_out=)`` leaves them)."""
        return self.w_o

    # --- per-step work list -----------------------------------------------------------------------------------

    def metadata_key(self):
        return ("sink_attention", self.nh // self.nkv, self.tile_rows, self.nkv if self.talk else 0)

    def step_metadata(self, shape: StepShape) -> StepMetadata:
        """Row tiles of the attention kernel: ``tile_rows`` consecutive (token, head in group) rows of one request each."""
        rows = self.tile_rows
        per_seq = (shape.q_lens.astype(np.int64) * (self.nh // self.nkv) + rows - 1) // rows
        tile_seq = np.repeat(np.arange(len(per_seq), dtype=np.int32), per_seq)
        first = np.cumsum(per_seq) - per_seq
        tile_row0 = ((np.arange(tile_seq.size) - np.repeat(first, per_seq)) * rows).astype(np.int32)
        # Few row tiles (decoding): deal each tile's key blocks out over several blocks of the grid. (A captured graph
        # serves every context: it takes the split for the longest.)
        n_tiles, splits = int(tile_seq.size), 1
        if self.tensor_cores and n_tiles:
            longest = shape.max_kv_len if shape.for_graph else int((shape.starts.astype(np.int64) + shape.q_lens).max())
            keys = min(longest, self.window + self.keep_first + rows) if self.window else longest
            blocks = n_tiles * self.nkv * (self.nkv if self.talk else 1)
            splits = max(1, min((keys // 64 + 1) // 2, SPLIT_BLOCKS // blocks, MAX_SPLITS))
        return StepMetadata({"tile_seq": tile_seq, "tile_row0": tile_row0}, {"n_tiles": n_tiles, "n_splits": splits},
                            constant_in_graph=True)

    # --- run --------------------------------------------------------------------------------------------------

    def forward(self, x: torch.Tensor, step: StepInputs, cache: LayerCache) -> torch.Tensor:
        return self.forward_projected(ops.linear32(x, self.w_in), step, cache)

    def forward_projected(self, proj: torch.Tensor, step: StepInputs, cache: LayerCache, *,
                          heads_out: torch.Tensor | None = None, out_scale: float = 1.0) -> torch.Tensor | None:
        """``proj`` [T, proj_width] float32 (a view of a wider product is fine): this mixer's columns [q | k | v | g]
        ([q | g] for a layer that reads another layer's keys and values). ``heads_out`` [T, heads * vdim] (columns of a
        wider matrix): the heads side by side times ``out_scale`` are left there and the output product is the caller's
        (mixers with mixed heads, whose last kernel writes anywhere)."""
        T, dev = proj.shape[0], proj.device
        if self.taps or self.bias:      # q, k and v through the convolution (the biases enter on the way); what follows
            # reads that. Biases alone: a convolution of one tap with weights of one, which carries nothing.
            conv = torch.empty((T, self.qkv_width), dtype=torch.float32, device=dev)
            state = cache.state if self.taps > 1 else torch.empty((1, 0), dtype=torch.float32, device=dev)
            proj = ops.short_conv_state(proj, 0, self.w_conv, self.b_in, state, cache.state_off if self.taps > 1 else 0,
                                        step.cu_q, step.seq_of_token, step.state_slots, conv)
        q = torch.empty((T, self.q_size), dtype=self.dtype, device=dev)
        gate = torch.empty((T, self.gate_cols), dtype=torch.float32, device=dev) if self.gate_cols else None
        rows = cache.k.view(-1, self.k_size + self.v_size)
        if self.shares_kv and cache.writes:
            raise ValueError("a layer without keys and values of its own reads another layer's cache")
        ops.qk_norm_rope_write(proj, heads=self.nh, kv_heads=self.nkv, dim=self.d, vdim=self.dv, rot_dims=self.rot_dims,
                               wq=self.g_q, wk=self.g_k, eps=self.eps, positions=step.positions, cos=self.cos, sin=self.sin,
                               slot_map=step.slot_maps[cache.group] if cache.writes else None, q_out=q,
                               cache=rows if cache.writes else None, gate_out=gate, has_kv=not self.shares_kv,
                               q_temp=self.q_temp, head_norm=self.head_norm)
        meta = step.meta[self.metadata_key()]
        if heads_out is not None and not self.talk:
            raise NotImplementedError("only the mix of the heads writes into columns of a wider matrix")
        heads = heads_out if heads_out is not None else torch.empty((T, self.nh * self.dv), dtype=self.dtype, device=dev)
        cross = torch.empty((T, self.nh * self.nkv * self.dv), dtype=torch.float32, device=dev) if self.talk else None
        splits, part = meta.host["n_splits"], None
        if splits > 1:
            part = step.workspace.get("sink_attention_part", meta.host["n_tiles"] * self.nkv * (self.nkv if self.talk else 1) *
                                      splits * self.tile_rows * (self.dv + 2), torch.float32)
        ops.sink_attention(q, cache.k, step.block_tables[cache.group], step.cu_q, step.kv_before, meta.arrays["tile_seq"],
                           meta.arrays["tile_row0"], meta.host["n_tiles"], gate, None if self.talk else heads, heads=self.nh,
                           kv_heads=self.nkv,
                           dim=self.d, vdim=self.dv, scale=self.scale, softcap=self.softcap, window=self.window,
                           keep_first=self.keep_first, sink=self.sink, tensor_cores=self.tensor_cores, n_splits=splits,
                           part=part, cross_out=cross)
        if self.talk:
            ops.talk_mix(cross, self.w_talk, heads, self.nh, self.nkv, self.dv, scale=out_scale)
        return ops.linear(heads, self.w_o) if heads_out is None else None


register_mixer("sink_window_attention", SinkWindowAttention)
