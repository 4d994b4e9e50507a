"""Tensor-level wrappers over the kernel entry points.

Each wrapper checks what the kernel assumes (device, dtype, contiguity, shapes) and launches on the
current CUDA stream. None of them has a fallback: a tensor on the CPU or a missing library raises.
"""

from __future__ import annotations

import os

import torch

from . import lib

F32, BF16 = 0, 1


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise lib.KernelError(f"kernels run in float32 or bfloat16, got {dtype}")


dtype_code = _code


def _stream() -> int:
    """The raw handle of the stream torch launches on right now (captured graphs included). The private
    C call is a fraction of a microsecond; the public ``torch.cuda.current_stream()`` builds objects on
    the way and costs ten times that, once per kernel launch."""
    return _raw_stream(torch.cuda.current_device())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None) or \
    (lambda device: torch.cuda.current_stream(device).cuda_stream)


def _req(t: torch.Tensor, name: str, dtype: torch.dtype | None = None) -> int:
    if not t.is_cuda:
        raise lib.KernelError(f"{name} is on {t.device}; the kernels have no CPU path")
    if not t.is_contiguous():
        raise lib.KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise lib.KernelError(f"{name} must be {dtype}, got {t.dtype}")
    return t.data_ptr()


def _opt(t: torch.Tensor | None, name: str, dtype: torch.dtype | None = None) -> int | None:
    return None if t is None else _req(t, name, dtype)


def add_rmsnorm(resid: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, *,
                branch: torch.Tensor | None = None, partials: torch.Tensor | None = None,
                ids: torch.Tensor | None = None, table: torch.Tensor | None = None,
                rows: torch.Tensor | None = None) -> torch.Tensor:
    """resid [T, H] float32 (updated in place unless ``rows``); out [n, H] in the activation dtype.
    ids + table: the stream starts as table[ids]. branch [T, H]: added to the stream. partials
    [n, T, H] float32: summed in index order and added. rows [n] int32: norm only these rows."""
    H = resid.shape[-1]
    n_rows = rows.numel() if rows is not None else resid.shape[0]
    if out.shape[0] < n_rows or out.shape[-1] != H or weight.numel() != H:
        raise lib.KernelError(f"add_rmsnorm: out {tuple(out.shape)} / weight {tuple(weight.shape)} do not fit "
                              f"{n_rows} rows of width {H}")
    if (ids is None) != (table is None):
        raise lib.KernelError("add_rmsnorm: ids and table come together")
    n_part, part_stride = 0, 0
    if partials is not None:
        n_part, part_stride = partials.shape[0], partials.stride(0)
    dt = out.dtype
    lib.call("tm_add_rmsnorm", _code(dt), _req(resid, "resid", torch.float32), _opt(branch, "branch", dt),
             _opt(partials, "partials", torch.float32), n_part, part_stride, _opt(ids, "ids", torch.int32),
             _opt(table, "table", dt), _opt(rows, "rows", torch.int32), _req(weight, "weight", torch.float32),
             float(eps), _req(out, "out"), n_rows, H, _stream())
    return out


def qkv_rope_write(qkv: torch.Tensor, bias: torch.Tensor | None, positions: torch.Tensor, cos: torch.Tensor | None,
                   sin: torch.Tensor | None, slot_map: torch.Tensor | None, q_out: torch.Tensor,
                   kcache: torch.Tensor | None, vcache: torch.Tensor | None, nh: int, nkv: int, D: int) -> None:
    """qkv [T, (nh + 2 nkv) D]; cos/sin [P, D/2] float32 (both None: no rotation); q_out [T, nh, D]; caches
    [pages, page, nkv, D]. Without a slot map but with "caches" of T rows, token t's k and v go to row t. A
    position outside the tables raises the device error word (``position_check``) instead of reading them."""
    T = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * D or positions.numel() < T or (cos is None) != (sin is None) or \
            (cos is not None and cos.shape[1] * 2 != D):
        raise lib.KernelError(f"qkv_rope_write: shapes do not fit (qkv {tuple(qkv.shape)}, nh {nh}, nkv {nkv}, D {D})")
    if slot_map is not None and (kcache is None or vcache is None):
        raise lib.KernelError("qkv_rope_write: a slot map needs both caches")
    if slot_map is None and kcache is not None and (kcache.numel() < T * nkv * D or vcache is None
                                                    or vcache.numel() < T * nkv * D):
        raise lib.KernelError("qkv_rope_write: dense k / v outputs need a row per token")
    dt = q_out.dtype
    lib.call("tm_qkv_rope_write", _code(qkv.dtype), _code(dt), _req(qkv, "qkv"), _opt(bias, "bias", torch.float32),
             _req(positions, "positions", torch.int32), _opt(cos, "cos", torch.float32),
             _opt(sin, "sin", torch.float32), _opt(slot_map, "slot_map", torch.int32), _req(q_out, "q_out"),
             _opt(kcache, "kcache", dt), _opt(vcache, "vcache", dt), T, nh, nkv, D, cos.shape[0] if cos is not None else 1,
             _tc_flag(qkv.device).data_ptr(), _stream())


def kv_cache_write(k: torch.Tensor, v: torch.Tensor, slot_map: torch.Tensor, kcache: torch.Tensor,
                   vcache: torch.Tensor) -> None:
    """k, v [T, nkv, D] -> rows slot_map[t] of the caches [pages, page, nkv, D] (negative slots are skipped)."""
    T = k.shape[0]
    width = k.numel() // max(T, 1)
    if v.shape != k.shape or kcache.shape[2:] != k.shape[1:] or vcache.shape != kcache.shape or slot_map.numel() < T:
        raise lib.KernelError("kv_cache_write: k / v / cache shapes disagree")
    dt = kcache.dtype
    lib.call("tm_kv_cache_write", _code(dt), _req(k, "k", dt), _req(v, "v", dt), _req(slot_map, "slot_map", torch.int32),
             _req(kcache, "kcache"), _req(vcache, "vcache", dt), T, width, _stream())


def paged_attention(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                    cu_q: torch.Tensor, kv_before: torch.Tensor, tile_seq: torch.Tensor, tile_row0: torch.Tensor,
                    n_tiles: int, out: torch.Tensor, *, scale: float, window: int = 0, split_keys: int = 0,
                    max_splits: int = 0, part_acc: torch.Tensor | None = None,
                    part_ml: torch.Tensor | None = None, seq_of_token: torch.Tensor | None = None) -> torch.Tensor:
    """q, out [T, nh, D]; caches [pages, page_size, nkv, D]; block_table [S, W] int32. With split_keys
    the partial results go through part_acc / part_ml and are merged into out by a second launch."""
    T, nh, D = q.shape
    page_size, nkv = kcache.shape[1], kcache.shape[2]
    if kcache.shape[3] != D or vcache.shape != kcache.shape or out.shape != q.shape:
        raise lib.KernelError("paged_attention: q / cache / out shapes disagree")
    dt = q.dtype
    if split_keys:
        need = T * nh * max_splits
        if part_acc is None or part_ml is None or seq_of_token is None or part_acc.numel() < need * D \
                or part_ml.numel() < need * 2:
            raise lib.KernelError("paged_attention: split mode needs part_acc, part_ml and seq_of_token of full size")
    lib.call("tm_paged_attention", _code(dt), _req(q, "q"), _req(kcache, "kcache", dt), _req(vcache, "vcache", dt),
             _req(block_table, "block_table", torch.int32), block_table.stride(0),
             _req(cu_q, "cu_q", torch.int32), _req(kv_before, "kv_before", torch.int32),
             _req(tile_seq, "tile_seq", torch.int32), _req(tile_row0, "tile_row0", torch.int32), n_tiles,
             _req(out, "out", dt), _opt(part_acc, "part_acc", torch.float32), _opt(part_ml, "part_ml", torch.float32),
             nh, nkv, D, page_size, float(scale), int(window), int(split_keys), int(max_splits), _stream())
    if split_keys:
        lib.call("tm_attention_combine", _code(dt), part_acc.data_ptr(), part_ml.data_ptr(), cu_q.data_ptr(),
                 kv_before.data_ptr(), _req(seq_of_token, "seq_of_token", torch.int32), out.data_ptr(), T, nh, D,
                 int(window), int(split_keys), int(max_splits), _stream())
    return out


def decode_attention_bf16(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                          cu_q: torch.Tensor, kv_before: torch.Tensor, n_seqs: int, out: torch.Tensor, *, scale: float,
                          window: int, split_keys: int, max_splits: int, part_acc: torch.Tensor, part_ml: torch.Tensor,
                          done: torch.Tensor | None = None) -> torch.Tensor:
    """Tensor-core attention for steps whose requests bring at most 16 / (nh / nkv) tokens each
    (decoding). bfloat16, head size 64 or 128; per-split partials through part_acc / part_ml, merged by the
    last block of each (request, kv head); ``done``: n_seqs * kv_heads int32 zeros (left zero), made here when
    not given."""
    T, nh, D = q.shape
    page_size, nkv = kcache.shape[1], kcache.shape[2]
    bf = torch.bfloat16
    need = T * nh * max_splits
    if part_acc.numel() < need * D or part_ml.numel() < need * 2:
        raise lib.KernelError("decode_attention_bf16: scratch too small")
    if kcache.shape[3] != D or vcache.shape != kcache.shape or out.shape != q.shape:
        raise lib.KernelError("decode_attention_bf16: q / cache / out shapes disagree")
    if done is None:
        done = torch.zeros(n_seqs * nkv, dtype=torch.int32, device=q.device)
    elif done.numel() < n_seqs * nkv:
        raise lib.KernelError("decode_attention_bf16: too few arrival counters")
    lib.call("tm_decode_attention_bf16", _req(q, "q", bf), _req(kcache, "kcache", bf), _req(vcache, "vcache", bf),
             _req(block_table, "block_table", torch.int32), block_table.stride(0), _req(cu_q, "cu_q", torch.int32),
             _req(kv_before, "kv_before", torch.int32), n_seqs, _req(part_acc, "part_acc", torch.float32),
             _req(part_ml, "part_ml", torch.float32), _req(out, "out", bf), _req(done, "done", torch.int32), nh, nkv, D,
             page_size, float(scale), int(window), int(split_keys), int(max_splits), _tc_flag(q.device).data_ptr(),
             _stream())
    return out


_DECODE_UNITS = os.environ.get("TOKENMILL_DECODE_UNITS", "1") != "0"


def decode_units_ok(page_size: int, head_dim: int) -> bool:
    """Whether decode attention runs as a persistent grid over a host-made list of units, with the keys and values
    brought in by tensor-map copies (attention_decode_tma_bf16.cu: pages of 8, 16, 32 or 64 tokens, heads of 64 or
    128). TOKENMILL_DECODE_UNITS=0 keeps the kernel with one block per (request, kv head, fixed split)."""
    return _DECODE_UNITS and page_size in (8, 16, 32, 64) and head_dim in (64, 128)


_units_slots: dict[tuple[int, int], int] = {}


def decode_units_slots(head_dim: int, device: torch.device | None = None) -> int:
    """Blocks of the unit-driven decode attention that are resident at once: what a plan of units should fill
    evenly (multiprocessors of the device; 148 where there is none to ask)."""
    sms = 148
    if device is not None and device.type == "cuda":
        sms = torch.cuda.get_device_properties(device).multi_processor_count
    key = (head_dim, sms)
    if key not in _units_slots:
        _units_slots[key] = sms * (4 if head_dim == 64 else 3)
    return _units_slots[key]


def decode_attention_units_bf16(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                                cu_q: torch.Tensor, kv_before: torch.Tensor, units: torch.Tensor, n_work: torch.Tensor,
                                out: torch.Tensor, *, scale: float, window: int, max_parts: int, grid: int,
                                part_acc: torch.Tensor, part_ml: torch.Tensor, done: torch.Tensor) -> torch.Tensor:
    """Tensor-core attention for steps whose requests bring at most 16 / (nh / nkv) tokens each (decoding), by a
    list of units (parts/attention_plan.py decode_units): ``units`` int32 [rows, 4] on the device, of which
    ``n_work`` (one int32 on the device) / kv_heads are valid; per-unit partials through part_acc / part_ml
    (``max_parts`` a request), merged by the block that writes a (request, kv head)'s last; ``done``:
    n_seqs * kv_heads int32 zeros (left zero); ``grid``: blocks to launch."""
    T, nh, D = q.shape
    page_size, nkv = kcache.shape[1], kcache.shape[2]
    bf, i32 = torch.bfloat16, torch.int32
    n_seqs = kv_before.numel()
    need = T * nh * max_parts
    if part_acc.numel() < need * D or part_ml.numel() < need * 2:
        raise lib.KernelError("decode_attention_units_bf16: scratch too small")
    if kcache.shape[3] != D or vcache.shape != kcache.shape or out.shape != q.shape:
        raise lib.KernelError("decode_attention_units_bf16: q / cache / out shapes disagree")
    if done.numel() < n_seqs * nkv:
        raise lib.KernelError("decode_attention_units_bf16: too few arrival counters")
    if units.dim() != 2 or units.shape[1] != 4 or units.data_ptr() % 16:
        raise lib.KernelError("decode_attention_units_bf16: units must be 16-byte aligned int32 records of 4")
    lib.call("tm_decode_attention_units_bf16", _req(q, "q", bf), _req(kcache, "kcache", bf), _req(vcache, "vcache", bf),
             kcache.shape[0], _req(block_table, "block_table", i32), block_table.stride(0), _req(cu_q, "cu_q", i32),
             _req(kv_before, "kv_before", i32), _req(units, "units", i32), _req(n_work, "n_work", i32),
             units.shape[0] * nkv, int(grid), _req(part_acc, "part_acc", torch.float32),
             _req(part_ml, "part_ml", torch.float32), _req(out, "out", bf), _req(done, "done", i32), nh, nkv, D, page_size,
             float(scale), int(window), int(max_parts), _tc_flag(q.device).data_ptr(), _stream())
    return out


_DECODE_ROPE = os.environ.get("TOKENMILL_DECODE_ROPE", "1") != "0"


def decode_rope_fused_ok() -> bool:
    """Whether the unit-driven decode attention finishes the q/k/v projection itself (bias, rotation, cache
    write) instead of the kernel that otherwise stands between the two. TOKENMILL_DECODE_ROPE=0 keeps that kernel."""
    return _DECODE_ROPE


def decode_attention_units_rope_bf16(qkv: torch.Tensor, bias: torch.Tensor | None, positions: torch.Tensor,
                                     cos: torch.Tensor, sin: torch.Tensor, slot_map: torch.Tensor, kcache: torch.Tensor,
                                     vcache: torch.Tensor, block_table: torch.Tensor, cu_q: torch.Tensor,
                                     kv_before: torch.Tensor, units: torch.Tensor, n_work: torch.Tensor,
                                     out: torch.Tensor, *, scale: float, window: int, max_parts: int, grid: int,
                                     part_acc: torch.Tensor, part_ml: torch.Tensor, done: torch.Tensor) -> torch.Tensor:
    """``decode_attention_units_bf16`` straight from the raw q/k/v product ``qkv`` [T, (nh + 2 nkv) D]: the kernel
    adds the bias, rotates queries and the new keys (rotate-half tables ``cos`` / ``sin`` [n_pos, D / 2]), writes
    each token's key and value to cache slot ``slot_map[t]`` and attends. ``out``: [T, nh, D]."""
    T, nh, D = out.shape
    page_size, nkv = kcache.shape[1], kcache.shape[2]
    bf, i32, f32 = torch.bfloat16, torch.int32, torch.float32
    n_seqs = kv_before.numel()
    need = T * nh * max_parts
    if part_acc.numel() < need * D or part_ml.numel() < need * 2:
        raise lib.KernelError("decode_attention_units_rope_bf16: scratch too small")
    if qkv.shape != (T, (nh + 2 * nkv) * D) or not qkv.is_contiguous() or kcache.shape[3] != D or vcache.shape != kcache.shape:
        raise lib.KernelError("decode_attention_units_rope_bf16: qkv / cache / out shapes disagree")
    if cos.shape != sin.shape or cos.shape[1] != D // 2 or not cos.is_contiguous() or not sin.is_contiguous():
        raise lib.KernelError("decode_attention_units_rope_bf16: rotation tables of [positions, head_dim / 2] wanted")
    if done.numel() < n_seqs * nkv:
        raise lib.KernelError("decode_attention_units_rope_bf16: too few arrival counters")
    if units.dim() != 2 or units.shape[1] != 4 or units.data_ptr() % 16:
        raise lib.KernelError("decode_attention_units_rope_bf16: units must be 16-byte aligned int32 records of 4")
    lib.call("tm_decode_attention_units_rope_bf16", _req(qkv, "qkv", bf), _opt(bias, "bias", f32),
             _req(positions, "positions", i32), _req(cos, "cos", f32), _req(sin, "sin", f32), cos.shape[0],
             _req(slot_map, "slot_map", i32), _req(kcache, "kcache", bf), _req(vcache, "vcache", bf), kcache.shape[0],
             _req(block_table, "block_table", i32), block_table.stride(0), _req(cu_q, "cu_q", i32),
             _req(kv_before, "kv_before", i32), _req(units, "units", i32), _req(n_work, "n_work", i32),
             units.shape[0] * nkv, int(grid), _req(part_acc, "part_acc", f32), _req(part_ml, "part_ml", f32),
             _req(out, "out", bf), _req(done, "done", i32), nh, nkv, D, page_size, float(scale), int(window),
             int(max_parts), _tc_flag(out.device).data_ptr(), _stream())
    return out


def prefill_attention_bf16(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                           units, counters: torch.Tensor, out: torch.Tensor, *, scale: float, window: int = 0,
                           part_acc: torch.Tensor | None = None, part_ml: torch.Tensor | None = None,
                           tile_done: torch.Tensor | None = None) -> torch.Tensor:
    """Tensor-core causal attention for prompt portions (bfloat16, head size 64 or 128). ``units``: the
    step's PrefillUnits for this group size (records of row tiles of 64 (token, head-in-group) rows cut into
    key chunks of units.chunk_keys, heaviest first); part_acc / part_ml: float32 scratch for the tiles with
    several chunks, at least n_slots * kv_heads * 64 * (head_dim | 2) elements, and tile_done, n_tiles *
    kv_heads int32 zeros (left zero); counters: two int32 zeros the kernel uses as work ticket and leaves zero."""
    T, nh, D = q.shape
    page_size, nkv = kcache.shape[1], kcache.shape[2]
    bf, i32 = torch.bfloat16, torch.int32
    if kcache.shape[3] != D or vcache.shape != kcache.shape or out.shape != q.shape:
        raise lib.KernelError("prefill_attention_bf16: q / cache / out shapes disagree")
    if scale <= 0:
        raise lib.KernelError("prefill_attention_bf16: the score scale must be positive")
    if units.tile_rows != 64:
        raise lib.KernelError("prefill_attention_bf16: units of 64-row tiles only")
    if units.n_slots and (part_acc is None or part_ml is None or tile_done is None
                          or part_acc.numel() < units.n_slots * nkv * 64 * D
                          or part_ml.numel() < units.n_slots * nkv * 64 * 2 or tile_done.numel() < units.n_tiles * nkv):
        raise lib.KernelError("prefill_attention_bf16: scratch for the partial results is missing or too small")
    lib.call("tm_prefill_attention_bf16", _req(q, "q", bf), _req(kcache, "kcache", bf), _req(vcache, "vcache", bf),
             _req(block_table, "block_table", i32), block_table.stride(0), _req(units.records, "unit records", i32),
             units.n_units, int(units.chunk_keys),
             _req(part_acc, "part_acc", torch.float32) if units.n_slots else None,
             _req(part_ml, "part_ml", torch.float32) if units.n_slots else None,
             _req(tile_done, "tile_done", i32) if units.n_slots else None,
             _req(counters, "counters", i32), _req(out, "out", bf), nh, nkv, D, page_size, float(scale), int(window),
             _stream())
    return out


def tc_attention_enabled() -> bool:
    """The tcgen05 prompt-attention kernel is used where it applies unless TOKENMILL_TC_ATTENTION=0."""
    return os.environ.get("TOKENMILL_TC_ATTENTION", "1") != "0"


def prefill_attention_tc_bf16(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                              units, counters: torch.Tensor, out: torch.Tensor, *, scale: float, window: int = 0,
                              part_acc: torch.Tensor | None = None, part_ml: torch.Tensor | None = None,
                              tile_done: torch.Tensor | None = None) -> torch.Tensor:
    """As prefill_attention_bf16, on tcgen05 with the scores and outputs in tensor memory: head size 64 or 128, units of
    128-row tiles (units.tile_rows == 128; the scratch holds 128 rows per slot). A block that gives up on a
    bounded wait raises the device error word that tc_check reads."""
    T, nh, D = q.shape
    page_size, nkv = kcache.shape[1], kcache.shape[2]
    bf, i32 = torch.bfloat16, torch.int32
    if D not in (64, 128) or units.tile_rows != 128:
        raise lib.KernelError("prefill_attention_tc_bf16: head size 64 or 128 and 128-row tiles only")
    if kcache.shape[3] != D or vcache.shape != kcache.shape or out.shape != q.shape:
        raise lib.KernelError("prefill_attention_tc_bf16: q / cache / out shapes disagree")
    if scale <= 0:
        raise lib.KernelError("prefill_attention_tc_bf16: the score scale must be positive")
    if units.n_slots and (part_acc is None or part_ml is None or tile_done is None
                          or part_acc.numel() < units.n_slots * nkv * 128 * D
                          or part_ml.numel() < units.n_slots * nkv * 128 * 2 or tile_done.numel() < units.n_tiles * nkv):
        raise lib.KernelError("prefill_attention_tc_bf16: scratch for the partial results is missing or too small")
    lib.call("tm_prefill_attention_tc_bf16", _req(q, "q", bf), _req(kcache, "kcache", bf), _req(vcache, "vcache", bf),
             _req(block_table, "block_table", i32), block_table.stride(0), _req(units.records, "unit records", i32),
             units.n_units, int(units.chunk_keys),
             _req(part_acc, "part_acc", torch.float32) if units.n_slots else None,
             _req(part_ml, "part_ml", torch.float32) if units.n_slots else None,
             _req(tile_done, "tile_done", i32) if units.n_slots else None,
             _req(counters, "counters", i32), _req(out, "out", bf), nh, nkv, D, page_size, float(scale), int(window),
             _tc_flag(q.device).data_ptr(), _stream())
    return out


def swiglu(gu: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """gu [T, 2 I] (gate columns first) -> out [T, I] = silu(gate) * up."""
    T, two_i = gu.shape
    if two_i % 2 or out.shape[0] < T or out.shape[1] * 2 != two_i:
        raise lib.KernelError(f"swiglu: gu {tuple(gu.shape)} and out {tuple(out.shape)} do not fit")
    lib.call("tm_swiglu", _code(gu.dtype), _req(gu, "gu"), _req(out, "out", gu.dtype), T, two_i // 2, _stream())
    return out


def linear(x: torch.Tensor, w: torch.Tensor, *, bias: torch.Tensor | None = None,
           out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """x [T, K] . w [N, K]^T -> [T, N].

    float32: this library's own CUDA-core kernel (true 32-bit, k-ordered accumulation).
    bfloat16: the library matrix product (cuBLAS through torch.mm), as the reference uses a library
    for its projections (src/infer/model/layers.py:144,150,163,164); fp32 accumulation, output in
    ``out_dtype`` (bfloat16 or float32)."""
    T, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise lib.KernelError(f"linear: x {tuple(x.shape)} and w {tuple(w.shape)} do not fit")
    if x.dtype == torch.float32:
        if out is None:
            out = torch.empty((T, N), dtype=torch.float32, device=x.device)
        lib.call("tm_gemm_f32_nt", _req(x, "x", torch.float32), x.stride(0), _req(w, "w", torch.float32),
                 _opt(bias, "bias", torch.float32), _req(out, "out", torch.float32), out.stride(0), T, N, K,
                 _stream())
        return out
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not x.is_cuda:
        raise lib.KernelError(f"linear: unsupported operands {x.dtype} / {w.dtype} on {x.device}")
    if bias is not None:
        raise lib.KernelError("linear: the bfloat16 product takes no bias (it is added by the kernel that follows)")
    want = out_dtype or (out.dtype if out is not None else torch.bfloat16)
    if want == torch.float32:
        res = torch.mm(x, w.t(), out_dtype=torch.float32)
        if out is not None:
            out.copy_(res)
            return out
        return res
    if out is not None:
        return torch.mm(x, w.t(), out=out)
    return torch.mm(x, w.t())


def argmax(logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """logits [n, V] float32 -> [n] int32, lowest index on ties."""
    n, V = logits.shape
    if logits.stride(1) != 1:
        raise lib.KernelError("argmax: rows must be contiguous")
    if out is None:
        out = torch.empty(n, dtype=torch.int32, device=logits.device)
    if not logits.is_cuda or logits.dtype != torch.float32:
        raise lib.KernelError("argmax: float32 logits on the GPU")
    chunks = lib.load().tm_argmax_chunks(V)
    sval = sidx = None
    if chunks > 1:                      # wide vocabulary: per-chunk winners, then a final pick
        sval = torch.empty(n * chunks, dtype=torch.float32, device=logits.device)
        sidx = torch.empty(n * chunks, dtype=torch.int32, device=logits.device)
    lib.call("tm_argmax", logits.data_ptr(), n, V, logits.stride(0), _req(out, "out", torch.int32),
             _opt(sval, "scratch"), _opt(sidx, "scratch"), _stream())
    return out


# TOKENMILL_SAMPLE_CLUSTER=0: every row sampled by one block (else rows of 8,192 logits and more go over a cluster
# of eight blocks, an eighth of the row in each block's shared memory).
_SAMPLE_CLUSTER = os.environ.get("TOKENMILL_SAMPLE_CLUSTER", "1") != "0"


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           uniform: torch.Tensor, rows: torch.Tensor | None = None, out: torch.Tensor | None = None,
           scatter: bool = False) -> torch.Tensor:
    """One draw per entry: entry i reads row rows[i] (default i) of logits [*, V] float32.
    temperature/top_p/uniform float32 [n], top_k int32 [n]; returns int32 [n]. With ``scatter`` (and rows and
    out given) draw i is written to out[rows[i]], so the draws land in an array indexed like the logits rows."""
    V = logits.shape[1]
    n = temperature.numel()
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise lib.KernelError("sample: float32 logits with contiguous rows on the GPU")
    if rows is None and logits.shape[0] < n:
        raise lib.KernelError("sample: fewer logits rows than draws")
    if out is None:
        out = torch.empty(n, dtype=torch.int32, device=logits.device)
    lib.call("tm_sample", logits.data_ptr(), n, V, logits.stride(0), _req(temperature, "temperature", torch.float32),
             _req(top_k, "top_k", torch.int32), _req(top_p, "top_p", torch.float32),
             _req(uniform, "uniform", torch.float32), _opt(rows, "rows", torch.int32),
             _req(out, "out", torch.int32), int(bool(scatter and rows is not None)),
             _tc_flag(logits.device).data_ptr() if _SAMPLE_CLUSTER else None, _stream())
    return out


# --- weight-streaming products for decode steps (bfloat16, at most 64 tokens) -------------------------

SKINNY_MAX_TOKENS = 16             # the kernel takes up to 64; beyond 16 the library product is faster today
# Matrices beyond this size go to the library product at every token count: the weight-streaming kernel tops out
# near 1.2 to 2.1 TB/s, which is what a small matrix gets anyway (its time is latency) but half of what the
# library reaches on a large one (7B layer sizes, 8 tokens: gate/up 127 vs 66 us, down 116 vs 42 us).
SKINNY_MAX_WEIGHT_BYTES = 20 << 20
_SKINNY_X_BYTES = 200 * 1024       # shared memory the staged activations may take


def _padded_tokens(T: int) -> int:
    return 16 if T <= 16 else (32 if T <= 32 else 64)


def skinny_ok(x: torch.Tensor, w: torch.Tensor, allow_split: bool = False) -> bool:
    """Whether the weight-streaming kernel takes this product (else the library product does).
    A product with a fused epilogue cannot cut its K range, so its activations must fit shared memory."""
    if not (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_cuda and x.dim() == 2
            and x.shape[0] <= SKINNY_MAX_TOKENS and w.numel() * 2 <= SKINNY_MAX_WEIGHT_BYTES
            and x.shape[1] % 8 == 0 and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.is_contiguous()):
        return False
    return allow_split or _padded_tokens(x.shape[0]) * (x.shape[1] + 64) * 2 <= _SKINNY_X_BYTES


def skinny_k_splits(T: int, K: int) -> int:
    """Cuts of the K range so that the staged activations fit shared memory."""
    return max(1, -(-(_padded_tokens(T) * K * 2) // _SKINNY_X_BYTES))


def skinny_linear(x: torch.Tensor, w: torch.Tensor, *, bias: torch.Tensor | None = None,
                  out_dtype: torch.dtype = torch.bfloat16, k_splits: int = 1, rows_per_block: int = 8) -> torch.Tensor:
    """x [T, K] . w [N, K]^T for T <= 64. k_splits == 1: returns [T, N] in out_dtype. k_splits > 1:
    returns float32 partial products [k_splits, T, N] for the add+norm kernel to sum."""
    T, K = x.shape
    N = w.shape[0]
    ng = rows_per_block // 8
    if k_splits > 1:
        partials = torch.empty((k_splits, T, N), dtype=torch.float32, device=x.device)
        lib.call("tm_skinny_linear", x.data_ptr(), x.stride(0), w.data_ptr(), None, None, 0, 0, partials.data_ptr(),
                 k_splits, T, N, K, ng, _stream())
        return partials
    out = torch.empty((T, N), dtype=out_dtype, device=x.device)
    lib.call("tm_skinny_linear", x.data_ptr(), x.stride(0), w.data_ptr(), _opt(bias, "bias", torch.float32),
             out.data_ptr(), N, 1 if out_dtype == torch.float32 else 0, None, 1, T, N, K, ng, _stream())
    return out


LM_HEAD_MAX_TOKENS, LM_HEAD_MAX_K = 16, 1024


def lm_head_ok(T: int, K: int) -> bool:
    """Whether the streaming output-matrix kernel takes a product of T tokens over K columns."""
    return 0 < T <= LM_HEAD_MAX_TOKENS and K % 8 == 0 and K <= LM_HEAD_MAX_K


def lm_head(x: torch.Tensor, w_packed: torch.Tensor, n_rows: int, error: torch.Tensor | None = None) -> torch.Tensor:
    """x [T, K] bfloat16 (T <= 16) times the output matrix, given as its packed copy (kernels/fused.py
    pack_rows of w [n_rows, K]) -> logits [T, n_rows] float32. The weights stream through shared memory at
    memory speed; the kernel's waits are bounded and report (code 21) through ``error``, an int32 device word
    that is zero, by default the word that tc_check reads."""
    T, K = x.shape
    if not lm_head_ok(T, K) or x.dtype != torch.bfloat16 or w_packed.dtype != torch.bfloat16:
        raise lib.KernelError(f"lm_head: {T} tokens of {K} columns in {x.dtype} are not taken")
    if w_packed.dim() != 5 or w_packed.shape[0] * 8 < n_rows or w_packed.shape[1] * 32 < K or not w_packed.is_contiguous():
        raise lib.KernelError("lm_head: the packed matrix does not fit the sizes given")
    out = torch.empty((T, n_rows), dtype=torch.float32, device=x.device)
    lib.call("tm_lm_head_bf16", _req(x, "x", torch.bfloat16), w_packed.data_ptr(), out.data_ptr(), T, n_rows, K,
             (error if error is not None else _tc_flag(x.device)).data_ptr(), _stream())
    return out


_lm_head_scratch: dict[torch.device, tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = {}


def lm_head_argmax(x: torch.Tensor, w_packed: torch.Tensor, n_rows: int, tokens: torch.Tensor,
                   logits: torch.Tensor | None = None, error: torch.Tensor | None = None) -> torch.Tensor:
    """``lm_head`` with the arg-max found in its epilogue: tokens[:T] (int32, on the device) receives the index
    of each token's largest logit, the lowest index on ties. ``logits`` [T, n_rows] float32 is written as well
    when given; without it no logits reach memory at all."""
    T, K = x.shape
    if not lm_head_ok(T, K) or x.dtype != torch.bfloat16 or w_packed.dtype != torch.bfloat16:
        raise lib.KernelError(f"lm_head_argmax: {T} tokens of {K} columns in {x.dtype} are not taken")
    if w_packed.dim() != 5 or w_packed.shape[0] * 8 < n_rows or w_packed.shape[1] * 32 < K or not w_packed.is_contiguous():
        raise lib.KernelError("lm_head_argmax: the packed matrix does not fit the sizes given")
    if tokens.dtype != torch.int32 or tokens.numel() < T or (logits is not None and logits.shape != (T, n_rows)):
        raise lib.KernelError("lm_head_argmax: tokens are int32 [T], logits float32 [T, rows]")
    if x.device not in _lm_head_scratch:       # per-block winners (one row of 16 per block) and the arrival counter
        n_blocks = torch.cuda.get_device_properties(x.device).multi_processor_count
        _lm_head_scratch[x.device] = (torch.empty(n_blocks * 16, dtype=torch.float32, device=x.device),
                                      torch.empty(n_blocks * 16, dtype=torch.int32, device=x.device),
                                      torch.zeros(1, dtype=torch.int32, device=x.device))
    best_val, best_idx, done = _lm_head_scratch[x.device]
    lib.call("tm_lm_head_argmax_bf16", _req(x, "x", torch.bfloat16), w_packed.data_ptr(),
             _opt(logits, "logits", torch.float32), _req(tokens, "tokens", torch.int32), best_val.data_ptr(),
             best_idx.data_ptr(), done.data_ptr(), T, n_rows, K,
             (error if error is not None else _tc_flag(x.device)).data_ptr(), _stream())
    return tokens


def stream_linear_ok(T: int, K: int) -> bool:
    """Whether the streaming kernel takes a product of T tokens over K columns (any number of rows)."""
    return 0 < T <= LM_HEAD_MAX_TOKENS and K % 8 == 0 and -(-K // 1024) <= 128


def stream_linear(x: torch.Tensor, w_packed: torch.Tensor, n_rows: int, error: torch.Tensor | None = None) -> torch.Tensor:
    """x [T, K] bfloat16 (T <= 16) times a matrix given as its packed copy (kernels/fused.py pack_rows of
    w [n_rows, K]) -> float32 partial products [S, T, n_rows], one per slice of at most 1024 columns of K
    (S = 1 for K <= 1024): the weights stream through shared memory at the memory's rate. The norm kernel adds
    such slices in index order (``Pending.partials``), ``swiglu_partials`` does for a gate/up product."""
    T, K = x.shape
    if not stream_linear_ok(T, K) or x.dtype != torch.bfloat16 or w_packed.dtype != torch.bfloat16:
        raise lib.KernelError(f"stream_linear: {T} tokens of {K} columns in {x.dtype} are not taken")
    if w_packed.dim() != 5 or w_packed.shape[0] * 8 < n_rows or w_packed.shape[1] * 32 < K or not w_packed.is_contiguous():
        raise lib.KernelError("stream_linear: the packed matrix does not fit the sizes given")
    S = int(lib.load().tm_stream_linear_slices(K))
    out = torch.empty((S, T, n_rows), dtype=torch.float32, device=x.device)
    lib.call("tm_stream_linear_bf16", _req(x, "x", torch.bfloat16), w_packed.data_ptr(), out.data_ptr(), T, n_rows, K,
             (error if error is not None else _tc_flag(x.device)).data_ptr(), _stream())
    return out


def swiglu_partials(parts: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """parts [S, T, 2 I] float32 partial gate/up products -> out [T, I] bfloat16 = silu(gate) * up."""
    S, T, two_i = parts.shape
    if two_i % 8 or out.shape != (T, two_i // 2) or out.dtype != torch.bfloat16:
        raise lib.KernelError(f"swiglu_partials: parts {tuple(parts.shape)} and out {tuple(out.shape)} do not fit")
    lib.call("tm_swiglu_partials", _req(parts, "parts", torch.float32), S, parts.stride(0), _req(out, "out", torch.bfloat16),
             T, two_i // 2, _stream())
    return out


def skinny_qkv_rope_write(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, positions: torch.Tensor,
                          cos: torch.Tensor, sin: torch.Tensor, slot_map: torch.Tensor | None, q_out: torch.Tensor,
                          kcache: torch.Tensor | None, vcache: torch.Tensor | None, nh: int, nkv: int, D: int) -> None:
    """The fused q/k/v projection of a decode step with its whole epilogue: bias, position encoding,
    q to q_out, k and v to their cache slots."""
    T, K = x.shape
    if w.shape != ((nh + 2 * nkv) * D, K) or cos.shape[1] * 2 != D:
        raise lib.KernelError("skinny_qkv_rope_write: shapes do not fit")
    bf = torch.bfloat16
    lib.call("tm_skinny_qkv_rope_write", x.data_ptr(), x.stride(0), _req(w, "w", bf), _opt(bias, "bias", torch.float32),
             _req(positions, "positions", torch.int32), _req(cos, "cos", torch.float32),
             _req(sin, "sin", torch.float32), _opt(slot_map, "slot_map", torch.int32), _req(q_out, "q_out", bf),
             _opt(kcache, "kcache", bf), _opt(vcache, "vcache", bf), T, K, nh, nkv, D, cos.shape[0],
             _tc_flag(x.device).data_ptr(), _stream())


def skinny_gate_up_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out [T, I] = silu(x . gate^T) * (x . up^T), w_gate_up [2 I, K] with the gate rows first."""
    T, K = x.shape
    inter = w_gate_up.shape[0] // 2
    lib.call("tm_skinny_gate_up_swiglu", x.data_ptr(), x.stride(0), _req(w_gate_up, "w_gate_up", torch.bfloat16),
             _req(out, "out", torch.bfloat16), out.stride(0), T, K, inter, _stream())
    return out


# --- prompt-step products on tcgen05 tensor cores (bfloat16) ------------------------------------------

TC_MIN_TOKENS = 128                # below this the 128-token tiles are mostly padding
# Which prompt-step products run on this library's tcgen05 kernels (TOKENMILL_TC_GEMM): "0" (default) none: they
# go to the library product, as in the reference; "qkv": the q/k/v projection with bias, rotation and cache write in
# its epilogue, and narrow plain products (o_proj), both while tiles of 128 columns fill the chip in one wave; "1"
# every prompt product. Measured inside the prompt step at the 0.5B layer sizes (24 layers, 2,048 tokens): 3.83 ms
# with "0", 4.07 ms with "qkv" (at 512 tokens 2.16 against 2.45 ms; 1.5B sizes, 8 layers: 2.69 against 2.90 ms):
# one wave of tiles with its epilogue exposed, two tensor maps encoded per launch and the kernel's set-up cost more
# than the rotary kernel and the launch they save, so the default stays with the library. (A loop of Python-driven
# launches shows the opposite, 21 against 34 us, because there the library path pays two interpreter round trips.)
_TC_MODE = os.environ.get("TOKENMILL_TC_GEMM", "0")
if _TC_MODE == "auto":
    _TC_MODE = "qkv"
if _TC_MODE not in ("qkv", "0", "1"):
    _TC_MODE = "0"
TC_QKV_MIN_TOKENS = 384            # fused q/k/v projection: tokens from which it beats library product + rotary kernel
TC_NARROW_MIN_TOKENS = 1024        # plain narrow product: tokens from which it beats the library product
_tc_error: dict[torch.device, torch.Tensor] = {}
_sm_count: dict[int, int] = {}


def tc_gemm_enabled() -> bool:
    """Whether EVERY prompt-step product goes to the tcgen05 kernels (TOKENMILL_TC_GEMM=1)."""
    return _TC_MODE == "1"


def _sms(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _sm_count:
        _sm_count[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _sm_count[idx]


def tc_one_wave(T: int, N: int, device: torch.device) -> bool:
    """Whether the tcgen05 kernel takes the product in tiles of 128 columns that fill the chip in one wave (it does
    so while tiles of 256 columns would leave SMs without a tile)."""
    return -(-T // 128) * -(-N // 256) < _sms(device)


def _tc_flag(device: torch.device) -> torch.Tensor:
    if device not in _tc_error:
        _tc_error[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return _tc_error[device]


tc_error_word = _tc_flag


_tc_host: dict[torch.device, torch.Tensor] = {}


def tc_post(device: torch.device) -> None:
    """Send the error word on its way to pinned host memory behind the work launched so far, without waiting;
    ``tc_poll`` looks at the copy."""
    flag = _tc_error.get(device)
    if flag is not None:
        if device not in _tc_host:
            _tc_host[device] = torch.zeros(1, dtype=torch.int32, pin_memory=True)
        _tc_host[device].copy_(flag, non_blocking=True)


def tc_poll(device: torch.device) -> None:
    """Raise if the last copy ``tc_post`` made that has arrived holds an error (no synchronisation: a failure
    shows once the stream has been synchronised, at the latest one step later)."""
    host = _tc_host.get(device)
    if host is not None and int(host[0]):
        with torch.inference_mode():         # (the word may have been made inside a step: an inference tensor)
            host.zero_()
        tc_check(device)


def tc_check(device: torch.device) -> None:
    """Raise if a kernel reported through the device error word since the last check: a tcgen05 block that gave
    up on a bounded wait, or a position outside the rotary tables (reads one int back, which waits for the
    device)."""
    flag = _tc_error.get(device)
    if flag is not None:
        code = int(flag.item())
        if code:
            with torch.inference_mode():     # (the word may have been made inside a step: an inference tensor)
                flag.zero_()
            if code == 32:
                raise lib.KernelError("decode attention met a request with more rows than a tile holds, keys beyond "
                                      "max_splits * split_keys or a unit of more stages than it takes; its output is "
                                      "incomplete")
            if code in (33, 34):
                raise lib.KernelError(f"decode attention gave up waiting for {'a stage of keys' if code == 33 else 'a free stage'}"
                                      f" (code {code}); its output is incomplete")
            if code == 41:
                raise lib.KernelError("sampling: a block of a row's cluster gave up waiting for the others; the "
                                      "step's tokens are incomplete")
            if code == 31:
                raise lib.KernelError("a token's position lies outside the position tables (the rotation was not "
                                      "applied as asked; the step's results are wrong)")
            raise lib.KernelError(f"a tcgen05 block gave up waiting (code {code}: matrix product 1 loader, 2/3 issuer, "
                                  f"4 epilogue; attention 11/13 second product, 12 scores, 14 merge; 21 output matrix stream); "
                                  f"its results are incomplete")


def _tc_operands_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_cuda and x.dim() == 2
            and x.shape[0] >= TC_MIN_TOKENS and x.shape[1] % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.is_contiguous() and w.data_ptr() % 16 == 0)


def tc_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether a wide prompt product (gate/up, down) goes to the tcgen05 kernels: only with TOKENMILL_TC_GEMM=1."""
    return _TC_MODE == "1" and _tc_operands_ok(x, w)


def tc_qkv_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the q/k/v projection of a prompt step runs as ONE tcgen05 kernel with bias, rotation and cache write
    in its epilogue (else: library product, then the rotary kernel)."""
    if _TC_MODE == "0" or not _tc_operands_ok(x, w):
        return False
    return _TC_MODE == "1" or (x.shape[0] >= TC_QKV_MIN_TOKENS and tc_one_wave(x.shape[0], w.shape[0], x.device))


def tc_narrow_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether a plain narrow prompt product (o_proj) runs on the tcgen05 kernel."""
    if _TC_MODE == "0" or not _tc_operands_ok(x, w):
        return False
    return _TC_MODE == "1" or (x.shape[0] >= TC_NARROW_MIN_TOKENS and tc_one_wave(x.shape[0], w.shape[0], x.device))


def tc_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """x [T, K] . w [N, K]^T -> [T, N] bfloat16 on tcgen05 (N a multiple of 8)."""
    T, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty((T, N), dtype=torch.bfloat16, device=x.device)
    lib.call("tm_tc_linear", x.data_ptr(), x.stride(0), w.data_ptr(), _req(out, "out", torch.bfloat16), out.stride(0),
             T, N, K, _tc_flag(x.device).data_ptr(), _stream())
    return out


_TC_ADD = os.environ.get("TOKENMILL_TC_DECODE", "1") != "0"
_TC_ADD_ALL = os.environ.get("TOKENMILL_TC_DECODE", "1") == "all"
TC_ADD_MIN_TOKENS, TC_ADD_MAX_TOKENS = 1, 128
TC_ADD_MIN_K = 2048     # shorter rows: the library's kernel is as fast (o_proj of 896: 4.9 us against 6 us here). Rows of
                        # 3,584 (the 7B sizes' output projection) win inside the step (3.45 against 3.54 ms at batch 8)
                        # although the library's kernel is ahead when both are timed alone (9 against 12 us).


def tc_add_ok(x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor | None) -> bool:
    """Whether ``tc_linear_add`` takes this projection: a step of up to 128 tokens (the callers ask the
    weight-streaming kernels first, which take small matrices at up to 16 tokens; above 128 tokens the library
    product is one pass over the weights at full tiles anyway), rows long enough
    that cutting them pays (the down projection: 7.9 us against the library's 9.5 at 64 x 4864 -> 896), bfloat16
    operands, a 32-bit residual stream of the product's shape. TOKENMILL_TC_DECODE=0 switches it off; =all takes
    short rows too."""
    return (_TC_ADD and resid is not None and x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and x.dim() == 2 and TC_ADD_MIN_TOKENS <= x.shape[0] <= TC_ADD_MAX_TOKENS and x.shape[1] % 8 == 0
            and (x.shape[1] >= TC_ADD_MIN_K or _TC_ADD_ALL)
            and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.is_contiguous()
            and w.data_ptr() % 16 == 0 and w.shape[0] % 4 == 0 and resid.dtype == torch.float32
            and resid.shape == (x.shape[0], w.shape[0]) and resid.stride(1) == 1 and resid.stride(0) % 4 == 0
            and resid.data_ptr() % 16 == 0)


def tc_swiglu_decode_ok(x: torch.Tensor, w_gate_up: torch.Tensor) -> bool:
    """Whether a step of up to 128 tokens takes its gate/up projection with the activation in the epilogue on
    tcgen05 (tiles of 32 gate and 32 up rows, one for every multiprocessor) instead of the library product and
    the activation kernel. Only with TOKENMILL_TC_DECODE=all: measured at 64 tokens, 896 -> 2 x 4864, the fused
    kernel takes about 16 us against the library's 7.0 + 2.8 us (every tile reads all of x again, 14 blocks of K
    one after the other), so a step of 64 requests takes 1.37 ms with it and 1.21 without."""
    return (_TC_ADD_ALL and x.is_cuda and x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and x.dim() == 2
            and TC_ADD_MIN_TOKENS <= x.shape[0] <= TC_ADD_MAX_TOKENS and x.shape[1] % 8 == 0 and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w_gate_up.is_contiguous()
            and w_gate_up.data_ptr() % 16 == 0 and (w_gate_up.shape[0] // 2) % 8 == 0)


def tc_linear_add(x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor) -> None:
    """resid [T, N] float32 += x [T, K] . w [N, K]^T on tcgen05, the K range cut over the chip (atomic adds)."""
    T, K = x.shape
    lib.call("tm_tc_linear_add_f32", x.data_ptr(), x.stride(0), w.data_ptr(), _req(resid, "resid", torch.float32),
             resid.stride(0), T, w.shape[0], K, _tc_flag(x.device).data_ptr(), _stream())


def tc_gate_up_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out [T, I] = silu(x . gate^T) * (x . up^T) on tcgen05; the [T, 2I] product stays in tensor memory."""
    T, K = x.shape
    lib.call("tm_tc_gate_up_swiglu", x.data_ptr(), x.stride(0), _req(w_gate_up, "w_gate_up", torch.bfloat16),
             _req(out, "out", torch.bfloat16), out.stride(0), T, K, w_gate_up.shape[0] // 2,
             _tc_flag(x.device).data_ptr(), _stream())
    return out


def tc_qkv_rope_write(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, positions: torch.Tensor,
                      cos: torch.Tensor, sin: torch.Tensor, slot_map: torch.Tensor | None, q_out: torch.Tensor,
                      kcache: torch.Tensor | None, vcache: torch.Tensor | None, nh: int, nkv: int, D: int) -> None:
    """The fused q/k/v projection of a prompt step on tcgen05, epilogue as skinny_qkv_rope_write."""
    T, K = x.shape
    bf = torch.bfloat16
    lib.call("tm_tc_qkv_rope_write", x.data_ptr(), x.stride(0), _req(w, "w", bf), _opt(bias, "bias", torch.float32),
             _req(positions, "positions", torch.int32), _req(cos, "cos", torch.float32),
             _req(sin, "sin", torch.float32), _opt(slot_map, "slot_map", torch.int32), _req(q_out, "q_out", bf),
             _opt(kcache, "kcache", bf), _opt(vcache, "vcache", bf), T, K, nh, nkv, D, cos.shape[0],
             _tc_flag(x.device).data_ptr(), _stream())


# --- 32-bit norms for parallel blocks, token shift ------------------------------------------------------------

def add_norm_pair(resid: torch.Tensor, w1: torch.Tensor, eps: float, out1: torch.Tensor, *, dtype: torch.dtype,
                  w2: torch.Tensor | None = None, out2: torch.Tensor | None = None, a: torch.Tensor | None = None,
                  b: torch.Tensor | None = None, scale: float = 1.0, ids: torch.Tensor | None = None,
                  table: torch.Tensor | None = None, rows: torch.Tensor | None = None) -> None:
    """resid [T, H] float32 += scale * (a + b) (or = table[ids]); out1 = norm(resid) * w1 (float32 or ``dtype``),
    out2 = norm(resid) * w2 (``dtype``, optional). 32-bit arithmetic, each output rounded once. With ``rows`` only
    those rows are normed and the stream is not written."""
    H = resid.shape[-1]
    n_rows = rows.numel() if rows is not None else resid.shape[0]
    if out1.shape[0] < n_rows or out1.shape[-1] != H or w1.numel() != H or (out2 is None) != (w2 is None):
        raise lib.KernelError("add_norm_pair: outputs and weights do not fit the stream")
    if out1.dtype not in (torch.float32, dtype) or (ids is None) != (table is None):
        raise lib.KernelError("add_norm_pair: out1 is float32 or the activation dtype; ids and table come together")
    lib.call("tm_add_norm_pair", _code(dtype), _req(resid, "resid", torch.float32), _opt(a, "a", dtype),
             _opt(b, "b", dtype), float(scale), _opt(ids, "ids", torch.int32), _opt(table, "table", dtype),
             _opt(rows, "rows", torch.int32), _req(w1, "w1", torch.float32), _opt(w2, "w2", torch.float32), float(eps),
             _req(out1, "out1"), int(out1.dtype == torch.float32 and dtype != torch.float32), _opt(out2, "out2", dtype),
             n_rows, H, _stream())


def token_shift(h: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, cu_q: torch.Tensor, seq_of_token: torch.Tensor,
                state_slots: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] = h[t] + (h[t-1] - h[t]) * mu; a request's first row takes h[t-1] from its slot of ``state``
    [slots, >= H] float32, which then receives the request's last h of this step."""
    T, H = h.shape
    if state.dim() != 2 or state.shape[1] < H or mu.numel() != H or out.shape != h.shape:
        raise lib.KernelError("token_shift: shapes do not fit")
    lib.call("tm_token_shift", _code(out.dtype), _req(h, "h", torch.float32), _req(mu, "mu", torch.float32),
             _req(state, "state", torch.float32), state.stride(0), _req(cu_q, "cu_q", torch.int32),
             _req(seq_of_token, "seq_of_token", torch.int32), _req(state_slots, "state_slots", torch.int32),
             _req(out, "out"), T, H, _stream())
    return out


def gated_group_norm(y: torch.Tensor, proj: torch.Tensor, weight: torch.Tensor, eps: float, groups: int,
                     out: torch.Tensor) -> torch.Tensor:
    """out = group_rms_norm(y * silu(z)) * weight; y [T, inner] float32, z = proj[:, :inner]."""
    T, inner = y.shape
    if proj.shape[0] != T or proj.shape[1] < inner or weight.numel() != inner or out.shape != y.shape:
        raise lib.KernelError("gated_group_norm: shapes do not fit")
    lib.call("tm_gated_group_norm", _code(out.dtype), _req(y, "y", torch.float32), _req(proj, "proj", out.dtype),
             proj.stride(0), _req(weight, "weight", torch.float32), float(eps), _req(out, "out"), T, inner, int(groups),
             _stream())
    return out


# --- attention over a cache of latents ------------------------------------------------------------------------

def latent_prepare(proj: torch.Tensor, q_rank: int, rank: int, rot: int, rot_dims: int, wq: torch.Tensor,
                   wkv: torch.Tensor, eps: float, positions: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                   slot_map: torch.Tensor, cq_out: torch.Tensor, cache: torch.Tensor) -> None:
    """proj [T, q_rank + rank + rot] -> cq_out [T, q_rank] (normed), cache rows slot_map[t] = [norm(c) | rope(k_rot)]."""
    T = proj.shape[0]
    if proj.shape[1] != q_rank + rank + rot or cache.shape[-1] != rank + rot or cos.shape[1] * 2 != rot_dims or \
            cq_out.shape != (T, q_rank):
        raise lib.KernelError("latent_prepare: shapes do not fit")
    dt = proj.dtype
    lib.call("tm_latent_prepare", _code(dt), _req(proj, "proj"), q_rank, rank, rot, rot_dims, _req(wq, "wq", torch.float32),
             _req(wkv, "wkv", torch.float32), float(eps), _req(positions, "positions", torch.int32),
             _req(cos, "cos", torch.float32), _req(sin, "sin", torch.float32), cos.shape[0],
             _req(slot_map, "slot_map", torch.int32), _req(cq_out, "cq_out", dt), _req(cache, "cache", dt), T,
             _tc_flag(proj.device).data_ptr(), _stream())


def latent_attention_tc_ok(dtype: torch.dtype, rank: int, rot: int) -> bool:
    """Whether the tensor-core kernel takes these shapes (bfloat16, both parts of a cache row multiples of 16 wide)."""
    return dtype == torch.bfloat16 and rank % 16 == 0 and rot % 16 == 0 and \
        os.environ.get("TOKENMILL_LATENT_TC", "1") != "0"


LATENT_TC_TILE_ROWS, LATENT_TILE_ROWS = 64, 32
LATENT_TC_PAIRED = os.environ.get("TOKENMILL_LATENT_PAIRED", "1") != "0"    # the tensor-core kernel with warps in pairs


def latent_attention_tc_chunks(rank: int) -> int:
    """Blocks that share a row tile of the tensor-core kernel (each takes a slice of the result columns)."""
    if LATENT_TC_PAIRED:
        return -(-rank // (64 if rank <= 64 else 128 if rank <= 128 else 256 if rank <= 256 else 512))
    return -(-rank // (64 if rank <= 64 else 128 if rank <= 128 else 256))


def latent_attention(q_lat: torch.Tensor, q_rot: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rot_dims: int,
                     cache: torch.Tensor, block_table: torch.Tensor, cu_q: torch.Tensor, kv_before: torch.Tensor,
                     tile_seq: torch.Tensor, tile_row0: torch.Tensor, n_tiles: int, out: torch.Tensor, *, scale: float,
                     window: int, tensor_cores: bool = False, n_splits: int = 1,
                     part: torch.Tensor | None = None, paired: bool | None = None) -> torch.Tensor:
    """q_lat [T, nh, rank] float32, q_rot [T, nh, rot] (unrotated), out [T, nh, rank]: any strides with a unit last
    one; cache [pages, page, 1, rank + rot]. Tiles of 32 (token, head) rows, or of 64 with ``tensor_cores``
    (bfloat16, mma.sync; see ``latent_attention_tc_ok``); that kernel may deal a tile's keys out in ``n_splits``
    runs, whose partial results pass through ``part`` (n_tiles * n_splits * 64 * (rank + 2) float32)."""
    T, nh, rank = q_lat.shape
    rot = q_rot.shape[2]
    dt = cache.dtype
    for t, name in ((q_lat, "q_lat"), (q_rot, "q_rot"), (out, "out")):
        if not t.is_cuda or t.stride(2) != 1:
            raise lib.KernelError(f"latent_attention: {name} must be on the GPU with a unit last stride")
    if q_lat.dtype != torch.float32 or q_rot.dtype != dt or out.dtype != dt or out.shape != q_lat.shape or \
            cache.shape[-1] != rank + rot or cos.shape[1] * 2 != rot_dims:
        raise lib.KernelError("latent_attention: dtypes or shapes do not fit")
    if tensor_cores:
        if not latent_attention_tc_ok(dt, rank, rot):
            raise lib.KernelError("latent_attention: the tensor-core kernel takes bfloat16 with rank and rot multiples of 16")
        if n_splits > 1 and (part is None or part.numel() < n_tiles * n_splits * LATENT_TC_TILE_ROWS * (rank + 2)):
            raise lib.KernelError("latent_attention: scratch for the split runs is missing or too small")
        lib.call("tm_latent_attention_mma_bf16", q_lat.data_ptr(), q_lat.stride(0), q_lat.stride(1), q_rot.data_ptr(),
                 q_rot.stride(0), q_rot.stride(1), _req(cos, "cos", torch.float32), _req(sin, "sin", torch.float32), rot_dims,
                 _req(cache, "cache"), _req(block_table, "block_table", torch.int32), block_table.stride(0),
                 _req(cu_q, "cu_q", torch.int32), _req(kv_before, "kv_before", torch.int32),
                 _req(tile_seq, "tile_seq", torch.int32), _req(tile_row0, "tile_row0", torch.int32), n_tiles, out.data_ptr(),
                 out.stride(0), out.stride(1), nh, rank, rot, cache.shape[1], float(scale), int(window), int(n_splits),
                 _opt(part, "part", torch.float32), int(LATENT_TC_PAIRED if paired is None else paired), _stream())
        return out
    lib.call("tm_latent_attention", _code(dt), q_lat.data_ptr(), q_lat.stride(0), q_lat.stride(1), q_rot.data_ptr(),
             q_rot.stride(0), q_rot.stride(1), _req(cos, "cos", torch.float32), _req(sin, "sin", torch.float32), rot_dims,
             _req(cache, "cache"), _req(block_table, "block_table", torch.int32), block_table.stride(0),
             _req(cu_q, "cu_q", torch.int32), _req(kv_before, "kv_before", torch.int32),
             _req(tile_seq, "tile_seq", torch.int32), _req(tile_row0, "tile_row0", torch.int32), n_tiles, out.data_ptr(),
             out.stride(0), out.stride(1), nh, rank, rot, cache.shape[1], float(scale), int(window), _stream())
    return out


def bmm_nt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[b] = a[b] . w[b]^T for a [B, M, K], w [B, N, K] (contiguous), out [B, M, N]; a and out may be strided views
    with a unit last stride. float32: this library's CUDA-core kernel (true 32-bit); bfloat16 in, float32 or
    bfloat16 out: the library's batched product."""
    B, M, K = a.shape
    N = w.shape[1]
    if w.shape != (B, N, K) or out.shape != (B, M, N) or a.stride(2) != 1 or out.stride(2) != 1:
        raise lib.KernelError("bmm_nt: shapes do not fit")
    if a.dtype == torch.float32 and w.dtype == torch.float32 and out.dtype == torch.float32:
        lib.call("tm_gemm_f32_nt_batched", a.data_ptr(), a.stride(0), a.stride(1), _req(w, "w"), w.stride(0),
                 out.data_ptr(), out.stride(0), out.stride(1), B, M, N, K, _stream())
        return out
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise lib.KernelError(f"bmm_nt: unsupported operands {a.dtype} / {w.dtype}")
    if out.dtype == torch.float32:
        out.copy_(torch.bmm(a, w.transpose(1, 2), out_dtype=torch.float32))
    else:
        torch.bmm(a, w.transpose(1, 2), out=out)
    return out


# --- state-space mixer ----------------------------------------------------------------------------------------

def conv_silu_state(proj: torch.Tensor, col0: int, channels: int, weight: torch.Tensor, bias: torch.Tensor | None,
                    state: torch.Tensor, cu_q: torch.Tensor, seq_of_token: torch.Tensor, state_slots: torch.Tensor,
                    out: torch.Tensor, weight_t: torch.Tensor | None = None) -> torch.Tensor:
    """Causal convolution + silu over columns col0 .. col0 + channels of proj [T, P]; weight [channels, taps] float32;
    the request's last taps - 1 inputs live at the start of its slot of ``state`` [slots, n] float32. ``weight_t``: the
    weights once more as [taps, channels], which the 16-bytes-per-access kernel reads."""
    if weight_t is not None and tuple(weight_t.shape) != (weight.shape[1], weight.shape[0]):
        raise lib.KernelError("conv_silu_state: weight_t is weight transposed")
    T = proj.shape[0]
    taps = weight.shape[1]
    if weight.shape[0] != channels or out.shape != (T, channels) or state.shape[1] < (taps - 1) * channels or \
            col0 + channels > proj.shape[1]:
        raise lib.KernelError("conv_silu_state: shapes do not fit")
    lib.call("tm_conv_silu_state", _code(proj.dtype), _req(proj, "proj"), proj.stride(0), col0, channels, taps,
             _req(weight, "weight", torch.float32), _opt(weight_t, "weight_t", torch.float32),
             _opt(bias, "bias", torch.float32), _req(state, "state", torch.float32),
             state.stride(0), _req(cu_q, "cu_q", torch.int32), _req(seq_of_token, "seq_of_token", torch.int32),
             _req(state_slots, "state_slots", torch.int32), _req(out, "out", proj.dtype), T, _stream())
    return out


def ssm_scan(xbc: torch.Tensor, proj: torch.Tensor, dt_col: int, A_log: torch.Tensor, dt_bias: torch.Tensor,
             D: torch.Tensor, state: torch.Tensor, state_off: int, cu_q: torch.Tensor, state_slots: torch.Tensor,
             y: torch.Tensor, *, n_seqs: int, heads: int, vdim: int, N: int, groups: int, max_q_len: int = 64,
             slice_len: int = 0, slice_S: torch.Tensor | None = None, slice_a: torch.Tensor | None = None) -> torch.Tensor:
    """The state recurrence over this step's tokens; y [T, heads * vdim] float32; S of a request lives at
    ``state_off`` inside its slot, laid out [heads, vdim, N]. ``slice_len`` > 0: three passes over time slices of
    that many tokens (for long prompt portions), through ``slice_S`` (n_seqs * slices * heads * vdim * N float32)
    and ``slice_a`` (n_seqs * slices * heads float32), slices = ceil(max_q_len / slice_len)."""
    T, channels = xbc.shape
    if channels != heads * vdim + 2 * groups * N or y.shape != (T, heads * vdim) or \
            state.shape[1] < state_off + heads * vdim * N or dt_col + heads > proj.shape[1]:
        raise lib.KernelError("ssm_scan: shapes do not fit")
    def scan(mode, max_slices):
        lib.call("tm_ssm_scan", _code(xbc.dtype), _req(xbc, "xbc"), channels, _req(proj, "proj", xbc.dtype), proj.stride(0),
                 dt_col, _req(A_log, "A_log", torch.float32), _req(dt_bias, "dt_bias", torch.float32),
                 _req(D, "D", torch.float32), _req(state, "state", torch.float32), state.stride(0), int(state_off),
                 _req(cu_q, "cu_q", torch.int32), _req(state_slots, "state_slots", torch.int32), _req(y, "y", torch.float32),
                 int(n_seqs), heads, vdim, N, groups, int(max_q_len), mode, int(slice_len), max_slices,
                 _opt(slice_S, "slice_S", torch.float32), _opt(slice_a, "slice_a", torch.float32), _stream())

    if slice_len <= 0:
        scan(0, 1)
        return y
    slices = -(-int(max_q_len) // int(slice_len))
    if slice_S is None or slice_a is None or slice_S.numel() < n_seqs * slices * heads * vdim * N or \
            slice_a.numel() < n_seqs * slices * heads:
        raise lib.KernelError("ssm_scan: scratch for the time slices is missing or too small")
    scan(1, slices)
    lib.call("tm_ssm_pass_states", state.data_ptr(), state.stride(0), int(state_off), cu_q.data_ptr(), state_slots.data_ptr(),
             slice_S.data_ptr(), slice_a.data_ptr(), int(n_seqs), heads, vdim, N, int(slice_len), slices, _stream())
    scan(2, slices)
    return y


# --- feed-forwards beyond SwiGLU ------------------------------------------------------------------------------

def relu2(x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out = max(x, 0)^2, elementwise."""
    if out.shape != x.shape or out.dtype != x.dtype:
        raise lib.KernelError("relu2: out must match x")
    lib.call("tm_relu2", _code(x.dtype), _req(x, "x"), _req(out, "out"), x.numel(), _stream())
    return out


def moe_route(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, top: int, w_low: torch.Tensor | None = None):
    """x [T, H]; w [E, H] float32 -> (top_idx [T, top] int32, top_w [T, top] float32, dense_w [T, E] float32). The
    logits are 32-bit: this library's 32-bit product for float32 inputs; for bfloat16 inputs the library's product
    of x with ``w_low``, a bfloat16 copy of w that holds the same values, with its 32-bit accumulator as the result
    (products of two bfloat16 numbers are exact in 32-bit), or x converted and the 32-bit product when there is no
    such copy."""
    T, H = x.shape
    E = w.shape[0]
    if x.dtype == torch.float32:
        logits, bias = linear(x, w, bias=bias), None
    elif w_low is not None:
        logits = torch.mm(x, w_low.t(), out_dtype=torch.float32)
    else:
        logits, bias = linear(x.float(), w, bias=bias), None
    idx = torch.empty((T, top), dtype=torch.int32, device=x.device)
    tw = torch.empty((T, top), dtype=torch.float32, device=x.device)
    dense = torch.empty((T, E), dtype=torch.float32, device=x.device)
    lib.call("tm_moe_topk", _req(logits, "logits", torch.float32), _opt(bias, "bias", torch.float32), idx.data_ptr(),
             tw.data_ptr(), dense.data_ptr(), T, E, int(top), E, 0, _stream())
    return idx, tw, dense


MOE_SCORING = {"softmax_of_chosen": 0, "sigmoid": 1}


def moe_topk(logits: torch.Tensor, experts: int, top: int, scoring: str):
    """logits [T, >= experts] float32 (further columns are not read) -> (top_idx [T, top] int32, top_w [T, top], dense_w
    [T, experts] float32): the ``top`` largest logits, the lowest index winning a tie; weights a softmax over the chosen
    logits (``softmax_of_chosen``) or each chosen logit's sigmoid as it is (``sigmoid``)."""
    T = logits.shape[0]
    if scoring not in MOE_SCORING or logits.dim() != 2 or logits.shape[1] < experts or logits.stride(1) != 1:
        raise lib.KernelError("moe_topk: shapes do not fit")
    idx = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    tw = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    dense = torch.empty((T, experts), dtype=torch.float32, device=logits.device)
    lib.call("tm_moe_topk", _req(logits, "logits", torch.float32), None, idx.data_ptr(), tw.data_ptr(), dense.data_ptr(), T,
             int(experts), int(top), logits.stride(0), MOE_SCORING[scoring], _stream())
    return idx, tw, dense


def glu_routed_in(gu: torch.Tensor, dense_w: torch.Tensor, act: torch.Tensor, E: int, F: int, shared: int = 0,
                  shared_logit: torch.Tensor | None = None) -> torch.Tensor:
    """Experts whose weight multiplies their input. gu [T, E * 2 F + 2 shared] (per expert gate rows then up rows, then the
    shared expert's) -> act [T, E F + shared] = silu(w gate) * (w up) for the chosen experts, zero for the others, and
    silu(gate) * up * sigmoid(shared_logit) for the shared expert; shared_logit [T] float32 (may be strided) or None."""
    T = gu.shape[0]
    if gu.shape[1] != E * 2 * F + 2 * shared or act.shape != (T, E * F + shared) or dense_w.shape != (T, E) or \
            (shared_logit is not None and (shared_logit.dim() != 1 or shared_logit.numel() != T or
                                           shared_logit.dtype != torch.float32)):
        raise lib.KernelError("glu_routed_in: shapes do not fit")
    lib.call("tm_glu_routed_in", _code(gu.dtype), _req(gu, "gu"), _req(dense_w, "dense_w", torch.float32),
             _req(act, "act", gu.dtype), T, E, F, int(shared), shared_logit.data_ptr() if shared_logit is not None else None,
             shared_logit.stride(0) if shared_logit is not None else 0, _stream())
    return act


def glu_routed(gu: torch.Tensor, dense_w: torch.Tensor, act: torch.Tensor, E: int, F: int) -> torch.Tensor:
    """gu [T, E * 2 * F] (per expert gate rows then up rows) -> act [T, E * F] = silu(gate) * up * weight."""
    T = gu.shape[0]
    if gu.shape[1] != E * 2 * F or act.shape != (T, E * F) or dense_w.shape != (T, E):
        raise lib.KernelError("glu_routed: shapes do not fit")
    lib.call("tm_glu_routed", _code(gu.dtype), _req(gu, "gu"), _req(dense_w, "dense_w", torch.float32),
             _req(act, "act", gu.dtype), T, E, F, _stream())
    return act


def router_logits(x: torch.Tensor, w: torch.Tensor, w_low: torch.Tensor | None = None) -> torch.Tensor:
    """x [T, H] . w [n, H]^T in 32-bit: this library's 32-bit product for float32 inputs; for bfloat16 inputs the library's
    product of x with ``w_low``, a bfloat16 copy of w that holds the same values, with its 32-bit accumulator as the result
    (products of two bfloat16 numbers are exact in 32-bit), or x converted and the 32-bit product when there is no such copy."""
    if x.dtype == torch.float32:
        return linear(x, w)
    if w_low is not None:
        return torch.mm(x, w_low.t(), out_dtype=torch.float32)
    return linear(x.float(), w)


def moe_choose(logits: torch.Tensor, correction: torch.Tensor | None, top: int, groups: int = 1, keep: int = 1,
               identity: int = 0):
    """logits [T, n] float32 over experts and identity outputs -> (top_idx [T, top] int32, top_w [T, top], dense_w [T, n],
    identity_w [T] float32). Scores are a softmax over all n; the choice is by score + correction, restricted to the best
    ``keep`` of ``groups`` equal groups of neighbours; weights are the chosen scores over their sum; identity_w sums the
    weights of chosen outputs among the last ``identity``."""
    T, n = logits.shape
    dev = logits.device
    idx = torch.empty((T, top), dtype=torch.int32, device=dev)
    tw = torch.empty((T, top), dtype=torch.float32, device=dev)
    dense = torch.empty((T, n), dtype=torch.float32, device=dev)
    idw = torch.empty((T,), dtype=torch.float32, device=dev)
    if correction is not None and correction.numel() != n:
        raise lib.KernelError("moe_choose: the correction has one number per router output")
    lib.call("tm_moe_choose", _req(logits, "logits", torch.float32), _opt(correction, "correction", torch.float32),
             idx.data_ptr(), tw.data_ptr(), dense.data_ptr(), idw.data_ptr(), T, n, int(top), int(groups), int(keep),
             int(identity), _stream())
    return idx, tw, dense, idw


def act_routed(up: torch.Tensor, dense_w: torch.Tensor, act: torch.Tensor, E: int, F: int) -> torch.Tensor:
    """up [T, E * F] -> act [T, E * F] = relu(up)^2 * weight of the expert (dense_w [T, >= E] float32), zero where not chosen."""
    T = up.shape[0]
    if up.shape[1] != E * F or act.shape != (T, E * F) or dense_w.shape[0] != T or dense_w.shape[1] < E:
        raise lib.KernelError("act_routed: shapes do not fit")
    lib.call("tm_act_routed", _code(up.dtype), _req(up, "up"), _req(dense_w, "dense_w", torch.float32), dense_w.shape[1],
             _req(act, "act", up.dtype), T, E, F, _stream())
    return act


def add_scaled_rows(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """out[t] += w[t] * x[t]; out and x [T, H] in the same dtype, w [T] float32."""
    if out.shape != x.shape or out.dtype != x.dtype or w.numel() != out.shape[0]:
        raise lib.KernelError("add_scaled_rows: shapes do not fit")
    lib.call("tm_add_scaled_rows", _code(out.dtype), _req(out, "out"), _req(x, "x"), _req(w, "w", torch.float32), out.shape[0],
             out.shape[1], _stream())
    return out


# --- gated convolutional blocks, windowed attention with a sink, matrix memory --------------------------------

GLU_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


def linear32(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [T, K] . w [N, K]^T with the 32-bit accumulator kept as the result ([T, N] float32) in both run dtypes."""
    return linear(x, w, out_dtype=torch.float32)


def gated_add_rmsnorm(resid: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, *,
                      branch: torch.Tensor | None = None, gate: torch.Tensor | None = None,
                      gate_bias: torch.Tensor | None = None, ids: torch.Tensor | None = None,
                      table: torch.Tensor | None = None, table_scale: float = 1.0,
                      rows: torch.Tensor | None = None) -> torch.Tensor:
    """resid [T, H] float32 += sigmoid(gate + gate_bias) * branch (or = table[ids] * table_scale); out = rmsnorm(resid) * w.
    gate [T, H] float32 (rows may be strided) holds the gate's pre-activations. With ``rows`` only those rows are normed."""
    H = resid.shape[-1]
    n_rows = rows.numel() if rows is not None else resid.shape[0]
    if out.shape[0] < n_rows or out.shape[-1] != H or weight.numel() != H or (ids is None) != (table is None):
        raise lib.KernelError("gated_add_rmsnorm: shapes do not fit")
    if gate is not None and (branch is None or gate.dtype != torch.float32 or gate.stride(-1) != 1 or gate.shape[-1] != H):
        raise lib.KernelError("gated_add_rmsnorm: the gate is a float32 [T, H] beside a branch")
    dt = out.dtype
    lib.call("tm_gated_add_rmsnorm", _code(dt), _req(resid, "resid", torch.float32), _opt(branch, "branch", dt),
             gate.data_ptr() if gate is not None else None, gate.stride(0) if gate is not None else 0,
             _opt(gate_bias, "gate_bias", torch.float32), _opt(ids, "ids", torch.int32), _opt(table, "table", dt),
             float(table_scale), _opt(rows, "rows", torch.int32), _req(weight, "weight", torch.float32), float(eps),
             _req(out, "out"), n_rows, H, _stream())
    return out


def canon_conv(h: torch.Tensor, weight: torch.Tensor, state: torch.Tensor, cu_q: torch.Tensor, seq_of_token: torch.Tensor,
               state_slots: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] = h[t] + sum_j weight[:, j] h[t - taps + 1 + j]; weight [C, taps] float32; ``state`` [slots, (taps - 1) * C]
    float32 (a view whose rows may be strided) carries each request's last taps - 1 inputs from step to step."""
    T, C = h.shape
    taps = weight.shape[1]
    if weight.shape[0] != C or out.shape != h.shape or state.shape[1] < (taps - 1) * C or state.stride(1) != 1:
        raise lib.KernelError("canon_conv: shapes do not fit")
    lib.call("tm_canon_conv", _code(h.dtype), _req(h, "h"), _req(weight, "weight", torch.float32), state.data_ptr(),
             state.stride(0), _req(cu_q, "cu_q", torch.int32), _req(seq_of_token, "seq_of_token", torch.int32),
             _req(state_slots, "state_slots", torch.int32), _req(out, "out", h.dtype), T, C, taps, _stream())
    return out


def glu(gu: torch.Tensor, out: torch.Tensor, activation: str) -> torch.Tensor:
    """gu [T, 2 I] (gate columns first) -> out [T, I] = act(gate) * up, act in GLU_ACTIVATIONS."""
    T, two_i = gu.shape
    if two_i % 2 or out.shape != (T, two_i // 2) or activation not in GLU_ACTIVATIONS:
        raise lib.KernelError(f"glu: gu {tuple(gu.shape)}, out {tuple(out.shape)}, activation {activation!r} do not fit")
    lib.call("tm_glu", _code(gu.dtype), GLU_ACTIVATIONS[activation], _req(gu, "gu"), _req(out, "out", gu.dtype), T,
             two_i // 2, _stream())
    return out


def norm_pair_mean(a: torch.Tensor, b: torch.Tensor, wa: torch.Tensor, wb: torch.Tensor, eps: float,
                   out: torch.Tensor) -> torch.Tensor:
    """out = (rmsnorm(a) * wa + rmsnorm(b) * wb) / 2, row by row."""
    T, H = a.shape
    if b.shape != a.shape or out.shape != a.shape or wa.numel() != H or wb.numel() != H:
        raise lib.KernelError("norm_pair_mean: shapes do not fit")
    lib.call("tm_norm_pair_mean", _code(a.dtype), _req(a, "a"), _req(b, "b", a.dtype), _req(wa, "wa", torch.float32),
             _req(wb, "wb", torch.float32), float(eps), _req(out, "out", a.dtype), T, H, _stream())
    return out


def weighted_pair(a: torch.Tensor, b: torch.Tensor, sa: float, sb: float, out: torch.Tensor) -> torch.Tensor:
    """out = sa * a + sb * b, elementwise (32-bit arithmetic, one rounding)."""
    if b.shape != a.shape or out.shape != a.shape or b.dtype != a.dtype:
        raise lib.KernelError("weighted_pair: shapes do not fit")
    lib.call("tm_weighted_pair", _code(a.dtype), _req(a, "a"), _req(b, "b"), float(sa), float(sb), _req(out, "out", a.dtype),
             a.numel(), _stream())
    return out


HEAD_GATES = {"sigmoid": 0, "silu": 1}


def head_norm_gate(y: torch.Tensor, gate: torch.Tensor | None, weight: torch.Tensor, eps: float, heads: int,
                   out: torch.Tensor, den: torch.Tensor | None = None, gate_act: str = "sigmoid") -> torch.Tensor:
    """y [T, heads * dv] float32 (divided by den [T, heads] first, where given): each head by its own root mean square,
    times weight [heads * dv], times sigmoid(gate) or silu(gate) (``gate_act``); gate [T, heads * dv] float32
    pre-activations (rows may be strided), or None for no gate. out [T, heads * dv] may be columns of a wider matrix."""
    T, inner = y.shape
    if inner % heads or weight.numel() != inner or out.shape != y.shape or (den is not None and den.shape != (T, heads)) or \
            gate_act not in HEAD_GATES or out.stride(1) != 1 or not out.is_cuda or \
            (gate is not None and (gate.shape != y.shape or gate.stride(1) != 1 or gate.dtype != torch.float32)):
        raise lib.KernelError("head_norm_gate: shapes do not fit")
    lib.call("tm_head_norm_gate", _code(out.dtype), _req(y, "y", torch.float32), _opt(den, "den", torch.float32),
             gate.data_ptr() if gate is not None else None, gate.stride(0) if gate is not None else 0, HEAD_GATES[gate_act],
             _req(weight, "weight", torch.float32), float(eps), out.data_ptr(), out.stride(0), T, heads, inner // heads, _stream())
    return out


def qk_norm_rope_write(proj: torch.Tensor, *, heads: int, kv_heads: int, dim: int, vdim: int, rot_dims: int,
                       wq: torch.Tensor | None, wk: torch.Tensor | None, eps: float, positions: torch.Tensor,
                       cos: torch.Tensor, sin: torch.Tensor, slot_map: torch.Tensor | None, q_out: torch.Tensor,
                       cache: torch.Tensor | None, gate_out: torch.Tensor | None, has_kv: bool = True,
                       q_temp: tuple[float, int] | None = None, head_norm: bool = False) -> None:
    """proj [T, >= H d + G d + G dv (+ gate columns)] float32 (rows may be strided) -> q_out [T, H d] normed and rotated,
    the token's cache row [k | v], gate_out [T, H] or [T, H dv] = sigmoid of the last columns. ``has_kv`` False: the row
    is [q | g] only (a layer that reads another layer's keys and values). ``q_temp`` (coef, every): the query is
    multiplied by 1 + coef ln(floor((p + 1) / every) + 1) at position p. ``head_norm``: every head of q and of k is divided
    by its own root mean square (wq and wk then optional) instead of the whole projections by theirs."""
    T = proj.shape[0]
    gate_cols = gate_out.shape[1] if gate_out is not None else 0
    need = heads * dim + (kv_heads * (dim + vdim) if has_kv else 0) + gate_cols
    if gate_cols not in (0, heads, heads * vdim) or (not has_kv and (cache is not None or wk is not None)):
        raise lib.KernelError("qk_norm_rope_write: the gate has one column per head or per output number; a row without "
                              "keys writes no cache")
    coef, every = (float(q_temp[0]), int(q_temp[1])) if q_temp else (0.0, 0)
    if proj.dtype != torch.float32 or proj.stride(1) != 1 or proj.shape[1] < need or q_out.shape != (T, heads * dim) or \
            cos.shape[1] * 2 != rot_dims or (cache is not None and cache.shape[-1] != kv_heads * (dim + vdim)):
        raise lib.KernelError("qk_norm_rope_write: shapes do not fit")
    dt = q_out.dtype
    lib.call("tm_qk_norm_rope_write", _code(dt), proj.data_ptr(), proj.stride(0), heads, kv_heads, dim, vdim, rot_dims,
             _opt(wq, "wq", torch.float32), _opt(wk, "wk", torch.float32), float(eps),
             _req(positions, "positions", torch.int32), _req(cos, "cos", torch.float32), _req(sin, "sin", torch.float32),
             cos.shape[0], _opt(slot_map, "slot_map", torch.int32) if cache is not None else None, _req(q_out, "q_out"),
             _opt(cache, "cache", dt), _opt(gate_out, "gate_out", torch.float32), gate_cols, int(bool(has_kv)), coef, every,
             int(bool(head_norm)), T, _tc_flag(proj.device).data_ptr(), _stream())


SINK_TILE_ROWS = 32
SINK_TC_TILE_ROWS = 64


def sink_attention_tc_ok(dtype: torch.dtype, dim: int, vdim: int) -> bool:
    """Whether the tensor-core kernel takes these shapes (bfloat16, key and value heads of 32, 64 or 128 each)."""
    return dtype == torch.bfloat16 and dim in (32, 64, 128) and vdim in (32, 64, 128) and \
        os.environ.get("TOKENMILL_SINK_TC", "1") != "0"


def sink_attention(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, cu_q: torch.Tensor,
                   kv_before: torch.Tensor, tile_seq: torch.Tensor, tile_row0: torch.Tensor, n_tiles: int,
                   gate: torch.Tensor | None, out: torch.Tensor, *, heads: int, kv_heads: int, dim: int, vdim: int,
                   scale: float, softcap: float, window: int, keep_first: int, sink: bool,
                   tensor_cores: bool = False, n_splits: int = 1, part: torch.Tensor | None = None,
                   cross_out: torch.Tensor | None = None) -> torch.Tensor:
    """q [T, H d]; cache [pages, page_size, 1, G d + G dv]; tiles of 32 (``tensor_cores``: 64) (token, head in group)
    rows of one request; gate [T, H] (or [T, H dv]: one per output number) float32 or None; out [T, H dv]. ``n_splits`` > 1 (tensor cores only): a tile's
    key blocks dealt out over that many blocks and merged, through ``part``, float32 scratch of
    n_tiles * G * n_splits * 64 * (dv + 2) numbers. ``cross_out`` [T, H * G * dv] float32 (then ``out`` may be None and
    there is no gate; the scratch has G times the numbers): every head's softmax weights applied to the values of each of
    the G value heads, [T, H, G, dv], for a mixer that mixes the heads' weights afterwards."""
    T = q.shape[0]
    row = kv_heads * (dim + vdim)
    if cache.shape[-1] != row or q.shape != (T, heads * dim) or \
            (cross_out is None and out.shape != (T, heads * vdim)) or \
            (cross_out is not None and (cross_out.shape != (T, heads * kv_heads * vdim) or cross_out.dtype != torch.float32
                                        or gate is not None)) or \
            (gate is not None and tuple(gate.shape) not in ((T, heads), (T, heads * vdim))):
        raise lib.KernelError("sink_attention: shapes do not fit")
    wide = int(gate is not None and gate.shape[1] != heads)
    cross = _opt(cross_out, "cross_out", torch.float32)
    out_ptr = _req(out, "out", q.dtype) if out is not None else None
    if tensor_cores:
        part_o = part_ml = None
        if n_splits > 1:
            rows64 = int(n_tiles) * kv_heads * (kv_heads if cross_out is not None else 1) * int(n_splits) * SINK_TC_TILE_ROWS
            if part is None or part.dtype != torch.float32 or part.numel() < rows64 * (vdim + 2):
                raise lib.KernelError("sink_attention: scratch for the key splits is missing or too small")
            part_o, part_ml = part.data_ptr(), part.data_ptr() + rows64 * vdim * 4
        lib.call("tm_sink_attention_mma_bf16", _req(q, "q", torch.bfloat16), _req(cache, "cache", torch.bfloat16), row,
                 kv_heads * dim, _req(block_table, "block_table", torch.int32), block_table.stride(0),
                 _req(cu_q, "cu_q", torch.int32), _req(kv_before, "kv_before", torch.int32),
                 _req(tile_seq, "tile_seq", torch.int32), _req(tile_row0, "tile_row0", torch.int32), int(n_tiles),
                 _opt(gate, "gate", torch.float32), out_ptr, heads, kv_heads, dim, vdim,
                 cache.shape[1], float(scale), float(softcap), int(window), int(keep_first), int(bool(sink)),
                 int(n_splits), part_o, part_ml, wide, cross, _stream())
        return out if cross_out is None else cross_out
    lib.call("tm_sink_attention", _code(q.dtype), _req(q, "q"), _req(cache, "cache", q.dtype), row, kv_heads * dim,
             _req(block_table, "block_table", torch.int32), block_table.stride(0), _req(cu_q, "cu_q", torch.int32),
             _req(kv_before, "kv_before", torch.int32), _req(tile_seq, "tile_seq", torch.int32),
             _req(tile_row0, "tile_row0", torch.int32), int(n_tiles), _opt(gate, "gate", torch.float32),
             out_ptr, heads, kv_heads, dim, vdim, cache.shape[1], float(scale), float(softcap),
             int(window), int(keep_first), int(bool(sink)), wide, cross, _stream())
    return out if cross_out is None else cross_out


MEMORY_THREADS = 256


def matrix_memory_geometry(dim: int, vdim: int) -> tuple[int, int, int]:
    """(d_pad, columns per block, column tiles) of the matrix-memory kernel for heads of dim x vdim (+ 1 column): a column's
    state is spread over ``parts`` lanes of 8, 16 or 32 rows each (csrc/matrix_memory.cu)."""
    R = 8 if dim <= 256 else 16 if dim <= 512 else 32
    parts = 1
    while parts * R < dim:
        parts *= 2
    cols = MEMORY_THREADS // parts
    return parts * R, cols, -(-(vdim + 1) // cols)


def matrix_memory_state_floats(heads: int, dim: int, vdim: int) -> int:
    """Floats of a request's memory: S with n as one more column, [heads][vdim + 1][d_pad], and four per block."""
    d_pad, _cols, tiles = matrix_memory_geometry(dim, vdim)
    return heads * (vdim + 1) * d_pad + heads * tiles * 4


def matrix_memory(proj: torch.Tensor, *, q_col: int, k_col: int, v_col: int, i_col: int, f_col: int,
                  i_bias: torch.Tensor | None, f_bias: torch.Tensor | None, cap: float, q_scale: float,
                  state: torch.Tensor, state_off: int, cu_q: torch.Tensor, state_slots: torch.Tensor, y: torch.Tensor,
                  den: torch.Tensor, n_seqs: int, heads: int, dim: int, vdim: int, slice_len: int = 0,
                  slices: torch.Tensor | None = None) -> torch.Tensor:
    """The recurrence over this step's tokens. proj [T, P] float32 (rows may be strided) holds q, k (heads x dim), v
    (heads x vdim) and the raw gates (heads each) at the named columns; y [T, heads * vdim] float32 receives S^T q and
    den [T, heads] float32 what each head's y is still to be divided by (``head_norm_gate`` does); a request's memory
    lives at ``state_off`` inside its slot of ``state`` [slots, n] float32. ``slice_len`` > 0: three passes over time
    slices of that many tokens (for long prompt portions), through ``slices``, float32 scratch for
    ``matrix_memory_slice_records(T, n_seqs, slice_len)`` records of ``matrix_memory_state_floats`` floats."""
    T = proj.shape[0]
    floats = matrix_memory_state_floats(heads, dim, vdim)
    if proj.dtype != torch.float32 or proj.stride(1) != 1 or y.shape != (T, heads * vdim) or dim > 1024 or \
            den.shape != (T, heads) or state.shape[1] < state_off + floats or state.stride(1) != 1:
        raise lib.KernelError("matrix_memory: shapes do not fit")
    records = matrix_memory_slice_records(T, n_seqs, slice_len) if slice_len > 0 else 0
    if slice_len > 0 and (slices is None or slices.numel() < records * floats):
        raise lib.KernelError("matrix_memory: scratch for the time slices is missing or too small")

    def walk(mode):
        lib.call("tm_matrix_memory", proj.data_ptr(), proj.stride(0), q_col, k_col, v_col, i_col, f_col,
                 _opt(i_bias, "i_bias", torch.float32), _opt(f_bias, "f_bias", torch.float32), float(cap), float(q_scale),
                 _req(state, "state", torch.float32), state.stride(0), int(state_off), _req(cu_q, "cu_q", torch.int32),
                 _req(state_slots, "state_slots", torch.int32), _req(y, "y", torch.float32), _req(den, "den", torch.float32),
                 int(n_seqs), heads, dim, vdim, mode, int(slice_len), _opt(slices, "slices", torch.float32), floats, records, _stream())

    if slice_len <= 0:
        walk(0)
        return y
    walk(1)
    lib.call("tm_matrix_memory_pass_states", state.data_ptr(), state.stride(0), int(state_off), cu_q.data_ptr(),
             state_slots.data_ptr(), int(n_seqs), heads, dim, vdim, int(slice_len), slices.data_ptr(), floats, _stream())
    walk(2)
    return y


def matrix_memory_slice_records(n_tokens: int, n_seqs: int, slice_len: int) -> int:
    """Slice records a step needs: request s owns records cu_q[s] // slice_len + s onwards."""
    return n_tokens // slice_len + n_seqs


# --- several residual streams behind a norm, selective scan, linear attention with a decay --------------------

STREAM_NORMS = {"dyt": 0, "rms": 1}
MAX_STREAMS = 8


def stream_norm(resid: torch.Tensor, streams: int, out: torch.Tensor, *, kind: str, weight: torch.Tensor,
                bias: torch.Tensor | None = None, alpha: torch.Tensor | None = None, eps: float = 0.0,
                ids: torch.Tensor | None = None, table: torch.Tensor | None = None, positions: torch.Tensor | None = None,
                pos_table: torch.Tensor | None = None, branch: torch.Tensor | None = None, branch2: torch.Tensor | None = None,
                row_scale: torch.Tensor | None = None, mix: torch.Tensor | None = None, out_w: torch.Tensor | None = None,
                in_w: torch.Tensor | None = None, rows: torch.Tensor | None = None, table_scale: float = 1.0) -> torch.Tensor:
    """resid [T, streams * H] float32: the streams of every token side by side. Starts them all as table[ids] * table_scale (+
    pos_table[positions]), or takes in y = branch + row_scale * branch2: x_t <- sum_s mix[s, t] x_s + out_w[t] y (no mix:
    x_t <- x_t + y); reads u = sum_s in_w[s] x_s (no in_w: the sum) and writes out = norm(u): ``dyt`` tanh(alpha u) w + b, or
    ``rms``. With ``rows`` only those rows are normed and the residual stays as it is."""
    H = out.shape[-1]
    n_rows = rows.numel() if rows is not None else resid.shape[0]
    if kind not in STREAM_NORMS or resid.shape[-1] != streams * H or out.shape[0] < n_rows or weight.numel() != H or \
            (ids is None) != (table is None) or (pos_table is None) != (positions is None and pos_table is None) or \
            (kind == "dyt" and (alpha is None or alpha.numel() != 1)) or not 1 <= streams <= MAX_STREAMS:
        raise lib.KernelError("stream_norm: shapes do not fit")
    if (mix is not None and mix.numel() != streams * streams) or (out_w is not None and out_w.numel() != streams) or \
            (in_w is not None and in_w.numel() != streams) or (mix is None and streams > 1 and (branch is not None or branch2 is not None)):
        raise lib.KernelError("stream_norm: mix is [streams, streams], out_w and in_w [streams]; several streams need a mix")
    dt = out.dtype
    lib.call("tm_stream_norm", _code(dt), _req(resid, "resid", torch.float32), int(streams), H, _opt(ids, "ids", torch.int32),
             _opt(table, "table", dt), _opt(positions, "positions", torch.int32) if pos_table is not None else None,
             _opt(pos_table, "pos_table", dt), _opt(branch, "branch", dt), _opt(branch2, "branch2", dt),
             row_scale.data_ptr() if row_scale is not None else None, row_scale.stride(0) if row_scale is not None else 0,
             _opt(mix, "mix", torch.float32), _opt(out_w, "out_w", torch.float32), _opt(in_w, "in_w", torch.float32),
             _opt(rows, "rows", torch.int32), STREAM_NORMS[kind], _opt(alpha, "alpha", torch.float32),
             _req(weight, "weight", torch.float32), _opt(bias, "bias", torch.float32), float(eps), _req(out, "out"), n_rows,
             float(table_scale), _stream())
    return out


def softcap_(x: torch.Tensor, cap: float, scale: float = 1.0) -> torch.Tensor:
    """x <- cap * tanh(scale x / cap), in place (float32); cap 0: x <- scale x."""
    lib.call("tm_softcap", _req(x, "x", torch.float32), x.numel(), float(cap), float(scale), _stream())
    return x


def selective_scan(x: torch.Tensor, z: torch.Tensor, z_col: int, dbc: torch.Tensor, w_dt: torch.Tensor, b_dt: torch.Tensor,
                   A_log: torch.Tensor, D: torch.Tensor, state: torch.Tensor, state_off: int, cu_q: torch.Tensor,
                   state_slots: torch.Tensor, out: torch.Tensor, *, n_seqs: int, rank: int, N: int, max_q_len: int = 0,
                   slice_len: int = 0, slice_S: torch.Tensor | None = None, slice_dt: torch.Tensor | None = None) -> torch.Tensor:
    """x [T, inner] (convolved, activated); z: the gate's pre-activations at columns z_col .. z_col + inner of a matrix in x's
    dtype; dbc [T, rank + 2 N] float32 = [low | B | C]; w_dt [inner, rank], b_dt [inner], A_log [inner, N], D [inner] float32;
    a request's states [inner, N] live ``state_off`` floats into its slot. out [T, inner] = (scan + D x) silu(z).
    ``slice_len`` > 0: three passes over time slices of that many tokens (for long prompt portions), through ``slice_S``
    (n_seqs * slices * inner * N float32) and ``slice_dt`` (n_seqs * slices * inner float32), slices =
    ceil(max_q_len / slice_len)."""
    T, inner = x.shape
    if out.shape != x.shape or dbc.shape != (T, rank + 2 * N) or z.shape[0] != T or z_col + inner > z.shape[1] or \
            tuple(w_dt.shape) != (inner, rank) or tuple(A_log.shape) != (inner, N) or b_dt.numel() != inner or D.numel() != inner or \
            state.shape[1] < state_off + inner * N or z.dtype != x.dtype or z.stride(1) != 1:
        raise lib.KernelError("selective_scan: shapes do not fit")

    def scan(mode, max_slices):
        lib.call("tm_selective_scan", _code(x.dtype), _req(x, "x"), inner, z.data_ptr(), z.stride(0), int(z_col),
                 _req(dbc, "dbc", torch.float32), dbc.stride(0), int(rank), int(N), _req(w_dt, "w_dt", torch.float32),
                 _req(b_dt, "b_dt", torch.float32), _req(A_log, "A_log", torch.float32), _req(D, "D", torch.float32),
                 _req(state, "state", torch.float32), state.stride(0), int(state_off), _req(cu_q, "cu_q", torch.int32),
                 _req(state_slots, "state_slots", torch.int32), _req(out, "out", x.dtype), int(n_seqs), mode, int(slice_len),
                 max_slices, _opt(slice_S, "slice_S", torch.float32), _opt(slice_dt, "slice_dt", torch.float32), _stream())

    if slice_len <= 0:
        scan(0, 1)
        return out
    slices = -(-int(max_q_len) // int(slice_len))
    if slices < 1 or slice_S is None or slice_dt is None or slice_S.numel() < n_seqs * slices * inner * N or \
            slice_dt.numel() < n_seqs * slices * inner:
        raise lib.KernelError("selective_scan: scratch for the time slices is missing or too small")
    scan(1, slices)
    lib.call("tm_selective_pass_states", _code(x.dtype), state.data_ptr(), state.stride(0), int(state_off), cu_q.data_ptr(),
             state_slots.data_ptr(), A_log.data_ptr(), slice_S.data_ptr(), slice_dt.data_ptr(), int(n_seqs), inner, int(N),
             int(slice_len), slices, _stream())
    scan(2, slices)
    return out


DECAY_ACTIVATIONS = {None: 0, "none": 0, "silu": 1}


def decay_memory_state_floats(heads: int, dim: int, vdim: int) -> int:
    """Floats of a request's memories as the kernel lays them out: [heads][vdim][d_pad], a column's rows side by side, 16
    rows on each of the power-of-two lanes that share a column (csrc/decay_memory.cu)."""
    parts = 1
    while parts * 16 < dim:
        parts *= 2
    return heads * vdim * parts * 16


def decay_memory(proj: torch.Tensor, *, q_col: int, k_col: int, v_col: int, activation: str | None, decay: torch.Tensor,
                 state: torch.Tensor, state_off: int, cu_q: torch.Tensor, state_slots: torch.Tensor, y: torch.Tensor,
                 n_seqs: int, heads: int, dim: int, vdim: int, max_q_len: int = 0, slice_len: int = 0,
                 slice_S: torch.Tensor | None = None) -> torch.Tensor:
    """proj [T, P] float32 (rows may be strided) with q, k (heads x dim) and v (heads x vdim) at the given columns, each
    through ``activation``; per head S <- decay S + k v^T, y = S^T q; a request's memories
    (``decay_memory_state_floats`` floats) live ``state_off`` floats into its slot; y [T, heads * vdim] float32.
    ``slice_len`` > 0: three passes over time slices of that many tokens (for long prompt portions), through ``slice_S``
    (n_seqs * slices memories, float32), slices = ceil(max_q_len / slice_len); this run applies the activation to the q,
    k and v columns of ``proj`` in place first."""
    T = proj.shape[0]
    if dim > 512:
        raise lib.KernelError("decay_memory: memories of up to 512 rows per head are built")
    floats = decay_memory_state_floats(heads, dim, vdim)
    if proj.dtype != torch.float32 or proj.stride(1) != 1 or y.shape != (T, heads * vdim) or decay.numel() != heads or \
            max(q_col, k_col) + heads * dim > proj.shape[1] or v_col + heads * vdim > proj.shape[1] or \
            state.shape[1] < state_off + floats or state.stride(1) != 1 or activation not in DECAY_ACTIVATIONS:
        raise lib.KernelError("decay_memory: shapes do not fit")
    act = DECAY_ACTIVATIONS[activation]

    def walk(mode, max_slices, act):
        lib.call("tm_decay_memory", proj.data_ptr(), proj.stride(0), int(q_col), int(k_col), int(v_col), act,
                 _req(decay, "decay", torch.float32), _req(state, "state", torch.float32),
                 state.stride(0), int(state_off), _req(cu_q, "cu_q", torch.int32), _req(state_slots, "state_slots", torch.int32),
                 _req(y, "y", torch.float32), int(n_seqs), heads, dim, vdim, mode, int(slice_len), max_slices,
                 _opt(slice_S, "slice_S", torch.float32), _stream())

    if slice_len <= 0:
        walk(0, 1, act)
        return y
    slices = -(-int(max_q_len) // int(slice_len))
    if slices < 1 or slice_S is None or slice_S.numel() < n_seqs * slices * floats:
        raise lib.KernelError("decay_memory: scratch for the time slices is missing or too small")
    if act:
        lib.call("tm_decay_activate", proj.data_ptr(), proj.stride(0), T, int(q_col), int(k_col), int(v_col), heads, dim, vdim,
                 act, _stream())
    walk(1, slices, 0)
    lib.call("tm_decay_pass_states", state.data_ptr(), state.stride(0), int(state_off), cu_q.data_ptr(), state_slots.data_ptr(),
             decay.data_ptr(), slice_S.data_ptr(), int(n_seqs), heads, dim, vdim, int(slice_len), slices, _stream())
    walk(2, slices, 0)
    return y


# --- matrix memories with a decay per token, the delta rule, short convolutions with carried inputs ---------------


def gated_memory_state_floats(heads: int, dim: int, vdim: int) -> int:
    """Floats of a request's memories as the kernel lays them out: [heads][vdim][d_pad], a column's rows side by side, 16
    rows on each of the power-of-two lanes that share a column (csrc/gated_memory.cu)."""
    parts = 1
    while parts * 16 < dim:
        parts *= 2
    return heads * vdim * parts * 16


def gated_memory_slice_floats(heads: int, dim: int, vdim: int, delta: bool) -> int:
    """Floats of one time slice's record in scratch: its own memory and what it does to the memory it starts from (one
    more column, or ``dim`` more with the delta rule)."""
    return gated_memory_state_floats(heads, dim, vdim + (dim if delta else 1))


def gated_memory(proj: torch.Tensor, *, q_col: int, k_col: int, v_col: int, gb: torch.Tensor | None, rule: str,
                 state: torch.Tensor, state_off: int, cu_q: torch.Tensor, state_slots: torch.Tensor, y: torch.Tensor,
                 n_seqs: int, heads: int, qk_heads: int, dim: int, vdim: int, max_q_len: int = 0, slice_len: int = 0,
                 slice_S: torch.Tensor | None = None) -> torch.Tensor:
    """proj [T, P] float32 (rows may be strided) with q and k (qk_heads x dim) and v (heads x vdim) at the given columns;
    head h reads q/k head h // (heads // qk_heads). ``rule``: "delta": S <- g S, u = beta (v - S^T k), S <- S + k u^T with
    (g, beta) = gb [T, 2 heads] float32; "forget": the columns at k_col hold f, S <- diag(f) S + (1 - f) v^T, gb unused;
    "decay": S <- g S + k v^T. y [T, heads * vdim] float32 = S^T q after the write. A request's memories
    (``gated_memory_state_floats`` floats) live ``state_off`` floats into its slot. ``slice_len`` > 0: three passes over
    time slices of that many tokens (for long prompt portions) through ``slice_S`` (n_seqs * slices records of
    ``gated_memory_slice_floats`` floats), slices = ceil(max_q_len / slice_len)."""
    T = proj.shape[0]
    if rule not in ("delta", "forget", "decay") or dim > 512:
        raise lib.KernelError("gated_memory: rules delta, forget and decay over memories of up to 512 rows are built")
    row_decay, delta = int(rule == "forget"), int(rule == "delta")
    floats = gated_memory_state_floats(heads, dim, vdim)
    if proj.dtype != torch.float32 or proj.stride(1) != 1 or y.shape != (T, heads * vdim) or heads % qk_heads or \
            max(q_col, k_col) + qk_heads * dim > proj.shape[1] or v_col + heads * vdim > proj.shape[1] or \
            state.shape[1] < state_off + floats or state.stride(1) != 1 or \
            (not row_decay and (gb is None or gb.shape != (T, 2 * heads))):
        raise lib.KernelError("gated_memory: shapes do not fit")

    def walk(mode, max_slices):
        lib.call("tm_gated_memory", proj.data_ptr(), proj.stride(0), int(q_col), int(k_col), int(v_col),
                 _opt(gb, "gb", torch.float32) if not row_decay else None, row_decay, delta,
                 _req(state, "state", torch.float32), state.stride(0), int(state_off), _req(cu_q, "cu_q", torch.int32),
                 _req(state_slots, "state_slots", torch.int32), _req(y, "y", torch.float32), int(n_seqs), heads, qk_heads, dim,
                 vdim, mode, int(slice_len), max_slices, _opt(slice_S, "slice_S", torch.float32), _stream())

    if slice_len <= 0:
        walk(0, 1)
        return y
    slices = -(-int(max_q_len) // int(slice_len))
    if slices < 1 or slice_S is None or slice_S.numel() < n_seqs * slices * gated_memory_slice_floats(heads, dim, vdim, bool(delta)):
        raise lib.KernelError("gated_memory: scratch for the time slices is missing or too small")
    walk(1, slices)
    lib.call("tm_gated_memory_pass_states", state.data_ptr(), state.stride(0), int(state_off), cu_q.data_ptr(),
             state_slots.data_ptr(), slice_S.data_ptr(), delta, int(n_seqs), heads, dim, vdim, int(slice_len), slices, _stream())
    walk(2, slices)
    return y


def short_conv_state(proj: torch.Tensor, col0: int, weight: torch.Tensor, bias: torch.Tensor | None, state: torch.Tensor,
                     state_off: int, cu_q: torch.Tensor, seq_of_token: torch.Tensor, state_slots: torch.Tensor,
                     out: torch.Tensor, out_col0: int = 0, activation: str | None = None) -> torch.Tensor:
    """A causal convolution over time on ``channels`` columns of proj [T, P] float32 from column col0 (rows may be
    strided): out[t, out_col0 + c] = act(sum_j weight[c, j] u[t - taps + 1 + j, c]) with u = proj + bias and act silu or
    none; weight [channels, taps] float32. A request's last taps - 1 inputs (bias included) are carried ``state_off`` floats
    into its slot, [taps - 1, channels]; zeros for a new request. out float32 [T, >= out_col0 + channels]."""
    T = proj.shape[0]
    channels, taps = weight.shape
    if proj.dtype != torch.float32 or proj.stride(1) != 1 or col0 + channels > proj.shape[1] or out.dtype != torch.float32 or \
            out.stride(1) != 1 or out.shape[0] != T or out_col0 + channels > out.shape[1] or \
            (bias is not None and bias.numel() != channels) or activation not in (None, "silu") or \
            state.shape[1] < state_off + (taps - 1) * channels or state.stride(1) != 1:
        raise lib.KernelError("short_conv_state: shapes do not fit")
    lib.call("tm_short_conv_state", proj.data_ptr(), proj.stride(0), int(col0), channels, taps,
             _req(weight, "weight", torch.float32), _opt(bias, "bias", torch.float32), _req(state, "state", torch.float32),
             state.stride(0), int(state_off), _req(cu_q, "cu_q", torch.int32), _req(seq_of_token, "seq_of_token", torch.int32),
             _req(state_slots, "state_slots", torch.int32), int(activation == "silu"), out.data_ptr(), out.stride(0),
             int(out_col0), T, _stream())
    return out


def delta_prepare(x: torch.Tensor, q_col: int, k_col: int, qk_heads: int, dim: int, q_scale: float, unit_eps: float,
                  raw: torch.Tensor, b_col: int, a_col: int, A_log: torch.Tensor, dt_bias: torch.Tensor, heads: int,
                  gb: torch.Tensor) -> torch.Tensor:
    """In place on x [T, P] float32: every q and k head (qk_heads x dim at the given columns) becomes x / sqrt(sum x^2 +
    unit_eps), q also times q_scale. From raw [T, R] float32 (rows may be strided): gb [T, 2 heads] <- (exp(-exp(A_log)
    softplus(raw[a_col + h] + dt_bias)), sigmoid(raw[b_col + h]))."""
    T = x.shape[0]
    if x.dtype != torch.float32 or x.stride(1) != 1 or max(q_col, k_col) + qk_heads * dim > x.shape[1] or \
            raw.dtype != torch.float32 or raw.stride(1) != 1 or max(a_col, b_col) + heads > raw.shape[1] or \
            gb.shape != (T, 2 * heads) or A_log.numel() != heads or dt_bias.numel() != heads:
        raise lib.KernelError("delta_prepare: shapes do not fit")
    lib.call("tm_delta_prepare", x.data_ptr(), x.stride(0), int(q_col), int(k_col), int(qk_heads), int(dim), float(q_scale),
             float(unit_eps), raw.data_ptr(), raw.stride(0), int(b_col), int(a_col), _req(A_log, "A_log", torch.float32),
             _req(dt_bias, "dt_bias", torch.float32), int(heads), _req(gb, "gb", torch.float32), T, _stream())
    return gb


def forget_gate_prepare(x: torch.Tensor, q_col: int, f_col: int, n: int, low: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
    """In place on x [T, P] float32 (rows may be strided): the n columns at q_col <- silu, the n columns at f_col <-
    low + (1 - low) sigmoid(. + bias); low, bias [n] float32."""
    if x.dtype != torch.float32 or x.stride(1) != 1 or max(q_col, f_col) + n > x.shape[1] or low.numel() != n or \
            (bias is not None and bias.numel() != n):
        raise lib.KernelError("forget_gate_prepare: shapes do not fit")
    lib.call("tm_forget_gate_prepare", x.data_ptr(), x.stride(0), int(q_col), int(f_col), int(n), _req(low, "low", torch.float32),
             _opt(bias, "bias", torch.float32), x.shape[0], _stream())
    return x


def talk_mix(cross: torch.Tensor, talk: torch.Tensor, out: torch.Tensor, heads: int, kv_heads: int, vdim: int,
             scale: float = 1.0) -> torch.Tensor:
    """cross [T, heads * kv_heads * vdim] float32 (head g's softmax weights applied to the values of every value head);
    talk [heads, heads] float32; out [T, heads * vdim] (rows may be strided: columns of a wider matrix) <- scale * sum_g
    talk[h, g] cross[t, g, value head of h]."""
    T = cross.shape[0]
    if cross.shape != (T, heads * kv_heads * vdim) or talk.shape != (heads, heads) or out.shape != (T, heads * vdim) or \
            out.stride(1) != 1 or not out.is_cuda:
        raise lib.KernelError("talk_mix: shapes do not fit")
    lib.call("tm_talk_mix", _code(out.dtype), _req(cross, "cross", torch.float32), _req(talk, "talk", torch.float32),
             out.data_ptr(), out.stride(0), float(scale), T, heads, kv_heads, vdim, _stream())
    return out
