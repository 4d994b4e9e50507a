"""ctypes binding of the compiled kernel library.

There is no other implementation behind these calls: if the library cannot be built or loaded, or a
launch reports an error, an exception is raised. ``launch_count`` counts every kernel entry point
called, which is what the benchmark reports as its own launches.
"""

from __future__ import annotations

import ctypes
import threading
from ctypes import c_float, c_int, c_longlong, c_void_p

from . import build as _build


class KernelError(RuntimeError):
    pass


_REFUSALS = {
    90001: "unsupported shape for this kernel",
    90002: "unsupported dtype for this kernel",
    90003: "scratch buffer missing or too small",
    90004: "size beyond the entry point's fixed scratch capacity",
    90005: "device-side wait ran out (kernel gave up and reported instead of hanging)",
    90006: "tensor map could not be encoded",
}

_lock = threading.Lock()
_libs: dict[str, ctypes.CDLL] = {}          # by library (kernels/build.py: "main", "hybrid"), loaded on first use
launch_count = 0

_P, _I, _F, _LL = c_void_p, c_int, c_float, c_longlong

# name -> argument types (the trailing stream pointer included)
_SIGNATURES: dict[str, list] = {
    "tm_add_rmsnorm": [_I, _P, _P, _P, _I, _LL, _P, _P, _P, _P, _F, _P, _I, _I, _P],
    "tm_qkv_rope_write": [_I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P],
    "tm_kv_cache_write": [_I, _P, _P, _P, _P, _P, _I, _I, _P],
    "tm_paged_attention": [_I, _P, _P, _P, _P, _I, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I,
                           _I, _P],
    "tm_attention_combine": [_I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "tm_decode_attention_bf16": [_P, _P, _P, _P, _I, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _I, _P, _P],
    "tm_decode_attention_units_bf16": [_P, _P, _P, _LL, _P, _I, _P, _P, _P, _P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I,
                                       _I, _P, _P],
    "tm_decode_attention_units_rope_bf16": [_P, _P, _P, _P, _P, _I, _P, _P, _P, _LL, _P, _I, _P, _P, _P, _P, _I, _I, _P, _P, _P,
                                            _P, _I, _I, _I, _I, _F, _I, _I, _P, _P],
    "tm_decode_attention_units_slots": [_I, _I],
    "tm_prefill_attention_bf16": [_P, _P, _P, _P, _I, _P, _I, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _P],
    "tm_prefill_attention_tc_timing": [_P],
    "tm_decode_attention_units_timing": [_P],
    "tm_prefill_attention_tc_bf16": [_P, _P, _P, _P, _I, _P, _I, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _P, _P],
    "tm_swiglu": [_I, _P, _P, _I, _I, _P],
    "tm_skinny_linear": [_P, _I, _P, _P, _P, _I, _I, _P, _I, _I, _I, _I, _I, _P],
    "tm_skinny_qkv_rope_write": [_P, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P],
    "tm_skinny_gate_up_swiglu": [_P, _I, _P, _P, _I, _I, _I, _I, _P],
    "tm_tc_linear": [_P, _I, _P, _P, _I, _I, _I, _I, _P, _P],
    "tm_tc_linear_add_f32": [_P, _I, _P, _P, _I, _I, _I, _I, _P, _P],
    "tm_tc_gate_up_swiglu": [_P, _I, _P, _P, _I, _I, _I, _I, _P, _P],
    "tm_tc_qkv_rope_write": [_P, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P],
    "tm_decode_fused": [_P, _P],
    "tm_decode_fused_max_tokens": [_I, _I, _I, _I, _I, _I],
    "tm_lm_head_bf16": [_P, _P, _P, _I, _I, _I, _P, _P],
    "tm_stream_linear_bf16": [_P, _P, _P, _I, _I, _I, _P, _P],
    "tm_lm_head_argmax_bf16": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P, _P],
    "tm_stream_linear_slices": [_I],
    "tm_swiglu_partials": [_P, _I, _LL, _P, _I, _I, _P],
    "tm_gemm_f32_nt": [_P, _I, _P, _P, _P, _I, _I, _I, _I, _P],
    "tm_add_norm_pair": [_I, _P, _P, _P, _F, _P, _P, _P, _P, _P, _F, _P, _I, _P, _I, _I, _P],
    "tm_token_shift": [_I, _P, _P, _P, _LL, _P, _P, _P, _P, _I, _I, _P],
    "tm_gated_group_norm": [_I, _P, _P, _LL, _P, _F, _P, _I, _I, _I, _P],
    "tm_latent_prepare": [_I, _P, _I, _I, _I, _I, _P, _P, _F, _P, _P, _P, _I, _P, _P, _P, _I, _P, _P],
    "tm_latent_attention": [_I, _P, _LL, _LL, _P, _LL, _LL, _P, _P, _I, _P, _P, _I, _P, _P, _P, _P, _I, _P, _LL, _LL,
                            _I, _I, _I, _I, _F, _I, _P],
    "tm_latent_attention_mma_bf16": [_P, _LL, _LL, _P, _LL, _LL, _P, _P, _I, _P, _P, _I, _P, _P, _P, _P, _I, _P, _LL, _LL,
                                     _I, _I, _I, _I, _F, _I, _I, _P, _I, _P],
    "tm_conv_silu_state": [_I, _P, _LL, _I, _I, _I, _P, _P, _P, _P, _LL, _P, _P, _P, _P, _I, _P],
    "tm_ssm_scan": [_I, _P, _I, _P, _LL, _I, _P, _P, _P, _P, _LL, _LL, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P, _P],
    "tm_ssm_pass_states": [_P, _LL, _LL, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "tm_relu2": [_I, _P, _P, _LL, _P],
    "tm_moe_topk": [_P, _P, _P, _P, _P, _I, _I, _I, _LL, _I, _P],
    "tm_glu_routed_in": [_I, _P, _P, _P, _I, _I, _I, _I, _P, _LL, _P],
    "tm_glu_routed": [_I, _P, _P, _P, _I, _I, _I, _P],
    "tm_gemm_f32_nt_batched": [_P, _LL, _I, _P, _LL, _P, _LL, _I, _I, _I, _I, _I, _P],
    "tm_gated_add_rmsnorm": [_I, _P, _P, _P, _LL, _P, _P, _P, _F, _P, _P, _F, _P, _I, _I, _P],
    "tm_canon_conv": [_I, _P, _P, _P, _LL, _P, _P, _P, _P, _I, _I, _I, _P],
    "tm_glu": [_I, _I, _P, _P, _I, _I, _P],
    "tm_norm_pair_mean": [_I, _P, _P, _P, _P, _F, _P, _I, _I, _P],
    "tm_weighted_pair": [_I, _P, _P, _F, _F, _P, _LL, _P],
    "tm_head_norm_gate": [_I, _P, _P, _P, _LL, _I, _P, _F, _P, _LL, _I, _I, _I, _P],
    "tm_qk_norm_rope_write": [_I, _P, _LL, _I, _I, _I, _I, _I, _P, _P, _F, _P, _P, _P, _I, _P, _P, _P, _P, _I, _I, _F, _I, _I,
                              _I, _P, _P],
    "tm_sink_attention": [_I, _P, _P, _I, _I, _P, _I, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _F, _I, _I, _I, _I, _P,
                          _P],
    "tm_sink_attention_mma_bf16": [_P, _P, _I, _I, _P, _I, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _F, _I, _I, _I, _I,
                                   _P, _P, _I, _P, _P],
    "tm_moe_choose": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "tm_act_routed": [_I, _P, _P, _I, _P, _I, _I, _I, _P],
    "tm_add_scaled_rows": [_I, _P, _P, _P, _I, _I, _P],
    "tm_stream_norm": [_I, _P, _I, _I, _P, _P, _P, _P, _P, _P, _P, _LL, _P, _P, _P, _P, _I, _P, _P, _P, _F, _P, _I, _F, _P],
    "tm_softcap": [_P, _LL, _F, _F, _P],
    "tm_gated_memory": [_P, _LL, _I, _I, _I, _P, _I, _I, _P, _LL, _LL, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "tm_gated_memory_pass_states": [_P, _LL, _LL, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "tm_short_conv_state": [_P, _LL, _I, _I, _I, _P, _P, _P, _LL, _LL, _P, _P, _P, _I, _P, _LL, _I, _I, _P],
    "tm_delta_prepare": [_P, _LL, _I, _I, _I, _I, _F, _F, _P, _LL, _I, _I, _P, _P, _I, _P, _I, _P],
    "tm_forget_gate_prepare": [_P, _LL, _I, _I, _I, _P, _P, _I, _P],
    "tm_talk_mix": [_I, _P, _P, _P, _LL, _F, _I, _I, _I, _I, _P],
    "tm_selective_scan": [_I, _P, _I, _P, _LL, _I, _P, _LL, _I, _I, _P, _P, _P, _P, _P, _LL, _LL, _P, _P, _P, _I, _I, _I, _I,
                          _P, _P, _P],
    "tm_selective_pass_states": [_I, _P, _LL, _LL, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    "tm_decay_memory": [_P, _LL, _I, _I, _I, _I, _P, _P, _LL, _LL, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "tm_decay_pass_states": [_P, _LL, _LL, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "tm_decay_activate": [_P, _LL, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "tm_matrix_memory": [_P, _LL, _I, _I, _I, _I, _I, _P, _P, _F, _F, _P, _LL, _LL, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P,
                         _LL, _I, _P],
    "tm_matrix_memory_pass_states": [_P, _LL, _LL, _P, _P, _I, _I, _I, _I, _I, _P, _LL, _P],
    "tm_argmax": [_P, _I, _I, _LL, _P, _P, _P, _P],
    "tm_sample": [_P, _I, _I, _LL, _P, _P, _P, _P, _P, _P, _I, _P, _P],
}


# Entry points of the libraries beside "main", file by file; everything else is in "main". A file may be part of several
# libraries (kernels/build.py); the 32-bit matrix product is in all.
_BY_FILE = {
    "norm_pair.cu": {"tm_add_norm_pair", "tm_token_shift", "tm_gated_group_norm"},
    "latent_attention.cu": {"tm_latent_prepare", "tm_latent_attention"},
    "latent_attention_mma_bf16.cu": {"tm_latent_attention_mma_bf16"},
    "ssm_scan.cu": {"tm_conv_silu_state", "tm_ssm_scan", "tm_ssm_pass_states"},
    "routed_ffn.cu": {"tm_relu2", "tm_moe_topk", "tm_glu_routed", "tm_gemm_f32_nt_batched", "tm_moe_choose", "tm_act_routed",
                      "tm_add_scaled_rows", "tm_glu_routed_in"},
    "gated_block.cu": {"tm_gated_add_rmsnorm", "tm_canon_conv", "tm_glu", "tm_norm_pair_mean", "tm_head_norm_gate",
                       "tm_weighted_pair"},
    "sink_attention.cu": {"tm_qk_norm_rope_write", "tm_sink_attention"},
    "sink_attention_mma_bf16.cu": {"tm_sink_attention_mma_bf16"},
    "matrix_memory.cu": {"tm_matrix_memory", "tm_matrix_memory_pass_states"},
    "stream_norm.cu": {"tm_stream_norm", "tm_softcap"},
    "selective_scan.cu": {"tm_selective_scan", "tm_selective_pass_states"},
    "decay_memory.cu": {"tm_decay_memory", "tm_decay_pass_states", "tm_decay_activate"},
    "gated_memory.cu": {"tm_gated_memory", "tm_gated_memory_pass_states", "tm_short_conv_state", "tm_delta_prepare",
                        "tm_forget_gate_prepare", "tm_talk_mix"},
}
_BOTH = {"tm_gemm_f32_nt"}            # in every library
_GROUPS_OF: dict[str, list[str]] = {}     # entry point -> the libraries that hold it, in the order of kernels/build.py
for _group, _files in _build._FILES.items():
    for _file in _files:
        for _name in _BY_FILE[_file]:
            _GROUPS_OF.setdefault(_name, []).append(_group)
_preferred: list[str] = []            # libraries a model has said it runs from (``prefer``), latest first


def prefer(group: str) -> None:
    """Say that entry points which several libraries hold are to come from ``group`` when none of those is loaded yet
    (a model whose kernels are all in one library then builds and loads that one only)."""
    if group not in _build.GROUPS:
        raise KernelError(f"unknown kernel library {group!r}")
    if group in _preferred:
        _preferred.remove(group)
    _preferred.insert(0, group)


def _in_group(name: str, group: str) -> bool:
    return name in _BOTH or (group in _GROUPS_OF[name] if name in _GROUPS_OF else group == "main")


def _group_of(name: str) -> str:
    if name in _BOTH:                 # from whichever library is loaded (none yet: the preferred one, or the small one)
        return next(iter(_libs), _preferred[0] if _preferred else "hybrid")
    homes = _GROUPS_OF.get(name)
    if homes is None:
        return "main"
    for group in _libs:               # a loaded library that holds it
        if group in homes:
            return group
    return next((g for g in _preferred if g in homes), homes[0])


def register_signature(name: str, argtypes: list) -> None:
    """Declare one more exported entry point of the main library (used by kernel files added later)."""
    _SIGNATURES[name] = argtypes
    if "main" in _libs:
        _bind(_libs["main"], name, argtypes)


def _bind(lib: ctypes.CDLL, name: str, argtypes: list) -> None:
    try:
        fn = getattr(lib, name)
    except AttributeError:
        raise KernelError(f"the kernel library lacks the entry point {name}") from None
    fn.argtypes = argtypes
    fn.restype = c_int


def load(group: str = "main") -> ctypes.CDLL:
    """Build (if needed) and load one of the libraries. Raises if that is impossible."""
    lib = _libs.get(group)
    if lib is not None:
        return lib
    with _lock:
        if group not in _libs:
            path = _build.build(group=group)
            lib = ctypes.CDLL(str(path))
            for name, argtypes in _SIGNATURES.items():
                if _in_group(name, group):
                    _bind(lib, name, argtypes)
            _libs[group] = lib
    return _libs[group]


def library_file(group: str = "main") -> str:
    return str(_build.library_path(group))


def loaded_libraries() -> list[str]:
    return [library_file(g) for g in _libs]


def call(name: str, *args) -> None:
    """Call an entry point; a non-zero status raises."""
    global launch_count
    lib = load(_group_of(name))
    status = getattr(lib, name)(*args)
    launch_count += 1
    if status != 0:
        reason = _REFUSALS.get(status)
        if reason is None:
            reason = f"CUDA error {status}"
            try:
                import torch

                reason += f" ({torch.cuda.cudart().cudaGetErrorString(status)})"  # type: ignore[attr-defined]
            except Exception:
                pass
        raise KernelError(f"{name}: {reason}")
