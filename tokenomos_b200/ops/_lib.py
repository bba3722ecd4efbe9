"""Loads the kernel library through ctypes and declares its entry points.

The entry points are plain C functions over device pointers, sizes and a stream; each returns 0
or a negative code, and ``tk_last_error`` gives the message. There is no other implementation
behind them: if the library cannot be built or loaded, the import of an op raises.
"""

from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p

from tokenomos_b200.csrc import build as _build

F32, BF16 = 0, 1

_lock = threading.Lock()
_lib: ctypes.CDLL | None = None

P, I, L, F = c_void_p, c_int, c_int64, c_float

_SIGNATURES = {
    "tk_check_device": [],
    "tk_built_for": [],
    "tk_set_pdl": [I],
    "tk_checks_enabled": [],
    "tk_checks_set_bounds": [I, I],
    "tk_checks_status": [P],
    "tk_gather_rows": [P, P, P, I, I, I, I, P],
    "tk_gather_rows_select": [P, P, P, P, P, P, I, I, I, I, P],
    "tk_add_rmsnorm": [P, L, P, P, F, P, F, P, P, I, I, I, P],
    "tk_swiglu": [P, P, I, I, I, I, P],
    "tk_head_gate": [P, P, L, I, I, I, I, P],
    "tk_qk_norm_rope_write": [P, L, P, P, P, P, F, P, P, P, P, I, I, I, I, I, I, I, I, P],
    "tk_attn_generic_rows": [],
    "tk_attn_generic": [P, P, P, P, P, P, I, P, P, I, I, I, I, I, I, I, I, I, I, I, I, F, I, P],
    "tk_rotary_write": [P, L, P, P, P, F, P, P, P, I, I, I, I, I, I, I, I, I, I, I, I, P],
    "tk_stream32_add_norm": [P, P, L, P, P, P, F, P, P, P, I, I, I, P],
    "tk_glu_clamped": [P, P, I, I, I, F, F, F, I, P],
    "tk_gemm_skinny_glu": [P, L, P, L, P, P, L, I, I, I, I, F, F, F, P],
    "tk_sigmoid_gate": [P, P, L, I, I, I, P],
    "tk_attn_mma_supported": [I, I, I],
    "tk_attn_prefill_mma_tokens": [I, I],
    "tk_attn_prefill_mma": [P, P, P, P, P, P, I, P, P, I, I, I, I, I, I, F, P, L, P],
    "tk_attn_prefill_mma_opt": [P, P, P, P, P, P, I, P, P, I, I, I, I, I, I, F, P, L, I, I, I, P],
    "tk_attn_decode_mma_opt": [P, P, P, P, P, P, I, P, I, I, I, I, I, I, F, I, P, P, L, I, I, I, P],
    "tk_attn_prefill_tc_supported": [I, I, I],
    "tk_attn_prefill_tc_tokens": [I, I],
    "tk_attn_prefill_tc_status": [],
    "tk_attn_prefill_tc": [P, P, P, P, P, P, I, P, P, I, I, I, I, I, I, F, P, L, I, P, P, P],
    "tk_attn_prefill_tc_opt": [P, P, P, P, P, P, I, P, P, I, I, I, I, I, I, F, P, L, I, P, P, I, I, I, P],
    "tk_attn_decode_mma": [P, P, P, P, P, P, I, P, I, I, I, I, I, I, F, I, P, P, L, P],
    "tk_attn_decode_fused_supported": [I, I, I, I],
    "tk_attn_decode_fused_max_splits": [I, I, I],
    "tk_attn_decode_fused_opt": [P, L, P, P, P, P, F, P, I, P, L, P, P, P, I, I, I, I, I, I, I, F, I, P, P, I, I,
                                 I, F, I, I, I, I, I, P],
    "tk_attn_decode_fused": [P, L, P, P, P, P, F, P, I, P, L, P, P, P, I, I, I, I, I, I, I, F, I, P, P, I, I, P],
    "tk_conv_min_tile": [I],
    "tk_conv_gated": [P, L, I, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, P],
    "tk_gemm_skinny_conv": [P, L, P, L, P, P, L, I, I, I, P, P, P, P, P, I, F, P],
    "tk_gemm_simt": [P, L, P, L, P, P, L, I, I, I, I, I, P],
    "tk_gemm_skinny": [P, L, P, L, P, P, L, I, I, I, I, I, F, P, L, P],
    "tk_sample": [P, L, I, I, P, P, P, P, P, P, P, P, P, P],
    "tk_scale_rows": [P, L, F, I, P],
    "tk_logit_options": [P, L, I, I, F, F, P, I, P],
    "tk_gemm_tc_status": [],
    "tk_sample_status": [],
    "tk_gemm_tc_decode": [P, L, P, L, P, P, L, I, I, I, I, I, I, P],
    "tk_embed_bigram_norm": [P, P, P, F, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, P],
    "tk_hc_mix_norm": [P, P, L, P, P, P, P, F, P, P, I, I, I, I, P, P, P, P, I, P],
    "tk_canon_conv": [P, P, P, P, P, P, P, P, P, P, I, P, I, I, I, P],
    "tk_latent_prepare": [P, L, P, P, F, P, P, P, P, I, P, P, I, I, I, I, I, I, I, P],
    "tk_latent_rotate_q": [P, P, P, I, I, I, I, I, I, P],
    "tk_attn_latent_rows": [],
    "tk_attn_latent_max_rank": [],
    "tk_attn_latent": [P, P, P, P, P, P, P, I, P, P, I, I, I, I, I, I, I, I, I, F, I, P],
    "tk_attn_latent_mma_rows": [],
    "tk_attn_latent_mma_supported": [I, I, I],
    "tk_attn_latent_mma": [P, P, P, P, P, P, P, I, P, P, I, I, I, I, I, I, I, I, I, F, I, P, P, I, P],
    "tk_attn_latent_merge": [P, P, P, I, I, I, P],
    "tk_head_gate_transpose": [P, P, L, P, I, I, I, I, P],
    "tk_moe_route": [P, L, I, I, I, F, I, P, P, P, P],
    "tk_moe_sort": [P, I, I, I, I, I, P, P, P, P, P],
    "tk_gather_rows_or_zero": [P, P, P, I, I, I, P],
    "tk_gemm_grouped_tile": [],
    "tk_gemm_grouped_simt": [P, L, L, P, P, L, L, P, P, L, L, I, I, I, I, I, I, P],
    "tk_gemm_grouped_mma": [P, L, L, P, P, L, L, P, P, L, L, I, I, I, I, I, I, P, L, P],
    "tk_moe_combine": [P, P, P, P, P, P, I, I, I, I, P],
    "tk_relu2": [P, L, I, P],
    "tk_scale_rows_f32": [P, L, P, F, I, I, I, P],
    "tk_seq_conv": [P, L, I, P, P, P, P, P, P, P, P, P, P, I, P, L, P, L, I, I, I, I, I, I, P, P, I, I, I, I, I, I, P],
    "tk_attn_pointwise_rows": [],
    "tk_attn_pointwise": [P, P, P, P, P, P, I, P, P, I, I, I, I, I, I, I, I, I, F, F, F, I, P, P, P, I, P],
    "tk_attn_pointwise_mma_supported": [I, I, I, I, I],
    "tk_attn_pointwise_mma_tokens": [I, I],
    "tk_attn_pointwise_mma": [P, P, P, P, P, P, I, P, P, I, P, I, I, P, I, I, I, I, I, F, F, F, I, P, P, P, P],
    "tk_rglru_scan": [P, I, P, P, P, P, L, P, L, P, P, P, P, I, P, I, I, I, P],
    "tk_mlstm_scan": [P, L, I, I, I, P, L, F, F, P, P, P, P, P, I, I, P, P, I, I, I, I, P],
    "tk_mlstm_norm_gate": [P, P, P, P, P, L, P, P, P, P, I, I, I, F, I, P],
    "tk_ssd_max_state": [],
    "tk_ssd_scan": [P, L, P, L, P, P, P, P, P, P, P, I, I, P, I, I, I, I, I, I, P],
    "tk_ssd_split": [I, I, I, I, I, I],
    "tk_gated_group_norm": [P, I, P, L, P, F, P, I, I, I, I, P],
    "tk_qkv_maps_write": [P, L, P, P, P, I, P, P, I, I, I, I, I, I, I, I, I, P],
    "tk_diff_combine": [P, P, I, I, F, F, F, I, P],
    "tk_stream32_group_norm": [P, P, L, P, L, P, F, P, P, I, I, I, I, P],
}


class KernelError(RuntimeError):
    """A kernel entry point refused its arguments or failed to launch."""


def lib() -> ctypes.CDLL:
    """The loaded library, built on first use."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            path = _build.build()
            loaded = ctypes.CDLL(str(path))
            loaded.tk_last_error.restype = c_char_p
            loaded.tk_last_error.argtypes = []
            for name, args in _SIGNATURES.items():
                fn = getattr(loaded, name)
                fn.restype = c_int
                fn.argtypes = args
            if os.environ.get("TOKENOMOS_B200_PDL", "1") == "0":
                loaded.tk_set_pdl(0)
            _lib = loaded
    return _lib


def declare(name: str, args: list) -> None:
    """Declare one more entry point (used by modules that add kernels to the table above)."""
    _SIGNATURES[name] = args
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.restype = c_int
        fn.argtypes = args


_calls = 0


def calls() -> int:
    """How many kernel entry points have been called in this process (each launches one
    kernel of this library; queries such as ``tk_conv_min_tile`` are not counted)."""
    return _calls


_QUERIES = {"tk_check_device", "tk_built_for", "tk_set_pdl", "tk_checks_enabled", "tk_checks_set_bounds", "tk_checks_status", "tk_attn_generic_rows", "tk_conv_min_tile",
            "tk_attn_mma_supported", "tk_attn_decode_fused_supported", "tk_attn_decode_fused_max_splits", "tk_attn_prefill_mma_tokens", "tk_attn_prefill_tc_supported",
            "tk_attn_prefill_tc_tokens", "tk_attn_prefill_tc_status", "tk_gemm_tc_status", "tk_sample_status",
            "tk_attn_latent_rows", "tk_attn_latent_max_rank", "tk_gemm_grouped_tile", "tk_attn_latent_mma_rows",
            "tk_attn_latent_mma_supported", "tk_attn_pointwise_rows", "tk_attn_pointwise_mma_supported",
            "tk_attn_pointwise_mma_tokens", "tk_ssd_max_state", "tk_ssd_split"}


_fns: dict = {}


def call(name: str, *args) -> int:
    """Call an entry point; a negative return raises ``KernelError`` with the library's message."""
    global _calls
    fn = _fns.get(name)
    if fn is None:
        fn = _fns[name] = (getattr(lib(), name), name not in _QUERIES)
    if fn[1]:
        _calls += 1
    rc = fn[0](*args)
    if rc < 0:
        raise KernelError(f"{name}: {lib().tk_last_error().decode()}")
    return rc
