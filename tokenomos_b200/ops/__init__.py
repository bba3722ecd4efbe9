"""The kernels as functions over torch tensors on a CUDA device.

torch is the allocator and the stream owner here, nothing more: every function checks its
tensors, picks the entry point for the storage type (float32 or bfloat16) and launches on the
current stream. Tensors on the CPU are refused: there is no CPU implementation on the product
path (the plain implementation under ``tests/`` is the oracle, not a fallback).
"""

from __future__ import annotations

import torch

from tokenomos_b200.ops import _lib
from tokenomos_b200.ops._lib import BF16, F32, KernelError

__all__ = [
    "KernelError", "available", "checks_enabled", "set_check_bounds", "checks_status", "gather_rows", "add_rmsnorm", "swiglu", "head_gate",
    "qk_norm_rope_write", "rotary_write", "stream32_add_norm", "glu_clamped", "gemm_skinny_glu", "sigmoid_gate", "attention", "attention_rows", "attention_mma_supported",
    "attention_prefill_mma", "attention_prefill_mma_tokens", "attention_decode_mma",
    "attention_prefill_tc", "attention_prefill_tc_supported", "attention_prefill_tc_tokens",
    "attention_prefill_tc_status",
    "conv_gated", "conv_min_tile",
    "gemm", "gemm_skinny", "gemm_skinny_conv", "gemm_skinny_ok", "gemm_tc", "gemm_tc_ok", "gemm_tc_status", "sample", "sample_status", "gather_rows_select",
]


# What the kernels take, so that a model that asks for more is refused when it is built and not
# at its first step (the entry points check the same limits: conv.cu and gemm_skinny.cu, the row
# that add_rmsnorm keeps in shared memory, attention_generic.cu's MAX_D, qk_rope.cu)
CONV_WIDTHS = (2, 8)
NORM_MAX_WIDTH = 51200
ATTENTION_MAX_HEAD_DIM = 256


def available() -> None:
    """Raise unless the library loads and the current device can run it."""
    _lib.call("tk_check_device")


def checks_enabled() -> bool:
    """Whether the loaded library is the debug build whose kernels check the indices they follow
    (``TOKENOMOS_B200_CHECKS=1`` at first use; csrc/checks.cuh)."""
    return bool(_lib.call("tk_checks_enabled"))


def set_check_bounds(pages: int, slots: int) -> None:
    """What the index checks compare against: pages per paged pool, rows per state tensor."""
    _lib.call("tk_checks_set_bounds", int(pages), int(slots))


CHECKED_KERNELS = {1: "row gather", 2: "q/k norm + rope + cache write", 3: "attention (generic)",
                   4: "attention (tensor cores)", 5: "gated short conv", 6: "projection with the conv inside"}
CHECKED_INDICES = {1: "page", 2: "state row", 3: "table row"}


def checks_status() -> str | None:
    """None, or what the first index was that a kernel found outside its pool since the last call
    (the kernel went on with the null page or row instead of following it)."""
    import ctypes

    word = (ctypes.c_int * 2)()
    _lib.call("tk_checks_status", ctypes.cast(word, ctypes.c_void_p))
    if word[0] == 0:
        return None
    kernel, what = divmod(word[0], 8)
    return (f"{CHECKED_KERNELS.get(kernel, f'kernel {kernel}')}: {CHECKED_INDICES.get(what, 'index')} "
            f"{word[1]} is outside its pool")


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"storage type {t.dtype} is not built (float32 and bfloat16 are)")


def _cuda(*tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("tokenomos_b200 kernels run on CUDA tensors only; got a "
                              f"{t.device} tensor (there is no CPU path)")


def _ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def _stream():
    # the raw handle of torch's current stream (a capture's side stream included); the private
    # getters skip torch.cuda's Python wrappers, which cost more than a kernel launch
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


def _i32(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous int32 tensor")
    return t


def _f32vec(t: torch.Tensor | None, name: str, n: int) -> torch.Tensor | None:
    if t is None:
        return None
    if t.dtype != torch.float32 or not t.is_contiguous() or t.numel() != n:
        raise KernelError(f"{name} must be a contiguous float32 vector of {n} elements, got "
                          f"{t.dtype} {tuple(t.shape)}")
    return t


def gather_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor | None = None):
    """``out[r] = table[ids[r]]``: the embedding lookup and the row selection before the head."""
    _cuda(table, ids, out)
    rows, width = ids.numel(), table.shape[1]
    if not table.is_contiguous():
        raise KernelError("gather_rows: the table must be contiguous")
    if out is None:
        out = torch.empty(rows, width, dtype=table.dtype, device=table.device)
    _lib.call("tk_gather_rows", _ptr(table), _ptr(_i32(ids, "ids")), _ptr(out), rows, width,
              table.shape[0], _dtype_code(table), _stream())
    return out


def gather_rows_select(table: torch.Tensor, ids_host: torch.Tensor, use_prev: torch.Tensor,
                       last_token: torch.Tensor, slot: torch.Tensor) -> torch.Tensor:
    """``out[r] = table[last_token[slot[r]] if use_prev[r] else ids_host[r]]`` (ids int32): the
    decode step's embedding lookup, fed on the device by the step before."""
    _cuda(table, ids_host, use_prev, last_token, slot)
    rows, width = ids_host.numel(), table.shape[1]
    if not table.is_contiguous():
        raise KernelError("gather_rows_select: the table must be contiguous")
    for name, t in (("use_prev", use_prev), ("slot", slot)):
        if _i32(t, name).numel() < rows:
            raise KernelError(f"gather_rows_select: {name} is shorter than ids_host")
    out = torch.empty(rows, width, dtype=table.dtype, device=table.device)
    _lib.call("tk_gather_rows_select", _ptr(table), _ptr(_i32(ids_host, "ids_host")), _ptr(use_prev),
              _ptr(_i32(last_token, "last_token")), _ptr(slot), _ptr(out), rows, width, table.shape[0],
              _dtype_code(table), _stream())
    return out


def scale_rows(x: torch.Tensor, scale: float) -> torch.Tensor:
    """In place ``x = round(x * round(scale))`` (both to ``x``'s type): an embedding scale."""
    _cuda(x)
    if not x.is_contiguous():
        raise KernelError("scale_rows: x must be contiguous")
    _lib.call("tk_scale_rows", _ptr(x), x.numel(), float(scale), _dtype_code(x), _stream())
    return x


def logit_options(logits: torch.Tensor, softcap: float | None, suppress: torch.Tensor | None,
                  scale: float | None = None) -> torch.Tensor:
    """In place on float32 ``logits`` [rows, vocab]: times ``scale`` if one is given, ``softcap *
    tanh(logits / softcap)`` if a cap is given, then ``-inf`` at the token ids of ``suppress`` (int32,
    each inside the vocabulary)."""
    _cuda(logits, suppress)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("logit_options: logits must be float32 [rows, vocab] with contiguous rows")
    n = 0 if suppress is None else _i32(suppress, "suppress").numel()
    _lib.call("tk_logit_options", _ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1],
              1.0 if scale is None else float(scale), float(softcap or 0.0), _ptr(suppress), n, _stream())
    return logits


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor | None, weight: torch.Tensor | None,
                eps: float, pre: tuple[torch.Tensor, float] | None = None):
    """``stream = residual + [pre-norm](x)``; ``y = rmsnorm(stream) * weight``.

    Returns ``(y, stream)``; ``stream`` is ``x`` itself when nothing was added, ``y`` is None
    without ``weight``. ``x`` may be a row-strided view; the other tensors are contiguous."""
    _cuda(x, residual, weight)
    rows, width = x.shape
    if x.stride(1) != 1:
        raise KernelError("add_rmsnorm: rows of x must be contiguous")
    w = _f32vec(weight, "norm weight", width)
    pre_w = _f32vec(pre[0], "pre-norm weight", width) if pre is not None else None
    y = torch.empty(rows, width, dtype=x.dtype, device=x.device) if w is not None else None
    writes = residual is not None or pre is not None
    stream = torch.empty(rows, width, dtype=x.dtype, device=x.device) if writes else None
    if residual is not None and (not residual.is_contiguous() or residual.shape != x.shape
                                 or residual.dtype != x.dtype):
        raise KernelError("add_rmsnorm: residual must match x and be contiguous")
    _lib.call("tk_add_rmsnorm", _ptr(x), x.stride(0), _ptr(residual), _ptr(pre_w),
              float(pre[1]) if pre is not None else 0.0, _ptr(w), float(eps), _ptr(y),
              _ptr(stream), rows, width, _dtype_code(x), _stream())
    if stream is None:
        stream = x if x.is_contiguous() else x.contiguous()
    return y, stream


def swiglu(gu: torch.Tensor, block: int = 0) -> torch.Tensor:
    """``silu(gate) * up`` for ``gu`` of width ``2 I``: ``gu = [gate | up]`` (``block`` 0), or gate
    and up alternating in runs of ``block`` channels."""
    _cuda(gu)
    if not gu.is_contiguous() or gu.shape[1] % 2:
        raise KernelError("swiglu: input must be contiguous with an even width")
    rows, inter = gu.shape[0], gu.shape[1] // 2
    out = torch.empty(rows, inter, dtype=gu.dtype, device=gu.device)
    _lib.call("tk_swiglu", _ptr(gu), _ptr(out), rows, inter, int(block), _dtype_code(gu), _stream())
    return out


def head_gate(x: torch.Tensor, g: torch.Tensor, heads: int, head_dim: int) -> torch.Tensor:
    """In place: ``x[t, h, :] *= sigmoid(g[t, h])``; ``g`` [T, heads] may be a column block of a
    wider tensor (rows any distance apart)."""
    _cuda(x, g)
    if not (x.is_contiguous() and g.dim() == 2 and g.stride(1) == 1 and g.dtype == x.dtype):
        raise KernelError("head_gate: contiguous x, g with contiguous rows, one storage type")
    rows = x.numel() // (heads * head_dim)
    if tuple(g.shape) != (rows, heads):
        raise KernelError("head_gate: one gate per (token, head)")
    _lib.call("tk_head_gate", _ptr(x), _ptr(g), g.stride(0), rows, heads, head_dim, _dtype_code(x),
              _stream())
    return x


def qk_norm_rope_write(qkv: torch.Tensor, kv_pool: torch.Tensor | None,
                       wq: torch.Tensor | None, wk: torch.Tensor | None, eps: float,
                       inv_freq: torch.Tensor, positions: torch.Tensor, tok_seq: torch.Tensor,
                       block_table: torch.Tensor | None, heads: int, kv_heads: int,
                       head_dim: int, page: int) -> torch.Tensor:
    """Norm + rotate the q and k heads of ``qkv`` [T, (H + 2 Hkv) D]; returns q [T, H, D] and
    writes k, v into ``kv_pool`` [pages, 2, Hkv, P, D] at each token's position. ``kv_heads`` 0:
    queries only (the layer reads another layer's cache)."""
    _cuda(qkv, kv_pool, wq, wk, inv_freq, positions, tok_seq, block_table)
    T = qkv.shape[0]
    if qkv.stride(1) != 1 or qkv.shape[1] != (heads + 2 * kv_heads) * head_dim:
        raise KernelError(f"qk_norm_rope_write: qkv of width {qkv.shape[1]} for {heads}+2*{kv_heads} "
                          f"heads of {head_dim}")
    rot = 2 * inv_freq.numel()
    _f32vec(inv_freq, "inv_freq", rot // 2)
    q = torch.empty(T, heads, head_dim, dtype=qkv.dtype, device=qkv.device)
    if kv_heads:
        if kv_pool is None or block_table is None:
            raise KernelError("qk_norm_rope_write: keys need a cache and a block table")
        if kv_pool.dtype != qkv.dtype or not kv_pool.is_contiguous() or tuple(kv_pool.shape[1:]) != (
                2, kv_heads, page, head_dim):
            raise KernelError(f"qk_norm_rope_write: cache {tuple(kv_pool.shape)} {kv_pool.dtype} does "
                              f"not match [pages, 2, {kv_heads}, {page}, {head_dim}] {qkv.dtype}")
        _i32(block_table, "block_table")
    _lib.call("tk_qk_norm_rope_write", _ptr(qkv), qkv.stride(0), _ptr(q), _ptr(kv_pool),
              _ptr(_f32vec(wq, "q_norm weight", head_dim)), _ptr(_f32vec(wk, "k_norm weight", head_dim)),
              float(eps), _ptr(inv_freq), _ptr(_i32(positions, "positions")),
              _ptr(_i32(tok_seq, "tok_seq")), _ptr(block_table),
              block_table.stride(0) if block_table is not None else 0, T, heads, kv_heads,
              head_dim, rot, page, _dtype_code(qkv), _stream())
    return q


def attention_rows() -> int:
    """Rows (token x query head of one group) a tile of the generic attention kernel holds."""
    return _lib.call("tk_attn_generic_rows")


def attention(q: torch.Tensor, kv_pool: torch.Tensor, positions: torch.Tensor,
              tok_seq: torch.Tensor, block_table: torch.Tensor, tile_tok0: torch.Tensor,
              tile_ntok: torch.Tensor, tokens_per_tile: int, window: int | None,
              scale: float, keep_first: int = 0, sink: bool = False, v_dim: int | None = None,
              round_p: bool = True) -> torch.Tensor:
    """Causal (optionally windowed) attention of ``q`` [T, H, D] over the paged cache
    ``kv_pool`` [pages, 2, Hkv, P, Dp], which already holds this step's keys. Tiles name runs of
    at most ``tokens_per_tile`` tokens of one sequence. ``keep_first``: that many first positions
    of a sequence stay visible behind the window; ``sink``: one is added to the softmax's
    denominator; ``v_dim``: the values' size (default: the keys'; the cache rows hold at least
    both); ``round_p``: the weights are rounded to the storage type before they meet the values
    (the 16-bit reference's rounding) instead of staying 32-bit. Returns [T, H, v_dim]."""
    _cuda(q, kv_pool, positions, tok_seq, block_table, tile_tok0, tile_ntok)
    T, H, D = q.shape
    _, two, Hkv, P, Dp = kv_pool.shape
    Dv = D if v_dim is None else int(v_dim)
    if two != 2 or Dp < max(D, Dv) or kv_pool.dtype != q.dtype or not (q.is_contiguous() and kv_pool.is_contiguous()):
        raise KernelError("attention: q / cache layouts do not match")
    out = torch.empty(T, H, Dv, dtype=q.dtype, device=q.device)
    _lib.call("tk_attn_generic", _ptr(q), _ptr(kv_pool), _ptr(out), _ptr(_i32(positions, "positions")),
              _ptr(_i32(tok_seq, "tok_seq")), _ptr(_i32(block_table, "block_table")),
              block_table.stride(0), _ptr(_i32(tile_tok0, "tile_tok0")),
              _ptr(_i32(tile_ntok, "tile_ntok")), tile_tok0.numel(), tokens_per_tile, H, Hkv, D, Dv, Dp, P,
              int(window or 0), int(keep_first), int(bool(sink)), int(bool(round_p)), float(scale),
              _dtype_code(q), _stream())
    return out


def rotary_write(qkv: torch.Tensor, kv_pool: torch.Tensor | None, freq: torch.Tensor, cs_mult: float,
                 positions: torch.Tensor, tok_seq: torch.Tensor, block_table: torch.Tensor | None,
                 heads: int, kv_heads: int, head_dim: int, v_dim: int, page: int, interleaved: bool,
                 v_is_k: bool) -> torch.Tensor:
    """Rotate the q and k heads of ``qkv`` (rows of ``heads`` query heads and ``kv_heads`` key
    heads of ``head_dim``, then, unless ``v_is_k``, ``kv_heads`` value heads of ``v_dim``) by
    ``position * freq`` with cos and sin times ``cs_mult``, columns paired (2i, 2i+1) when
    ``interleaved`` else (i, i + R/2), R = 2 len(freq). Returns q [T, H, head_dim]; keys and
    values go into ``kv_pool`` [pages, 2, Hkv, P, Dp] at each token's position (``v_is_k``: the
    value is the key as projected, not rotated). ``kv_heads`` 0: queries only."""
    _cuda(qkv, kv_pool, freq, positions, tok_seq, block_table)
    T = qkv.shape[0]
    width = (heads + kv_heads) * head_dim + (0 if v_is_k else kv_heads * v_dim)
    if qkv.stride(1) != 1 or qkv.shape[1] != width:
        raise KernelError(f"rotary_write: qkv of width {qkv.shape[1]}, the heads need {width}")
    rot = 2 * freq.numel()
    _f32vec(freq, "freq", rot // 2)
    q = torch.empty(T, heads, head_dim, dtype=qkv.dtype, device=qkv.device)
    row = 0
    if kv_heads:
        if kv_pool is None or block_table is None:
            raise KernelError("rotary_write: keys need a cache and a block table")
        row = kv_pool.shape[-1]
        if (kv_pool.dtype != qkv.dtype or not kv_pool.is_contiguous() or kv_pool.dim() != 5
                or tuple(kv_pool.shape[1:4]) != (2, kv_heads, page) or row < max(head_dim, v_dim)):
            raise KernelError(f"rotary_write: cache {tuple(kv_pool.shape)} {kv_pool.dtype} does not match "
                              f"[pages, 2, {kv_heads}, {page}, >= {max(head_dim, v_dim)}] {qkv.dtype}")
        _i32(block_table, "block_table")
    _lib.call("tk_rotary_write", _ptr(qkv), qkv.stride(0), _ptr(q), _ptr(kv_pool), _ptr(freq), float(cs_mult),
              _ptr(_i32(positions, "positions")), _ptr(_i32(tok_seq, "tok_seq")), _ptr(block_table),
              block_table.stride(0) if block_table is not None else 0, T, heads, kv_heads, head_dim,
              int(v_dim), int(row or max(head_dim, v_dim)), rot, page, int(bool(interleaved)), int(bool(v_is_k)),
              _dtype_code(qkv), _stream())
    return q


def stream32_add_norm(stream: torch.Tensor | None, x: torch.Tensor | None, weight: torch.Tensor | None,
                      eps: float, rows_add: torch.Tensor | None = None, vec_add: torch.Tensor | None = None,
                      out_dtype: torch.dtype | None = None, in_place: bool = False, wide: bool = False):
    """A residual stream kept in 32-bit: ``stream' = stream + x + rows_add + vec_add`` (each
    optional, ``stream`` float32 [rows, width], ``x`` and ``rows_add`` in the model's storage type,
    ``vec_add`` float32 [width]) and ``y = rmsnorm(stream') * weight`` in ``out_dtype`` (default: the
    type of ``x`` / ``rows_add``), rounded once. Returns ``(y, stream')``; ``y`` is None without
    ``weight``. ``in_place``: ``stream'`` overwrites ``stream``. ``wide``: the normed rows also unrounded, in
    float32: returns ``(y, y32, stream')``."""
    _cuda(stream, x, weight, rows_add, vec_add)
    ref = x if x is not None else (rows_add if rows_add is not None else stream)
    if ref is None:
        raise KernelError("stream32_add_norm: nothing to add up")
    rows, width = ref.shape
    store = out_dtype or (x.dtype if x is not None else (rows_add.dtype if rows_add is not None else torch.float32))
    if stream is not None and (stream.dtype != torch.float32 or not stream.is_contiguous()
                               or tuple(stream.shape) != (rows, width)):
        raise KernelError("stream32_add_norm: the stream is a contiguous float32 [rows, width] tensor")
    for name, t in (("x", x), ("rows_add", rows_add)):
        if t is not None and (t.dtype != store or tuple(t.shape) != (rows, width) or t.stride(1) != 1):
            raise KernelError(f"stream32_add_norm: {name} must be {store} [rows, width] with contiguous rows")
    if rows_add is not None and not rows_add.is_contiguous():
        raise KernelError("stream32_add_norm: rows_add must be contiguous")
    w = _f32vec(weight, "norm weight", width)
    v = _f32vec(vec_add, "vec_add", width)
    y = torch.empty(rows, width, dtype=store, device=ref.device) if w is not None else None
    out = stream if (in_place and stream is not None) else torch.empty(rows, width, dtype=torch.float32,
                                                                    device=ref.device)
    if store not in (torch.float32, torch.bfloat16):
        raise KernelError(f"storage type {store} is not built (float32 and bfloat16 are)")
    code = F32 if store == torch.float32 else BF16
    y32 = None
    if wide and w is not None:
        y32 = y if store == torch.float32 else torch.empty(rows, width, dtype=torch.float32, device=ref.device)
    _lib.call("tk_stream32_add_norm", _ptr(stream), _ptr(x), x.stride(0) if x is not None else 0, _ptr(rows_add),
              _ptr(v), _ptr(w), float(eps), _ptr(out), _ptr(y), _ptr(y32) if y32 is not y else None, rows, width, code,
              _stream())
    return (y, y32, out) if wide else (y, out)


def glu_clamped(gu: torch.Tensor, limit: float | None, alpha: float, shift: float, block: int = 0) -> torch.Tensor:
    """``g * sigmoid(alpha g) * (u + shift)`` with ``g = min(gate, limit)``, ``u = clamp(up,
    -limit, limit)`` for ``gu = [gate | up]`` of width ``2 I`` (``limit`` None: no clamp);
    ``block`` > 0: gate and up alternate in runs of ``block`` channels instead."""
    _cuda(gu)
    if not gu.is_contiguous() or gu.shape[1] % 2:
        raise KernelError("glu_clamped: input must be contiguous with an even width")
    rows, inter = gu.shape[0], gu.shape[1] // 2
    out = torch.empty(rows, inter, dtype=gu.dtype, device=gu.device)
    _lib.call("tk_glu_clamped", _ptr(gu), _ptr(out), rows, inter, int(block), float(limit or 0.0), float(alpha),
              float(shift), _dtype_code(gu), _stream())
    return out


def gemm_skinny_glu(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, limit: float | None,
                    alpha: float, shift: float) -> torch.Tensor:
    """The gate/up product of at most 16 rows with the clamped gated activation (``glu_clamped``)
    in its epilogue: ``w``'s rows (and ``bias``) alternate in runs of 8 (8 gate rows, the 8 up rows
    of the same channels); the activation is computed from the 32-bit sums and rounded once.
    Returns [M, N / 2]."""
    _cuda(x, w, bias)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or N % 16 or not gemm_skinny_ok(x, w):
        raise KernelError(f"gemm_skinny_glu: x {tuple(x.shape)} against w {tuple(w.shape)}")
    out = torch.empty(M, N // 2, dtype=x.dtype, device=x.device)
    _lib.call("tk_gemm_skinny_glu", _ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(_f32vec(bias, "bias", N)),
              _ptr(out), out.stride(0), M, N, K, _dtype_code(out), float(limit or 0.0), float(alpha), float(shift),
              _stream())
    return out


def sigmoid_gate(x: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """In place: ``x[t, c] *= sigmoid(g[t, c])`` for ``x`` [T, C] contiguous; ``g`` [T, C] may be a
    column block of a wider tensor."""
    _cuda(x, g)
    rows = g.shape[0]
    width = x.numel() // max(rows, 1)
    if not (x.is_contiguous() and g.dim() == 2 and g.stride(1) == 1 and g.dtype == x.dtype
            and g.shape[1] == width and x.numel() == rows * width):
        raise KernelError("sigmoid_gate: contiguous x [T, C], g [T, C] with contiguous rows, one storage type")
    _lib.call("tk_sigmoid_gate", _ptr(x), _ptr(g), g.stride(0), rows, width, _dtype_code(x), _stream())
    return x


def attention_mma_supported(heads: int, kv_heads: int, head_dim: int, dtype: torch.dtype) -> bool:
    """Whether the tensor-core attention kernels take this shape (else: ``attention``)."""
    return dtype == torch.bfloat16 and bool(_lib.call("tk_attn_mma_supported", heads, kv_heads, head_dim))


def attention_prefill_mma_tokens(heads: int, kv_heads: int) -> int:
    """Tokens per tile the tensor-core prefill kernel expects."""
    return _lib.call("tk_attn_prefill_mma_tokens", heads, kv_heads)


def _check_attention(q, kv_pool, name):
    T, H, D = q.shape
    _, two, Hkv, P, D2 = kv_pool.shape
    if (two != 2 or D2 != D or kv_pool.dtype != q.dtype or q.dtype != torch.bfloat16
            or not (q.is_contiguous() and kv_pool.is_contiguous())):
        raise KernelError(f"{name}: bfloat16 q [T, H, D] and cache [pages, 2, Hkv, P, D] expected")
    return T, H, D, Hkv, P


def _gate_view(gate: torch.Tensor | None, T: int, H: int, name: str):
    """(pointer, row stride) of an output gate [T, H] (one per head; with ``H`` the row's whole
    width, one per element: a bfloat16 view with unit column stride), or (None, 0)."""
    if gate is None:
        return None, 0
    if not gate.is_cuda or gate.dtype != torch.bfloat16 or tuple(gate.shape) != (T, H) or gate.stride(1) != 1:
        raise KernelError(f"{name}: gate must be a bfloat16 [T, {H}] CUDA view with unit column stride")
    return gate.data_ptr(), gate.stride(0)


def _gate_options(gate, gate_by_element: bool, T: int, H: int, D: int, name: str):
    """(pointer, row stride, gate mode of the kernels: 0 none, 1 per head, 2 per element)."""
    if gate is None:
        return None, 0, 0
    g_ptr, ldg = _gate_view(gate, T, H * D if gate_by_element else H, name)
    return g_ptr, ldg, 2 if gate_by_element else 1


def attention_prefill_mma(q: torch.Tensor, kv_pool: torch.Tensor, out: torch.Tensor,
                          positions: torch.Tensor, tok_seq: torch.Tensor,
                          block_table: torch.Tensor, tile_tok0: torch.Tensor,
                          tile_ntok: torch.Tensor, window: int | None, scale: float,
                          gate: torch.Tensor | None = None, keep_first: int = 0, sink: bool = False,
                          gate_by_element: bool = False) -> None:
    """Tensor-core attention for tiles of ``attention_prefill_mma_tokens`` tokens of one
    sequence; writes the tiles' rows of ``out`` [T, H, D], times the per-head output gate
    ``round(sigmoid(gate))`` [T, H] if one is given. ``keep_first``, ``sink``: as in
    ``attention``; ``gate_by_element``: ``gate`` is [T, H * D], one value per output element, and
    the 32-bit output times the 32-bit sigmoid is rounded once."""
    _cuda(q, kv_pool, out, positions, tok_seq, block_table, tile_tok0, tile_ntok)
    T, H, D, Hkv, P = _check_attention(q, kv_pool, "attention_prefill_mma")
    g_ptr, ldg, mode = _gate_options(gate, gate_by_element, T, H, D, "attention_prefill_mma")
    _lib.call("tk_attn_prefill_mma_opt", _ptr(q), _ptr(kv_pool), _ptr(out), _ptr(_i32(positions, "positions")),
              _ptr(_i32(tok_seq, "tok_seq")), _ptr(_i32(block_table, "block_table")),
              block_table.stride(0), _ptr(_i32(tile_tok0, "tile_tok0")),
              _ptr(_i32(tile_ntok, "tile_ntok")), tile_tok0.numel(), H, Hkv, D, P, int(window or 0),
              float(scale), g_ptr, ldg, int(keep_first), int(bool(sink)), mode, _stream())


def attention_prefill_tc_supported(heads: int, kv_heads: int, head_dim: int, dtype: torch.dtype) -> bool:
    """Whether the tcgen05 prefill kernel takes this shape (bfloat16, head size 64, a group that
    divides 128)."""
    return dtype == torch.bfloat16 and bool(_lib.call("tk_attn_prefill_tc_supported", heads, kv_heads, head_dim))


def attention_prefill_tc_tokens(heads: int, kv_heads: int) -> int:
    """Tokens of one sequence per tile of ``attention_prefill_tc``."""
    return _lib.call("tk_attn_prefill_tc_tokens", heads, kv_heads)


def attention_prefill_tc(q: torch.Tensor, kv_pool: torch.Tensor, out: torch.Tensor,
                         positions: torch.Tensor, tok_seq: torch.Tensor, block_table: torch.Tensor,
                         tile_tok0: torch.Tensor, tile_ntok: torch.Tensor, window: int | None,
                         scale: float, gate: torch.Tensor | None = None, nsplit: int = 1,
                         keep_first: int = 0, sink: bool = False, gate_by_element: bool = False) -> None:
    """``attention_prefill_mma`` on tcgen05.mma with the accumulators in tensor memory, for tiles
    of ``attention_prefill_tc_tokens`` tokens of one sequence; writes the tiles' rows of ``out``
    (gated like ``attention_prefill_mma``'s; ``keep_first``, ``sink``, ``gate_by_element`` as
    there). ``nsplit`` > 1: that many CTAs share each tile's keys and the last one to finish
    merges their shares (through scratch memory that this function allocates): for steps with
    few tiles behind long contexts."""
    _cuda(q, kv_pool, out, positions, tok_seq, block_table, tile_tok0, tile_ntok)
    T, H, D, Hkv, P = _check_attention(q, kv_pool, "attention_prefill_tc")
    g_ptr, ldg, mode = _gate_options(gate, gate_by_element, T, H, D, "attention_prefill_tc")
    n_tiles = tile_tok0.numel()
    nsplit = max(1, int(nsplit))
    scratch = tickets = None
    if nsplit > 1 and n_tiles:
        scratch = torch.empty(n_tiles * Hkv * nsplit * (128 * D + 256), dtype=torch.float32, device=q.device)
        tickets = _decode_tickets(n_tiles * Hkv, q.device)
    _lib.call("tk_attn_prefill_tc_opt", _ptr(q), _ptr(kv_pool), _ptr(out), _ptr(_i32(positions, "positions")),
              _ptr(_i32(tok_seq, "tok_seq")), _ptr(_i32(block_table, "block_table")),
              block_table.stride(0), _ptr(_i32(tile_tok0, "tile_tok0")),
              _ptr(_i32(tile_ntok, "tile_ntok")), n_tiles, H, Hkv, D, P, int(window or 0),
              float(scale), g_ptr, ldg, nsplit, _ptr(scratch), _ptr(tickets), int(keep_first), int(bool(sink)),
              mode, _stream())


def attention_prefill_tc_status() -> int:
    """0, or where a CTA of the tcgen05 prefill kernel gave up waiting since the last call."""
    return _lib.call("tk_attn_prefill_tc_status")


def attention_decode_mma(q: torch.Tensor, kv_pool: torch.Tensor, out: torch.Tensor,
                         positions: torch.Tensor, tok_seq: torch.Tensor, block_table: torch.Tensor,
                         tok_index: torch.Tensor | None, window: int | None, scale: float,
                         nsplit: int, gate: torch.Tensor | None = None, keep_first: int = 0,
                         sink: bool = False, gate_by_element: bool = False) -> None:
    """Tensor-core attention for sequences that bring one token (``tok_index``: their rows in
    the packed batch; None: every row of ``q`` is one, in order, which spares the kernel a
    lookup), each split ``nsplit`` ways over its keys; partial results go through scratch memory
    that this function allocates and a merge kernel. Writes those rows of ``out`` [T, H, D]
    (gated like ``attention_prefill_mma``'s)."""
    _cuda(q, kv_pool, out, positions, tok_seq, block_table, tok_index)
    T, H, D, Hkv, P = _check_attention(q, kv_pool, "attention_decode_mma")
    g_ptr, ldg, mode = _gate_options(gate, gate_by_element, T, H, D, "attention_decode_mma")
    n = tok_index.numel() if tok_index is not None else T
    scratch = None
    if nsplit > 1:
        scratch = torch.empty(n * H * nsplit * (D + 2), dtype=torch.float32, device=q.device)
    _lib.call("tk_attn_decode_mma_opt", _ptr(q), _ptr(kv_pool), _ptr(out), _ptr(_i32(positions, "positions")),
              _ptr(_i32(tok_seq, "tok_seq")), _ptr(_i32(block_table, "block_table")),
              block_table.stride(0), _ptr(_i32(tok_index, "tok_index") if tok_index is not None else None),
              n, H, Hkv, D, P, int(window or 0), float(scale), int(nsplit), _ptr(scratch), g_ptr, ldg,
              int(keep_first), int(bool(sink)), mode, _stream())


def attention_decode_fused_supported(heads: int, kv_heads: int, head_dim: int, rotary: int,
                                     dtype: torch.dtype) -> bool:
    """Whether ``attention_decode_fused`` takes this shape and rotary width."""
    return dtype == torch.bfloat16 and bool(
        _lib.call("tk_attn_decode_fused_supported", heads, kv_heads, head_dim, rotary))


# per device: [n * kv_heads] zeros the fused decode kernel counts finished splits in and zeroes
# again; a buffer that a captured step may point at is never freed, only outgrown
_tickets: dict = {}
_tickets_outgrown: list = []


def _decode_tickets(n: int, device: torch.device) -> torch.Tensor:
    have = _tickets.get(device)
    if have is None or have.numel() < n:
        if have is not None:
            _tickets_outgrown.append(have)
        have = _tickets[device] = torch.zeros(max(n, 4096), dtype=torch.int32, device=device)
    return have


def clear_tickets() -> None:
    """Put the ticket counters back to zero. The kernels that use them leave them at zero; one
    that gave up on a barrier half way may not have, and the next launch must not inherit that."""
    for t in list(_tickets.values()) + _tickets_outgrown:
        t.zero_()


def attention_decode_fused(qkv: torch.Tensor, kv_pool: torch.Tensor, q_norm: torch.Tensor | None,
                           k_norm: torch.Tensor | None, eps: float, inv_freq: torch.Tensor,
                           gate: torch.Tensor | None, positions: torch.Tensor, tok_seq: torch.Tensor,
                           block_table: torch.Tensor, heads: int, kv_heads: int, window: int | None,
                           scale: float, nsplit: int, write_kv: bool = True,
                           carveout: int = -1, general: bool = False, cs_mult: float = 1.0,
                           interleaved: bool = False, v_is_k: bool = False, keep_first: int = 0,
                           sink: bool = False, gate_by_element: bool = False) -> torch.Tensor:
    """A decode step's attention in one kernel, for sequences that bring one token each (row i of
    ``qkv`` is sequence i's): from the raw projection rows ``qkv`` [T, >= (H + 2 Hkv) D] (q heads,
    k heads, v heads; rows may be strided) through q/k norm, the rotate-half rotation by
    ``position * inv_freq`` [R / 2], the write of the new keys and values into ``kv_pool``
    [pages, 2, Hkv, P, D], attention over the cache split ``nsplit`` ways, the merge of the splits
    and the per-head gate ``gate`` [T, H] (a strided view; None: no gate) to the heads' outputs
    [T, H, D]. ``write_kv`` False: the layer reads a cache that another layer wrote this step and
    ``qkv`` holds queries only. ``carveout``: the share of an SM's memory, in percent of the most,
    that the launch prefers as shared memory (-1: the driver's choice). ``nsplit`` is cut to what
    the kernel's merge can hold.
    ``general``: the kernel's general form, without head norms: cos and sin are multiplied by
    ``cs_mult`` and not rounded, columns pair (2i, 2i + 1) when ``interleaved``, ``qkv`` holds no
    value heads when ``v_is_k`` (a key as projected is its value), ``keep_first`` positions stay
    visible behind the window, ``sink`` adds one to the softmax's denominator, and with
    ``gate_by_element`` the gate is [T, H * D], applied to the 32-bit output before its one rounding."""
    _cuda(qkv, kv_pool, q_norm, k_norm, inv_freq, gate, positions, tok_seq, block_table)
    T = qkv.shape[0]
    _, two, Hkv, P, D = kv_pool.shape
    need = (heads + ((1 if v_is_k else 2) * Hkv if write_kv else 0)) * D
    if (two != 2 or Hkv != kv_heads or qkv.dtype != torch.bfloat16 or kv_pool.dtype != torch.bfloat16
            or qkv.stride(1) != 1 or qkv.shape[1] < need or not kv_pool.is_contiguous()):
        raise KernelError("attention_decode_fused: qkv [T, >= (H + 2 Hkv) D] with contiguous rows and "
                          "kv_pool [pages, 2, Hkv, P, D], both bfloat16")
    gate_cols = heads * D if gate_by_element else heads
    if gate is not None and (gate.dtype != torch.bfloat16 or gate.shape != (T, gate_cols) or gate.stride(1) != 1):
        raise KernelError(f"attention_decode_fused: gate must be a bfloat16 [T, {gate_cols}] view with unit "
                          "column stride")
    if not general and (interleaved or v_is_k or keep_first or sink or gate_by_element or cs_mult != 1.0):
        raise KernelError("attention_decode_fused: these options belong to the general form")
    R = 2 * inv_freq.numel()
    out = torch.empty(T, heads, D, dtype=torch.bfloat16, device=qkv.device)
    nsplit = max(1, min(int(nsplit), _lib.call("tk_attn_decode_fused_max_splits", heads, Hkv, D)))
    scratch = tickets = None
    if nsplit > 1:
        scratch = torch.empty(T * heads * nsplit * (D + 2), dtype=torch.float32, device=qkv.device)
        tickets = _decode_tickets(T * Hkv, qkv.device)
    _lib.call("tk_attn_decode_fused_opt", _ptr(qkv), qkv.stride(0), _ptr(kv_pool), _ptr(out),
              _ptr(_f32vec(q_norm, "q_norm", D)), _ptr(_f32vec(k_norm, "k_norm", D)), float(eps),
              _ptr(_f32vec(inv_freq, "inv_freq", R // 2)), R, _ptr(gate),
              gate.stride(0) if gate is not None else 0, _ptr(_i32(positions, "positions")),
              _ptr(_i32(tok_seq, "tok_seq")), _ptr(_i32(block_table, "block_table")), block_table.stride(0),
              T, heads, Hkv, D, P, int(window or 0), float(scale), int(nsplit), _ptr(scratch), _ptr(tickets),
              1 if write_kv else 0, int(carveout), int(bool(general)), float(cs_mult), int(bool(interleaved)),
              int(bool(v_is_k)), int(keep_first), int(bool(sink)),
              0 if gate is None else (2 if gate_by_element else 1), _stream())
    return out


def conv_min_tile(width: int) -> int:
    return _lib.call("tk_conv_min_tile", width)


def conv_gated(bcx: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None,
               state: torch.Tensor, cu: torch.Tensor, seq_ctx: torch.Tensor,
               seq_slot: torch.Tensor, tile_seq: torch.Tensor, tile_off: torch.Tensor,
               tile_n: torch.Tensor, block: int = 0, tile_cap: int = 0,
               tile_tok0: torch.Tensor | None = None) -> torch.Tensor:
    """Gated short conv of ``bcx`` [T, 3d] = (B | C | X): returns ``C * conv(B * X)`` [T, d] and
    replaces each sequence's row of ``state`` [slots, W-1, d]. ``weight`` [d, W] float32.
    ``block`` b > 0: a row of ``bcx`` holds runs of b channels of B, of C and of X in turn.
    ``tile_cap``: the most tokens a tile has, if the caller knows (up to 16 a faster kernel takes
    the call); every tile but a portion's last has at least W - 1 tokens. ``tile_tok0``: each
    tile's first token in the batch, if the caller has it (it spares that kernel a lookup)."""
    _cuda(bcx, weight, bias, state, cu, seq_ctx, seq_slot, tile_seq, tile_off, tile_n)
    T, three_d = bcx.shape
    d = three_d // 3
    W = weight.shape[1]
    if bcx.stride(1) != 1 or three_d != 3 * d:
        raise KernelError("conv_gated: bcx must be [T, 3d] with contiguous rows")
    if weight.dtype != torch.float32 or not weight.is_contiguous() or weight.shape[0] != d:
        raise KernelError("conv_gated: weight must be contiguous float32 [d, W]")
    if state.dtype != bcx.dtype or not state.is_contiguous() or tuple(state.shape[1:]) != (W - 1, d):
        raise KernelError(f"conv_gated: state {tuple(state.shape)} does not match [slots, {W - 1}, {d}]")
    out = torch.empty(T, d, dtype=bcx.dtype, device=bcx.device)
    _lib.call("tk_conv_gated", _ptr(bcx), bcx.stride(0), d, _ptr(weight), _ptr(_f32vec(bias, "conv bias", d)),
              _ptr(state), _ptr(out), _ptr(_i32(cu, "cu")), _ptr(_i32(seq_ctx, "seq_ctx")),
              _ptr(_i32(seq_slot, "seq_slot")), _ptr(_i32(tile_seq, "tile_seq")),
              _ptr(_i32(tile_off, "tile_off")), _ptr(_i32(tile_n, "tile_n")),
              _ptr(_i32(tile_tok0, "tile_tok0")) if tile_tok0 is not None else None, tile_seq.numel(), W,
              int(block), int(tile_cap), _dtype_code(bcx), _stream())
    return out


def gemm_skinny_conv(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, taps: torch.Tensor,
                     conv_bias: torch.Tensor | None, state: torch.Tensor, seq_ctx: torch.Tensor,
                     seq_slot: torch.Tensor, norm_eps: float = 0.0) -> torch.Tensor:
    """A gated short conv's in-projection with the conv in its epilogue, for a step whose tokens
    are one new token of a sequence each (decoding): ``x`` [M <= 16, K] bfloat16, ``w`` [3d, K]
    with rows in blocks of 24 (8 rows of B, of C and of X of the same 8 channels), ``bias`` in the
    same order; returns ``C * conv(B * X)`` [M, d] and moves each request's row of ``state``
    [slots, W-1, d] on by its token. ``seq_ctx``, ``seq_slot``: [M]. ``norm_eps`` > 0 (at most 8
    rows): ``x`` is an un-normed stream; see ``gemm_skinny``."""
    _cuda(x, w, bias, taps, conv_bias, state, seq_ctx, seq_slot)
    M, K = x.shape
    d, W = taps.shape
    if tuple(w.shape) != (3 * d, K) or not gemm_skinny_ok(x, w):
        raise KernelError(f"gemm_skinny_conv: x {tuple(x.shape)} against w {tuple(w.shape)} for {d} channels")
    if taps.dtype != torch.float32 or not taps.is_contiguous():
        raise KernelError("gemm_skinny_conv: taps must be contiguous float32 [d, W]")
    if state.dtype != torch.bfloat16 or not state.is_contiguous() or tuple(state.shape[1:]) != (W - 1, d):
        raise KernelError(f"gemm_skinny_conv: state {tuple(state.shape)} for width {W}, {d} channels")
    if seq_ctx.numel() < M or seq_slot.numel() < M:
        raise KernelError("gemm_skinny_conv: one sequence per token")
    out = torch.empty(M, d, dtype=x.dtype, device=x.device)
    _lib.call("tk_gemm_skinny_conv", _ptr(x), x.stride(0), _ptr(w), w.stride(0),
              _ptr(_f32vec(bias, "bias", 3 * d)), _ptr(out), d, M, d, K, _ptr(taps),
              _ptr(_f32vec(conv_bias, "conv bias", d)), _ptr(state), _ptr(_i32(seq_ctx, "seq_ctx")),
              _ptr(_i32(seq_slot, "seq_slot")), W, float(norm_eps), _stream())
    return out


def gemm(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
         out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``x @ w.T (+ bias)`` on the CUDA cores with 32-bit accumulation, any shape.
    ``x`` [M, K] (row stride free), ``w`` [N, K]; ``bias`` float32 [N]."""
    _cuda(x, w, bias)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or x.dtype != w.dtype or x.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError(f"gemm: x {tuple(x.shape)} {x.dtype} against w {tuple(w.shape)} {w.dtype}")
    out_dtype = out_dtype or x.dtype
    out = torch.empty(M, N, dtype=out_dtype, device=x.device)
    _lib.call("tk_gemm_simt", _ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(_f32vec(bias, "bias", N)),
              _ptr(out), N, M, N, K, _dtype_code(x), _dtype_code(out), _stream())
    return out


SKINNY_MAX_ROWS = 16


def gemm_skinny_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether ``gemm_skinny`` takes this product: bfloat16, at most 16 rows of ``x``, K and the
    row strides multiples of 8 elements, 16-byte aligned."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_cuda
            and 0 < x.shape[0] <= SKINNY_MAX_ROWS and x.shape[1] % 8 == 0
            and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


SKINNY_FUSED_ROWS = 8


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
                out_dtype: torch.dtype | None = None, swiglu: bool = False, norm_eps: float = 0.0,
                residual: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ w.T (+ bias)`` for at most 16 rows of ``x`` (decode): a weight-streaming kernel.
    ``swiglu``: the rows of ``w`` alternate in runs of 8 (8 gate rows, the 8 up rows of the same
    channels) and the result is ``silu(gate) * up`` of width ``N / 2``.
    The two halves of a residual add + RMSNorm, for at most 8 rows: ``norm_eps`` > 0: ``x`` is the
    un-normed stream and row r of the product is scaled by ``1 / sqrt(mean(x[r]^2) + norm_eps)``
    (the norm's weight is expected in ``w``'s columns); ``residual`` [M, N]: the result is
    ``residual + product`` (the product rounded to 16 bits first, the sum once)."""
    _cuda(x, w, bias, residual)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm_skinny: x {tuple(x.shape)} against w {tuple(w.shape)}")
    width = N // 2 if swiglu else N
    if residual is not None and (tuple(residual.shape) != (M, N) or residual.dtype != torch.bfloat16
                                 or residual.stride(1) != 1):
        raise KernelError(f"gemm_skinny: residual {tuple(residual.shape)} {residual.dtype} for a "
                          f"[{M}, {N}] bfloat16 result")
    out = torch.empty(M, width, dtype=out_dtype or x.dtype, device=x.device)
    _lib.call("tk_gemm_skinny", _ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(_f32vec(bias, "bias", N)),
              _ptr(out), width, M, N, K, _dtype_code(out), int(swiglu), float(norm_eps), _ptr(residual),
              residual.stride(0) if residual is not None else 0, _stream())
    return out


TC_MAX_TOKENS = 256


def gemm_tc_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether ``gemm_tc`` takes this product: bfloat16, at most 256 rows of ``x``, K and the row
    strides multiples of 8 elements, 16-byte aligned bases."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_cuda
            and 0 < x.shape[0] <= TC_MAX_TOKENS and x.shape[1] % 8 == 0
            and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
            out_dtype: torch.dtype | None = None, swiglu: bool = False,
            split_k: bool = True) -> torch.Tensor:
    """``x @ w.T (+ bias)`` through TMA, tcgen05.mma and tensor memory, the weight rows on the
    MMA's M axis (decode: up to 256 rows of ``x``). ``swiglu`` as in ``gemm_skinny``. ``split_k``:
    matrices with few rows may be split along K over a thread-block cluster."""
    _cuda(x, w, bias)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm_tc: x {tuple(x.shape)} against w {tuple(w.shape)}")
    width = N // 2 if swiglu else N
    out = torch.empty(M, width, dtype=out_dtype or x.dtype, device=x.device)
    _lib.call("tk_gemm_tc_decode", _ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(_f32vec(bias, "bias", N)),
              _ptr(out), width, M, N, K, _dtype_code(out), int(swiglu), int(split_k), _stream())
    return out


def gemm_tc_status() -> int:
    """0, or where a tensor-core GEMM gave up waiting on a barrier since the last call (the
    kernels bound every wait instead of hanging)."""
    return _lib.call("tk_gemm_tc_status")


def sample_status() -> int:
    """0, or 1 + the first row since the last call whose logits held no finite value (the sampler
    answered token 0 for it)."""
    return _lib.call("tk_sample_status")


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor,
           top_k: torch.Tensor, min_p: torch.Tensor, seed: torch.Tensor, step: torch.Tensor,
           out: torch.Tensor | None = None, scatter: tuple[torch.Tensor, torch.Tensor] | None = None
           ) -> torch.Tensor:
    """One token per row of ``logits`` [rows, V] float32; the parameters are per-row arrays.
    ``scatter`` = (index [rows] int32, target int32): also ``target[index[r]] = token``."""
    _cuda(logits, temperature, top_p, top_k, min_p, seed, step, out)
    rows, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 with contiguous rows")
    for name, t, dt in (("temperature", temperature, torch.float32), ("top_p", top_p, torch.float32),
                        ("min_p", min_p, torch.float32), ("top_k", top_k, torch.int32),
                        ("seed", seed, torch.int32), ("step", step, torch.int32)):
        if t.dtype != dt or t.numel() < rows or not t.is_contiguous():
            raise KernelError(f"sample: {name} must be a contiguous {dt} array of {rows}")
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    idx, target = scatter if scatter is not None else (None, None)
    if scatter is not None:
        _cuda(idx, target)
        _i32(idx, "scatter index"), _i32(target, "scatter target")
    _lib.call("tk_sample", _ptr(logits), logits.stride(0), rows, V, _ptr(temperature), _ptr(top_p),
              _ptr(top_k), _ptr(min_p), _ptr(seed), _ptr(step), _ptr(out), _ptr(idx), _ptr(target),
              _stream())
    return out


# ---- several copies of the residual stream, hashed bigram embedding, input convolution --------

HYPER_MAX_STREAMS = 8
CANON_MAX_TAPS = 8


def embed_bigram_norm(table: torch.Tensor, bigram: torch.Tensor | None, norm_w: torch.Tensor | None, eps: float,
                      ids: torch.Tensor, select: tuple | None, tok_seq: torch.Tensor, cu_seqlens: torch.Tensor,
                      seq_ctx: torch.Tensor, seq_slot: torch.Tensor, prev_state: torch.Tensor | None,
                      copies: int, buckets: int = 0, mul_prev: int = 0, mul_cur: int = 0) -> torch.Tensor:
    """``rmsnorm(table[id] + bigram[(prev * mul_prev + id * mul_cur) % buckets]) * norm_w`` in 32-bit,
    written ``copies`` times side by side: float32 [T, copies * width]. A sequence's first token
    takes bigram row ``buckets``; the previous token of a portion's first token comes from
    ``prev_state`` (int32 [slots, 1]), which then takes the portion's last id. ``select``:
    ``(use_prev, last_token, tok_slot)``, token r reads ``last_token[tok_slot[r]]`` where
    ``use_prev[r]`` is set instead of ``ids[r]``."""
    _cuda(table, bigram, norm_w, ids, tok_seq, cu_seqlens, seq_ctx, seq_slot, prev_state)
    T, width = ids.numel(), table.shape[1]
    if not table.is_contiguous() or (bigram is not None and (not bigram.is_contiguous() or bigram.dtype != table.dtype
                                                             or tuple(bigram.shape) != (buckets + 1, width))):
        raise KernelError("embed_bigram_norm: tables must be contiguous, of one type, the bigram [buckets + 1, width]")
    if bigram is not None and (prev_state is None or prev_state.dtype != torch.int32):
        raise KernelError("embed_bigram_norm: the bigram needs an int32 state")
    use_prev, last_token, tok_slot = select if select is not None else (None, None, None)
    out = torch.empty(T, copies * width, dtype=torch.float32, device=table.device)
    _lib.call("tk_embed_bigram_norm", _ptr(table), _ptr(bigram), _ptr(_f32vec(norm_w, "norm weight", width)),
              float(eps), _ptr(_i32(ids, "ids")), _ptr(use_prev), _ptr(last_token), _ptr(tok_slot),
              _ptr(_i32(tok_seq, "tok_seq")), _ptr(_i32(cu_seqlens, "cu_seqlens")), _ptr(_i32(seq_ctx, "seq_ctx")),
              _ptr(_i32(seq_slot, "seq_slot")), _ptr(prev_state), _ptr(out), T, int(copies), width, table.shape[0],
              int(buckets), int(mul_prev), int(mul_cur), _dtype_code(table), _stream())
    return out


def hc_mix_norm(streams: torch.Tensor, y: torch.Tensor | None, mix: torch.Tensor | None, out_w: torch.Tensor | None,
                in_w: torch.Tensor | None, norm_w: torch.Tensor | None, eps: float, n_streams: int,
                out_dtype: torch.dtype, keep32: bool, conv: tuple | None = None) -> torch.Tensor | None:
    """Streams ``[T, S * width]`` float32, in place: ``x'_t = sum_s mix[s, t] x_s + out_w[t] * y``
    (when ``y`` [T, width] is given; ``mix`` None: identity, ``out_w`` None: ones), then
    ``h = rmsnorm(sum_s in_w[s] x'_s) * norm_w`` (``in_w`` None: ones): float32 when ``keep32``, else
    ``out_dtype``. ``norm_w`` None: only the write, returns None. ``conv``: ``(taps, state, seq_ctx,
    seq_slot)`` in a step where every sequence brings one token: the input convolution
    (``canon_conv``) and its state update in the same kernel; the result is in ``out_dtype``."""
    _cuda(streams, y, mix, out_w, in_w, norm_w)
    taps, state, seq_ctx, seq_slot = conv if conv is not None else (None, None, None, None)
    if conv is not None:
        keep32 = False
        if taps.dtype != torch.float32 or not taps.is_contiguous() or (
                state is not None and (state.dtype != torch.float32 or not state.is_contiguous())):
            raise KernelError("hc_mix_norm: taps and state are contiguous float32 tensors")
    S = int(n_streams)
    T, width = streams.shape[0], streams.shape[1] // S
    if streams.dtype != torch.float32 or not streams.is_contiguous() or streams.shape[1] != S * width:
        raise KernelError("hc_mix_norm: the streams are a contiguous float32 [T, S * width] tensor")
    if y is not None and (tuple(y.shape) != (T, width) or y.stride(1) != 1 or y.dtype != out_dtype):
        raise KernelError(f"hc_mix_norm: y {tuple(y.shape)} {y.dtype} for [{T}, {width}] {out_dtype}")
    h = None
    if norm_w is not None:
        h = torch.empty(T, width, dtype=torch.float32 if keep32 else out_dtype, device=streams.device)
    code = F32 if out_dtype == torch.float32 else BF16
    _lib.call("tk_hc_mix_norm", _ptr(streams), _ptr(y), y.stride(0) if y is not None else 0,
              _ptr(_f32vec(mix, "mix", S * S)), _ptr(_f32vec(out_w, "out", S)), _ptr(_f32vec(in_w, "in", S)),
              _ptr(_f32vec(norm_w, "norm weight", width)), float(eps), _ptr(h if keep32 else None),
              _ptr(None if keep32 else h), T, S, width, code, _ptr(taps), _ptr(state), _ptr(seq_ctx), _ptr(seq_slot),
              taps.shape[1] if taps is not None else 0, _stream())
    return h


def canon_conv(h: torch.Tensor, taps: torch.Tensor, state: torch.Tensor | None, cu_seqlens: torch.Tensor,
               seq_ctx: torch.Tensor, seq_slot: torch.Tensor, tiles: tuple, out_dtype: torch.dtype) -> torch.Tensor:
    """``o_t = h_t + sum_j taps[:, j] h_(t - K + 1 + j)`` within each sequence (zeros before its start),
    ``h`` float32 [T, width], ``taps`` float32 [width, K]; the last K - 1 rows of ``h`` of every
    sequence are kept in ``state`` (float32 [slots, K - 1, width]). ``tiles``: ``ctx.tiles(size)`` with
    size >= K - 1."""
    _cuda(h, taps, state, cu_seqlens, seq_ctx, seq_slot, *tiles)
    T, width = h.shape
    K = taps.shape[1]
    if h.dtype != torch.float32 or not h.is_contiguous() or taps.dtype != torch.float32 or not taps.is_contiguous():
        raise KernelError("canon_conv: h and taps are contiguous float32 tensors")
    if K > 1 and (state is None or state.dtype != torch.float32 or tuple(state.shape[1:]) != (K - 1, width)
                  or not state.is_contiguous()):
        raise KernelError(f"canon_conv: the state is float32 [slots, {K - 1}, {width}]")
    seq, tok0, off, n = tiles
    out = torch.empty(T, width, dtype=out_dtype, device=h.device)
    _lib.call("tk_canon_conv", _ptr(h), _ptr(taps), _ptr(state), _ptr(_i32(cu_seqlens, "cu_seqlens")),
              _ptr(_i32(seq_ctx, "seq_ctx")), _ptr(_i32(seq_slot, "seq_slot")), _ptr(_i32(seq, "tile_seq")),
              _ptr(_i32(tok0, "tile_tok0")), _ptr(_i32(off, "tile_off")), _ptr(_i32(n, "tile_n")), seq.numel(),
              _ptr(out), K, width, F32 if out_dtype == torch.float32 else BF16, _stream())
    return out


# ---- attention over a cache of latents ----------------------------------------------------------

def latent_prepare(proj: torch.Tensor, wq: torch.Tensor, wkv: torch.Tensor, eps: float, freq: torch.Tensor,
                   positions: torch.Tensor, tok_seq: torch.Tensor, block_table: torch.Tensor | None,
                   cache: torch.Tensor | None, q_rank: int, rank: int, rot_dim: int) -> torch.Tensor:
    """From the down-projection's rows ``[q latent | kv latent | rotated key part | ...]``: the normed
    query latent [T, q_rank] (returned), and into ``cache`` [pages, P, rank + rot_dim], at each token's
    position, the normed kv latent and the key part rotated by ``position * freq`` (pairs (2i, 2i+1),
    ``2 len(freq)`` columns). ``cache`` None: the rows hold the query latent only (a layer that reads
    another layer's cache)."""
    _cuda(proj, wq, wkv, freq, positions, tok_seq, block_table, cache)
    T = proj.shape[0]
    if cache is None:
        if proj.stride(1) != 1 or proj.shape[1] < q_rank:
            raise KernelError("latent_prepare: projection rows are too short")
        cq = torch.empty(T, q_rank, dtype=proj.dtype, device=proj.device)
        _lib.call("tk_latent_prepare", _ptr(proj), proj.stride(0), _ptr(_f32vec(wq, "q latent norm", q_rank)), None,
                  float(eps), _ptr(freq), _ptr(_i32(positions, "positions")), _ptr(_i32(tok_seq, "tok_seq")), None, 0,
                  _ptr(cq), None, T, q_rank, rank, rot_dim, 2 * freq.numel(), 1, _dtype_code(proj), _stream())
        return cq
    if proj.stride(1) != 1 or proj.shape[1] < q_rank + rank + rot_dim:
        raise KernelError("latent_prepare: projection rows are too short")
    if (cache.dim() != 3 or cache.shape[2] != rank + rot_dim or cache.dtype != proj.dtype
            or not cache.is_contiguous()):
        raise KernelError(f"latent_prepare: the cache is [pages, page, {rank + rot_dim}] {proj.dtype}")
    cq = torch.empty(T, q_rank, dtype=proj.dtype, device=proj.device)
    _lib.call("tk_latent_prepare", _ptr(proj), proj.stride(0), _ptr(_f32vec(wq, "q latent norm", q_rank)),
              _ptr(_f32vec(wkv, "kv latent norm", rank)), float(eps), _ptr(freq), _ptr(_i32(positions, "positions")),
              _ptr(_i32(tok_seq, "tok_seq")), _ptr(_i32(block_table, "block_table")), block_table.stride(0),
              _ptr(cq), _ptr(cache), T, q_rank, rank, rot_dim, 2 * freq.numel(), cache.shape[1],
              _dtype_code(proj), _stream())
    return cq


def latent_rotate_q(q: torch.Tensor, freq: torch.Tensor, positions: torch.Tensor, heads: int, dim: int,
                    rot_dim: int) -> torch.Tensor:
    """In place on ``q`` [T, heads * (dim + rot_dim)]: the last ``rot_dim`` columns of every head rotated."""
    _cuda(q, freq, positions)
    if not q.is_contiguous() or q.shape[1] != heads * (dim + rot_dim):
        raise KernelError("latent_rotate_q: q must be contiguous [T, heads * (dim + rot_dim)]")
    _lib.call("tk_latent_rotate_q", _ptr(q), _ptr(freq), _ptr(_i32(positions, "positions")), q.shape[0], heads, dim,
              rot_dim, 2 * freq.numel(), _dtype_code(q), _stream())
    return q


def attention_latent_rows() -> int:
    return _lib.call("tk_attn_latent_rows")


def attention_latent_mma_supported(dim: int, rank: int, rot_dim: int, dtype: torch.dtype) -> bool:
    """Whether the tensor-core form of the latent attention takes these sizes (else the general
    kernel does): bfloat16, a latent of a multiple of 32 up to 512, a rotated part of a multiple of 16."""
    return dtype == torch.bfloat16 and bool(_lib.call("tk_attn_latent_mma_supported", int(dim), int(rank), int(rot_dim)))


def attention_latent_tokens(heads: int, dim: int, rank: int, rot_dim: int, dtype: torch.dtype) -> int:
    """Tokens of one sequence a tile of the latent attention holds (rows of a tile / heads, at least one)."""
    rows = (_lib.call("tk_attn_latent_mma_rows") if attention_latent_mma_supported(dim, rank, rot_dim, dtype)
            else _lib.call("tk_attn_latent_rows"))
    return max(1, rows // heads)


ATTENTION_LATENT_MAX_RANK = 512


def attention_latent(q_lat: torch.Tensor, q: torch.Tensor, cache: torch.Tensor, positions: torch.Tensor,
                     tok_seq: torch.Tensor, block_table: torch.Tensor, tile_tok0: torch.Tensor,
                     tile_ntok: torch.Tensor, tokens_per_tile: int, heads: int, dim: int, rot_dim: int,
                     window: int | None, scale: float, nsplit: int = 1, rows16: bool = False) -> torch.Tensor:
    """Windowed causal attention over the latent cache [pages, P, R + rot_dim]: scores
    ``(q_lat[h, t] . c_j + q[t, h, dim:] . k_rot_j) * scale``, output ``sum_j p_j c_j`` as [heads, T, R].
    ``nsplit`` > 1 (tensor-core form only): that many CTAs share a tile's keys and a second kernel
    merges their shares, for steps with few tiles behind long contexts. ``rows16`` (with one token a
    tile): the tensor-core form with all of its warps on one group of 16 rows (a token's heads)."""
    _cuda(q_lat, q, cache, positions, tok_seq, block_table, tile_tok0, tile_ntok)
    H, T, R = q_lat.shape
    if (H != heads or not q_lat.is_contiguous() or not q.is_contiguous() or q.shape[0] != T
            or q.shape[1] != heads * (dim + rot_dim) or cache.shape[2] != R + rot_dim or cache.dtype != q.dtype
            or q_lat.dtype != q.dtype):
        raise KernelError("attention_latent: q / cache layouts do not match")
    out = torch.empty(H, T, R, dtype=q.dtype, device=q.device)
    if attention_latent_mma_supported(dim, R, rot_dim, q.dtype) and tokens_per_tile <= _lib.call("tk_attn_latent_mma_rows"):
        _lib.call("tk_attn_latent_mma", _ptr(q_lat), _ptr(q), _ptr(cache), _ptr(out), _ptr(_i32(positions, "positions")),
                  _ptr(_i32(tok_seq, "tok_seq")), _ptr(_i32(block_table, "block_table")), block_table.stride(0),
                  _ptr(_i32(tile_tok0, "tile_tok0")), _ptr(_i32(tile_ntok, "tile_ntok")), tile_tok0.numel(),
                  int(tokens_per_tile), T, H, dim, R, rot_dim, cache.shape[1], int(window or 0), float(scale), 1, None,
                  None, int(bool(rows16)), _stream()) if nsplit <= 1 else _attention_latent_split(
                      q_lat, q, cache, out, positions, tok_seq, block_table, tile_tok0, tile_ntok, tokens_per_tile, dim,
                      rot_dim, window, scale, int(nsplit), rows16)
        return out
    _lib.call("tk_attn_latent", _ptr(q_lat), _ptr(q), _ptr(cache), _ptr(out), _ptr(_i32(positions, "positions")),
              _ptr(_i32(tok_seq, "tok_seq")), _ptr(_i32(block_table, "block_table")), block_table.stride(0),
              _ptr(_i32(tile_tok0, "tile_tok0")), _ptr(_i32(tile_ntok, "tile_ntok")), tile_tok0.numel(),
              int(tokens_per_tile), T, H, dim, R, rot_dim, cache.shape[1], int(window or 0), float(scale),
              _dtype_code(q), _stream())
    return out


def _attention_latent_split(q_lat, q, cache, out, positions, tok_seq, block_table, tile_tok0, tile_ntok,
                            tokens_per_tile, dim, rot_dim, window, scale, nsplit, rows16=False) -> None:
    H, T, R = q_lat.shape
    part_o = torch.empty(nsplit, H, T, R, dtype=torch.float32, device=q.device)
    part_ml = torch.empty(nsplit, H, T, 2, dtype=torch.float32, device=q.device)
    _lib.call("tk_attn_latent_mma", _ptr(q_lat), _ptr(q), _ptr(cache), _ptr(out), _ptr(positions), _ptr(tok_seq),
              _ptr(block_table), block_table.stride(0), _ptr(tile_tok0), _ptr(tile_ntok), tile_tok0.numel(),
              int(tokens_per_tile), T, H, dim, R, rot_dim, cache.shape[1], int(window or 0), float(scale), nsplit,
              _ptr(part_o), _ptr(part_ml), int(bool(rows16)), _stream())
    _lib.call("tk_attn_latent_merge", _ptr(part_o), _ptr(part_ml), _ptr(out), H * T, R, nsplit, _stream())


def head_gate_transpose(x: torch.Tensor, gate: torch.Tensor | None) -> torch.Tensor:
    """``out[t, h, :] = x[h, t, :] * sigmoid(gate[t, h])``: [H, T, D] -> [T, H, D]; ``gate`` may be a
    column block of wider rows."""
    _cuda(x, gate)
    H, T, D = x.shape
    if not x.is_contiguous() or (gate is not None and (gate.stride(1) != 1 or gate.dtype != x.dtype
                                                       or tuple(gate.shape) != (T, H))):
        raise KernelError("head_gate_transpose: x contiguous [H, T, D], gate [T, H] of its type")
    out = torch.empty(T, H, D, dtype=x.dtype, device=x.device)
    _lib.call("tk_head_gate_transpose", _ptr(x), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(out),
              T, H, D, _dtype_code(x), _stream())
    return out


# ---- mixture of experts --------------------------------------------------------------------------

def moe_route(logits: torch.Tensor, experts: int, top: int, scale: float, has_gate: bool):
    """From float32 router rows ``[T, >= experts (+ 1)]``: the ``top`` experts of the largest
    softmax scores (int32 [T, top]), their scores over their sum times ``scale`` (float32 [T, top]),
    and ``sigmoid`` of column ``experts`` (float32 [T]) when ``has_gate``."""
    _cuda(logits)
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("moe_route: router rows are float32 with contiguous columns")
    T = logits.shape[0]
    idx = torch.empty(T, top, dtype=torch.int32, device=logits.device)
    w = torch.empty(T, top, dtype=torch.float32, device=logits.device)
    gate = torch.empty(T, dtype=torch.float32, device=logits.device) if has_gate else None
    _lib.call("tk_moe_route", _ptr(logits), logits.stride(0), T, int(experts), int(top), float(scale),
              int(bool(has_gate)), _ptr(idx), _ptr(w), _ptr(gate), _stream())
    return idx, w, gate


def gemm_grouped_tile() -> int:
    return _lib.call("tk_gemm_grouped_tile")


def moe_sort(idx: torch.Tensor, experts: int, tile: int, ends: bool = False):
    """(token, k) pairs grouped by expert, each expert's rows padded to whole tiles:
    ``row_token`` [rows] (-1: padding), ``pair_row`` [T * top], ``tile_expert`` [rows / tile] (-1: unused).
    ``rows`` is the bound ``T * top + min(experts, T * top) * (tile - 1)`` rounded up to whole tiles.
    ``ends``: also ``expert_end`` [experts] (int32), the row after each expert's padded block."""
    _cuda(idx)
    T, top = idx.shape
    pairs = T * top
    cap = -(-(pairs + min(experts, pairs) * (tile - 1)) // tile) * tile
    row_token = torch.empty(cap, dtype=torch.int32, device=idx.device)
    pair_row = torch.empty(pairs, dtype=torch.int32, device=idx.device)
    tile_expert = torch.empty(cap // tile, dtype=torch.int32, device=idx.device)
    expert_end = torch.empty(experts, dtype=torch.int32, device=idx.device) if ends else None
    _lib.call("tk_moe_sort", _ptr(_i32(idx, "idx")), pairs, top, int(experts), int(tile), cap, _ptr(row_token),
              _ptr(pair_row), _ptr(tile_expert), _ptr(expert_end), _stream())
    if ends:
        return row_token, pair_row, tile_expert, expert_end
    return row_token, pair_row, tile_expert


def gather_rows_or_zero(table: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    """``out[r] = table[index[r]]``, a row of zeros where ``index[r]`` is negative."""
    _cuda(table, index)
    if not table.is_contiguous():
        raise KernelError("gather_rows_or_zero: the table must be contiguous")
    out = torch.empty(index.numel(), table.shape[1], dtype=table.dtype, device=table.device)
    _lib.call("tk_gather_rows_or_zero", _ptr(table), _ptr(_i32(index, "index")), _ptr(out), index.numel(),
              table.shape[1], _dtype_code(table), _stream())
    return out


def gemm_grouped_tiles(a_dtype: torch.dtype, n: int, k: int, rows: int) -> int:
    """Rows of a tile of the grouped product, which the sort of the rows has to use too: 64, or, in
    the tensor-core form when there are many rows, 128."""
    big = a_dtype == torch.bfloat16 and k % 8 == 0 and n % 8 == 0 and rows >= 2048
    return 128 if big else _lib.call("tk_gemm_grouped_tile")


def gemm_grouped(a: torch.Tensor, w: torch.Tensor, tile_group: torch.Tensor, row_index: torch.Tensor | None,
                 rows: int, act: bool | str = False, tile: int = 64) -> torch.Tensor:
    """``out[m] = act(a[row_index[m]] @ w[g].T)`` with ``g = tile_group[m // tile]``; ``w`` [G, N, K];
    a row index of -1 reads zeros, a tile group of -1 is skipped (its rows are not written). ``act``
    True: ``relu(v)^2``; ``"swiglu8"`` (tensor-core form only, see ``gemm_grouped_fuses_swiglu``): the
    rows of ``w[g]`` are gate and up rows alternating in runs of 8 and ``out`` [rows, N / 2] is
    ``silu(gate) * up``."""
    _cuda(a, w, tile_group, row_index)
    G, N, K = w.shape
    if a.dtype != w.dtype or a.stride(1) != 1 or not w.is_contiguous() or a.shape[1] != K:
        raise KernelError(f"gemm_grouped: a {tuple(a.shape)} {a.dtype} against w {tuple(w.shape)} {w.dtype}")
    if act == "swiglu8":
        if not gemm_grouped_fuses_swiglu(a, w):
            raise KernelError("gemm_grouped: the gated activation in the epilogue is the tensor-core form's")
        out = torch.empty(rows, N // 2, dtype=a.dtype, device=a.device)
        _lib.call("tk_gemm_grouped_mma", _ptr(a), a.stride(0), 0, _ptr(row_index), _ptr(w), K, N * K,
                  _ptr(_i32(tile_group, "tile_group")), _ptr(out), N // 2, 0, rows, N, K, G, 2, int(tile), None, 0,
                  _stream())
        return out
    out = torch.empty(rows, N, dtype=a.dtype, device=a.device)
    if _grouped_mma_ok(a, w, N, K):
        _lib.call("tk_gemm_grouped_mma", _ptr(a), a.stride(0), 0, _ptr(row_index), _ptr(w), K, N * K,
                  _ptr(_i32(tile_group, "tile_group")), _ptr(out), N, 0, rows, N, K, G, int(bool(act)), int(tile),
                  None, 0, _stream())
        return out
    if tile != _lib.call("tk_gemm_grouped_tile"):
        raise KernelError(f"gemm_grouped: tiles of {tile} rows are the tensor-core form's")
    _lib.call("tk_gemm_grouped_simt", _ptr(a), a.stride(0), 0, _ptr(row_index), _ptr(w), K, N * K,
              _ptr(_i32(tile_group, "tile_group")), _ptr(out), N, 0, rows, N, K, G, int(bool(act)), _dtype_code(a),
              _stream())
    return out


def gemm_grouped_fuses_swiglu(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether ``gemm_grouped(a, w, ..., act="swiglu8")`` is built for these operands."""
    N, K = w.shape[-2:]
    return N % 16 == 0 and _grouped_mma_ok(a, w, N, K)


def _grouped_mma_ok(a: torch.Tensor, w: torch.Tensor, N: int, K: int) -> bool:
    """Whether the tensor-core form of the grouped / batched product takes these operands: bfloat16,
    K, N and the row strides in whole 16-byte chunks, 16-byte aligned."""
    return (a.dtype == torch.bfloat16 and K % 8 == 0 and N % 8 == 0 and a.stride(-2) % 8 == 0
            and w.stride(-2) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_batched(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None,
                 gate: torch.Tensor | None = None) -> torch.Tensor:
    """``out[g] = a[g] @ w[g].T``: ``a`` [G, M, K] (any strides with contiguous columns), ``w``
    [G, N, K] likewise, ``out`` [G, M, N] (any strides too: a view of [M, G, N] works). 32-bit FMA on
    the CUDA cores, or mma.sync for bfloat16 in whole 16-byte chunks. ``gate`` [M, G] (tensor-core
    form only): row m of ``out[g]`` times ``sigmoid(gate[m, g])``."""
    _cuda(a, w, out, gate)
    G, M, K = a.shape
    N = w.shape[1]
    if a.dtype != w.dtype or a.stride(2) != 1 or w.stride(2) != 1 or w.shape[0] != G or w.shape[2] != K:
        raise KernelError(f"gemm_batched: a {tuple(a.shape)} {a.dtype} against w {tuple(w.shape)} {w.dtype}")
    if out is None:
        out = torch.empty(G, M, N, dtype=a.dtype, device=a.device)
    if out.stride(2) != 1:
        raise KernelError("gemm_batched: out needs contiguous columns")
    if (_grouped_mma_ok(a, w, N, K) and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and out.stride(1) % 2 == 0
            and out.stride(0) % 2 == 0 and out.data_ptr() % 4 == 0):
        if gate is not None and (gate.dtype != torch.bfloat16 or gate.stride(1) != 1 or tuple(gate.shape) != (M, G)):
            raise KernelError("gemm_batched: the gate is bfloat16 [M, G] with contiguous columns")
        _lib.call("tk_gemm_grouped_mma", _ptr(a), a.stride(1), a.stride(0), None, _ptr(w), w.stride(1), w.stride(0),
                  None, _ptr(out), out.stride(1), out.stride(0), M, N, K, G, 0, 64 if M <= 64 else 128, _ptr(gate),
                  gate.stride(0) if gate is not None else 0, _stream())
        return out
    if gate is not None:
        raise KernelError("gemm_batched: the row gate needs the tensor-core form (bfloat16, 16-byte chunks)")
    _lib.call("tk_gemm_grouped_simt", _ptr(a), a.stride(1), a.stride(0), None, _ptr(w), w.stride(1), w.stride(0),
              None, _ptr(out), out.stride(1), out.stride(0), M, N, K, G, 0, _dtype_code(a), _stream())
    return out


def moe_combine(y: torch.Tensor, pair_row: torch.Tensor, w: torch.Tensor, shared: torch.Tensor | None,
                gate: torch.Tensor | None) -> torch.Tensor:
    """``out[t] = sum_k w[t, k] * y[pair_row[t * top + k]] + gate[t] * shared[t]`` (32-bit sum)."""
    _cuda(y, pair_row, w, shared, gate)
    T, top = w.shape
    width = y.shape[1]
    if not y.is_contiguous() or (shared is not None and (not shared.is_contiguous() or shared.dtype != y.dtype)):
        raise KernelError("moe_combine: contiguous inputs of one type")
    out = torch.empty(T, width, dtype=y.dtype, device=y.device)
    _lib.call("tk_moe_combine", _ptr(y), _ptr(_i32(pair_row, "pair_row")), _ptr(w), _ptr(shared), _ptr(gate),
              _ptr(out), T, top, width, _dtype_code(y), _stream())
    return out


def relu2(x: torch.Tensor) -> torch.Tensor:
    """In place ``x = relu(x) ** 2``."""
    _cuda(x)
    if not x.is_contiguous():
        raise KernelError("relu2: x must be contiguous")
    _lib.call("tk_relu2", _ptr(x), x.numel(), _dtype_code(x), _stream())
    return x


# ---- sequence convolutions, pointwise-weight attention, recurrent state updates ----------------------

SEQ_CONV_MAX_TAPS = 8
_SEQ_CONV_RESIDENT = 148 * 4      # blocks of the sequence convolution that run at once


def seq_conv_tile(base: int, tokens: int, channels: int) -> int:
    """The tile length for ``seq_conv`` on a step of ``tokens`` tokens: ``base``, doubled (up to 128)
    while the tiles of all channel blocks would not run at once. A thread walks its tile in order,
    so short tiles are quick, but a second wave of blocks costs more than a longer walk."""
    tile = max(int(base), 1)
    blocks = -(-int(channels) // 256)
    while tile < 128 and -(-int(tokens) // tile) * blocks > _SEQ_CONV_RESIDENT:
        tile *= 2
    return tile


MATRIX_MEMORY_MAX_DIM = 256


def scale_rows_f32(x: torch.Tensor, scale: float) -> torch.Tensor:
    """``float32(x) * scale`` as a new float32 tensor (rows of a 16-bit table that start a 32-bit
    stream: the product is not rounded to the table's type)."""
    _cuda(x)
    if x.dim() != 2 or x.stride(1) != 1:
        raise KernelError("scale_rows_f32: x is [rows, width] with contiguous columns")
    out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    _lib.call("tk_scale_rows_f32", _ptr(x), x.stride(0), _ptr(out), float(scale), x.shape[0], x.shape[1],
              _dtype_code(x), _stream())
    return out


def seq_conv(u: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor | None, state: torch.Tensor | None,
             cu_seqlens: torch.Tensor, seq_ctx: torch.Tensor, seq_slot: torch.Tensor, tiles: tuple,
             out_dtype: torch.dtype, residual: bool = False, plain: bool = False, out_channels: int | None = None,
             kv: tuple | None = None, act: bool = False):
    """Causal convolution over time on each channel: ``y_t = [u_t +] bias + sum_j taps[:, j] u_(t - K + 1 + j)``
    within each sequence (zeros before its start). ``u`` [T, C] (rows may be strided), ``taps`` float32
    [C, K]; the last K - 1 rows of ``u`` of every sequence are kept in ``state`` (float32
    [slots, K - 1, C]). ``tiles``: ``ctx.tiles(size)`` with size >= K - 1. ``plain``: also returns ``u``
    itself in ``out_dtype``. ``act``: ``y <- silu(y)``. ``kv`` = ``(pool, block_table, page, kv_heads, k_dim, v_dim)``: the
    channels from ``out_channels`` on are ``kv_heads`` key heads then as many value heads and go into
    the paged pool at each token's position instead of the result."""
    _cuda(u, taps, bias, state, cu_seqlens, seq_ctx, seq_slot, *tiles)
    T, C = u.shape
    K = taps.shape[1]
    if u.stride(1) != 1 or taps.dtype != torch.float32 or not taps.is_contiguous() or taps.shape[0] != C:
        raise KernelError(f"seq_conv: u [T, {C}] with contiguous columns against float32 taps [{C}, K]")
    if K > 1 and (state is None or state.dtype != torch.float32 or tuple(state.shape[1:]) != (K - 1, C)
                  or not state.is_contiguous()):
        raise KernelError(f"seq_conv: the state is float32 [slots, {K - 1}, {C}]")
    b = _f32vec(bias, "conv bias", C)
    n_out = C if out_channels is None else int(out_channels)
    seq, tok0, off, n = tiles
    out = torch.empty(T, n_out, dtype=out_dtype, device=u.device) if n_out else None
    same = torch.empty(T, n_out, dtype=out_dtype, device=u.device) if plain and n_out else None
    pool = table = None
    P = hkv = dk = dv = dp = bt = 0
    if kv is not None:
        pool, table, P, hkv, dk, dv = kv
        _cuda(pool, table)
        if pool.dtype != out_dtype or not pool.is_contiguous() or pool.dim() != 5 or pool.shape[1] != 2 \
                or pool.shape[2] != hkv or pool.shape[3] != P:
            raise KernelError(f"seq_conv: the pool is {out_dtype} [pages, 2, {hkv}, {P}, row]")
        dp, bt = pool.shape[4], _i32(table, "block_table").stride(0)
    elif n_out != C:
        raise KernelError("seq_conv: channels beyond the output need a key/value pool")
    code = {torch.float32: F32, torch.bfloat16: BF16}
    _lib.call("tk_seq_conv", _ptr(u), u.stride(0), _dtype_code(u), _ptr(taps), _ptr(b), _ptr(state),
              _ptr(_i32(cu_seqlens, "cu_seqlens")), _ptr(_i32(seq_ctx, "seq_ctx")), _ptr(_i32(seq_slot, "seq_slot")),
              _ptr(_i32(seq, "tile_seq")), _ptr(_i32(tok0, "tile_tok0")), _ptr(_i32(off, "tile_off")),
              _ptr(_i32(n, "tile_n")), seq.numel(), _ptr(out), n_out, _ptr(same), n_out, code[out_dtype], K, C,
              int(bool(residual)), int(bool(act)), n_out, _ptr(pool), _ptr(table), bt, int(P), int(hkv), int(dk), int(dv), int(dp),
              _stream())
    return (out, same) if plain else out


def attention_pointwise_rows() -> int:
    return _lib.call("tk_attn_pointwise_rows")


def attention_pointwise(q: torch.Tensor, kv_pool: torch.Tensor, positions: torch.Tensor, tok_seq: torch.Tensor,
                        block_table: torch.Tensor, tile_tok0: torch.Tensor, tile_ntok: torch.Tensor,
                        tokens_per_tile: int, window: int | None, scale: float, v_dim: int, cap: float = 0.0,
                        temp_coef: float = 0.0, temp_every: int = 0, r1: torch.Tensor | None = None,
                        r2: torch.Tensor | None = None, head_bias: torch.Tensor | None = None) -> torch.Tensor:
    """Attention with a weight per visible key instead of a softmax: ``w = sigmoid(s + head_bias[h])``
    with ``s = cap * tanh(q.k * scale * temp(i) / cap) - r1[h] * ln(1 + r2[h] * (i - j))`` and
    ``temp(i) = 1 + temp_coef * ln(floor((i + 1) / temp_every) + 1)``; ``out = sum_j w_j v_j``. ``q``
    [T, H, D], ``kv_pool`` [pages, 2, Hkv, P, row]; returns [T, H, v_dim]. The CUDA-core form: any
    sizes, both storage types, 32-bit scores, weights and sums."""
    _cuda(q, kv_pool)
    T, H, D = q.shape
    _, two, Hkv, P, Dp = kv_pool.shape
    if two != 2 or kv_pool.dtype != q.dtype or Dp < max(D, v_dim) or not (q.is_contiguous() and kv_pool.is_contiguous()):
        raise KernelError("attention_pointwise: q [T, H, D] and a cache [pages, 2, Hkv, P, >= D] of one type expected")
    for name, t in (("r1", r1), ("r2", r2), ("head_bias", head_bias)):
        _f32vec(t, name, H)
    out = torch.empty(T, H, v_dim, dtype=q.dtype, device=q.device)
    _lib.call("tk_attn_pointwise", _ptr(q), _ptr(kv_pool), _ptr(out), _ptr(_i32(positions, "positions")),
              _ptr(_i32(tok_seq, "tok_seq")), _ptr(_i32(block_table, "block_table")), block_table.stride(0),
              _ptr(_i32(tile_tok0, "tile_tok0")), _ptr(_i32(tile_ntok, "tile_ntok")), tile_tok0.numel(),
              int(tokens_per_tile), H, Hkv, D, int(v_dim), Dp, P, int(window or 0), float(scale), float(cap or 0.0),
              float(temp_coef or 0.0), int(temp_every or 0), _ptr(r1), _ptr(r2), _ptr(head_bias), _dtype_code(q),
              _stream())
    return out


def attention_pointwise_mma_supported(heads: int, kv_heads: int, head_dim: int, v_dim: int, row: int,
                                      dtype: torch.dtype) -> bool:
    """Whether the tensor-core form of ``attention_pointwise`` takes the shape (bfloat16, keys, values
    and cache rows of one size, 64 or 128, at most 16 query heads per key/value head)."""
    return dtype == torch.bfloat16 and bool(_lib.call("tk_attn_pointwise_mma_supported", heads, kv_heads, head_dim,
                                                      v_dim, row))


def attention_pointwise_mma_tokens(heads: int, kv_heads: int) -> int:
    """Tokens per tile the tensor-core form expects for prompt portions."""
    return _lib.call("tk_attn_pointwise_mma_tokens", heads, kv_heads)


def attention_pointwise_mma(q: torch.Tensor, kv_pool: torch.Tensor, out: torch.Tensor, positions: torch.Tensor,
                            tok_seq: torch.Tensor, block_table: torch.Tensor, tile_tok0: torch.Tensor | None,
                            tile_ntok: torch.Tensor | None, singles: torch.Tensor | None, n_single: int, nsplit: int,
                            window: int | None, scale: float, cap: float = 0.0, temp_coef: float = 0.0,
                            temp_every: int = 0, r1: torch.Tensor | None = None, r2: torch.Tensor | None = None,
                            head_bias: torch.Tensor | None = None) -> None:
    """``attention_pointwise`` on the tensor cores: the tiles of prompt portions (``tile_tok0`` /
    ``tile_ntok``, ``attention_pointwise_mma_tokens`` tokens each) and ``n_single`` single tokens (their
    rows in ``singles``; None: rows 0 .. n_single - 1), each shared ``nsplit`` ways over its keys. The
    32-bit weights are rounded to bfloat16 where they meet the values. Writes those rows of ``out``."""
    _cuda(q, kv_pool, out, positions, tok_seq, block_table, tile_tok0, tile_ntok, singles)
    T, H, D, Hkv, P = _check_attention(q, kv_pool, "attention_pointwise_mma")
    for name, t in (("r1", r1), ("r2", r2), ("head_bias", head_bias)):
        _f32vec(t, name, H)
    n_tiles = tile_tok0.numel() if tile_tok0 is not None else 0
    partial = None
    if n_single and nsplit > 1:
        partial = torch.empty(nsplit * n_single * H * D, dtype=torch.float32, device=q.device)
    _lib.call("tk_attn_pointwise_mma", _ptr(q), _ptr(kv_pool), _ptr(out), _ptr(_i32(positions, "positions")),
              _ptr(_i32(tok_seq, "tok_seq")), _ptr(_i32(block_table, "block_table")), block_table.stride(0),
              _ptr(_i32(tile_tok0, "tile_tok0")) if n_tiles else None,
              _ptr(_i32(tile_ntok, "tile_ntok")) if n_tiles else None, n_tiles,
              _ptr(_i32(singles, "singles")) if singles is not None else None, int(n_single), int(nsplit),
              _ptr(partial), H, Hkv, D, P, int(window or 0), float(scale), float(cap or 0.0), float(temp_coef or 0.0),
              int(temp_every or 0), _ptr(r1), _ptr(r2), _ptr(head_bias), _stream())


def rglru_scan(z: torch.Tensor, rb: torch.Tensor, ib: torch.Tensor, decay: torch.Tensor, u: torch.Tensor,
               y: torch.Tensor, state: torch.Tensor, cu_seqlens: torch.Tensor, seq_ctx: torch.Tensor,
               seq_slot: torch.Tensor, n_seqs: int) -> torch.Tensor:
    """``S_t = a S_(t-1) + sqrt(1 - a^2) i u_t`` per channel with ``a = exp(decay * sigmoid(zr + rb))``,
    ``i = sigmoid(zi + ib)``; returns ``S_t * gelu_tanh(y_t)`` [T, W] in the type of ``u``. ``z`` float32
    [blocks, T, 2 w] (each block's recurrence-gate then input-gate products), ``u`` / ``y`` [T, W] (rows
    may be strided), ``state`` float32 [slots, W]."""
    _cuda(z, rb, ib, decay, u, y, state)
    blocks, Tz, w2 = z.shape
    T, W = u.shape
    if z.dtype != torch.float32 or not z.is_contiguous() or Tz != T or blocks * w2 != 2 * W:
        raise KernelError(f"rglru_scan: z is float32 [blocks, {T}, 2 w] with blocks * w = {W}")
    if u.stride(1) != 1 or y.stride(1) != 1 or y.dtype != u.dtype or y.shape[0] != T or y.shape[1] != W:
        raise KernelError("rglru_scan: u and y are [T, W] of one type with contiguous columns")
    if state.dtype != torch.float32 or not state.is_contiguous() or state.shape[1] != W:
        raise KernelError(f"rglru_scan: the state is float32 [slots, {W}]")
    out = torch.empty(T, W, dtype=u.dtype, device=u.device)
    _lib.call("tk_rglru_scan", _ptr(z), T, _ptr(_f32vec(rb, "rb", W)), _ptr(_f32vec(ib, "ib", W)),
              _ptr(_f32vec(decay, "decay", W)), _ptr(u), u.stride(0), _ptr(y), y.stride(0), _ptr(state),
              _ptr(_i32(cu_seqlens, "cu_seqlens")), _ptr(_i32(seq_ctx, "seq_ctx")), _ptr(_i32(seq_slot, "seq_slot")),
              int(n_seqs), _ptr(out), W, blocks, _dtype_code(u), _stream())
    return out


def mlstm_scan(qkv: torch.Tensor, offsets: tuple, gates: torch.Tensor, cap: float, q_scale: float,
               S_state: torch.Tensor, m_state: torch.Tensor, cu_seqlens: torch.Tensor, seq_ctx: torch.Tensor,
               seq_slot: torch.Tensor, n_seqs: int, heads: int, dim: int, v_dim: int):
    """The matrix memory's recurrence over a step's tokens. ``qkv`` [T, *]: q (heads x dim) at column
    ``offsets[0]``, k at ``offsets[1]``, v (heads x v_dim) at ``offsets[2]``; ``gates`` float32 [T, >= 2
    heads]: input- then forget-gate pre-activations. ``S_state`` float32 [slots, heads, v_dim + 1, dim]
    (the last column is n), ``m_state`` float32 [slots, heads]. Returns ``num`` float32 [T, heads,
    v_dim + 1] (``S_t^T q_t``; the last column ``n_t . q_t``) and ``m`` float32 [T, heads];
    ``mlstm_norm_gate`` finishes the output and commits ``m``."""
    _cuda(qkv, gates, S_state, m_state)
    T = qkv.shape[0]
    if qkv.stride(1) != 1 or gates.dtype != torch.float32 or gates.stride(1) != 1 or gates.shape[1] < 2 * heads:
        raise KernelError("mlstm_scan: qkv with contiguous columns, gates float32 [T, >= 2 heads]")
    if (S_state.dtype != torch.float32 or tuple(S_state.shape[1:]) != (heads, v_dim + 1, dim) or not S_state.is_contiguous()
            or m_state.dtype != torch.float32 or tuple(m_state.shape[1:]) != (heads,) or not m_state.is_contiguous()):
        raise KernelError(f"mlstm_scan: states float32 [slots, {heads}, {v_dim + 1}, {dim}] and [slots, {heads}]")
    num = torch.empty(T, heads, v_dim + 1, dtype=torch.float32, device=qkv.device)
    m = torch.empty(T, heads, dtype=torch.float32, device=qkv.device)
    _lib.call("tk_mlstm_scan", _ptr(qkv), qkv.stride(0), int(offsets[0]), int(offsets[1]), int(offsets[2]), _ptr(gates),
              gates.stride(0), float(cap or 0.0), float(q_scale), _ptr(S_state), _ptr(m_state),
              _ptr(_i32(cu_seqlens, "cu_seqlens")), _ptr(_i32(seq_ctx, "seq_ctx")), _ptr(_i32(seq_slot, "seq_slot")),
              int(n_seqs), T, _ptr(num), _ptr(m), heads, dim, v_dim, _dtype_code(qkv), _stream())
    return num, m


def mlstm_norm_gate(num: torch.Tensor, m: torch.Tensor, m_state: torch.Tensor, weight: torch.Tensor,
                    gate: torch.Tensor | None, tok_seq: torch.Tensor, cu_seqlens: torch.Tensor,
                    seq_slot: torch.Tensor, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """``o = num[..., :-1] / (max(|num[..., -1]|, exp(-m)) + 1e-6)``, each head divided by its root mean
    square, times ``weight`` [heads * v_dim], times ``sigmoid(gate)`` [T, heads * v_dim] (rows may be
    strided); returns [T, heads * v_dim]. The last token of each sequence writes its ``m`` to ``m_state``."""
    _cuda(num, m, m_state, weight, gate)
    T, H, cols = num.shape
    vd = cols - 1
    if gate is not None and (gate.dtype != out_dtype or gate.stride(1) != 1 or gate.shape[1] != H * vd):
        raise KernelError(f"mlstm_norm_gate: the gate is {out_dtype} [T, {H * vd}] with contiguous columns")
    out = torch.empty(T, H * vd, dtype=out_dtype, device=num.device)
    _lib.call("tk_mlstm_norm_gate", _ptr(num), _ptr(m), _ptr(m_state), _ptr(_f32vec(weight, "norm weight", H * vd)),
              _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(_i32(tok_seq, "tok_seq")),
              _ptr(_i32(cu_seqlens, "cu_seqlens")), _ptr(_i32(seq_slot, "seq_slot")), _ptr(out), T, H, vd, float(eps),
              F32 if out_dtype == torch.float32 else BF16, _stream())
    return out


SSD_MAX_STATE = 256


def ssd_scan(xbc: torch.Tensor, dt_raw: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor, d_skip: torch.Tensor,
             state: torch.Tensor, cu_seqlens: torch.Tensor, seq_ctx: torch.Tensor, seq_slot: torch.Tensor, n_seqs: int,
             heads: int, v_dim: int, n_state: int, groups: int, sm_count: int = 148) -> torch.Tensor:
    """The state-space recurrence over a step's tokens: ``dt = softplus(dt_raw + dt_bias)``, ``S_t = exp(-exp(a_log)
    dt) S_(t-1) + dt B_t x_t^T``, ``y_t = S_t^T C_t + d_skip x_t`` per head. ``xbc`` [T, >= heads v_dim + 2 groups
    n_state] (rows may be strided): x, then B, then C; ``dt_raw`` float32 [T, >= heads]; ``state`` float32 [slots,
    heads, n_state, v_dim]. Returns ``y`` float32 [parts, T, heads v_dim]: a step of few, long portions is walked
    by several blocks a head, each over a part of the state's rows, and their sums are still to be added
    (``gated_group_norm`` does; ``y.sum(0)`` is the result)."""
    _cuda(xbc, dt_raw, dt_bias, a_log, d_skip, state)
    T = xbc.shape[0]
    if xbc.stride(1) != 1 or xbc.shape[1] < heads * v_dim + 2 * groups * n_state:
        raise KernelError("ssd_scan: rows of x, B and C with contiguous columns")
    if dt_raw.dtype != torch.float32 or dt_raw.stride(1) != 1 or dt_raw.shape[0] != T or dt_raw.shape[1] < heads:
        raise KernelError(f"ssd_scan: dt is float32 [{T}, >= {heads}]")
    if state.dtype != torch.float32 or tuple(state.shape[1:]) != (heads, n_state, v_dim) or not state.is_contiguous():
        raise KernelError(f"ssd_scan: the state is float32 [slots, {heads}, {n_state}, {v_dim}]")
    split = _lib.call("tk_ssd_split", T, int(n_seqs), heads, v_dim, n_state, int(sm_count))
    y = torch.empty(split, T, heads * v_dim, dtype=torch.float32, device=xbc.device)
    _lib.call("tk_ssd_scan", _ptr(xbc), xbc.stride(0), _ptr(dt_raw), dt_raw.stride(0), _ptr(_f32vec(dt_bias, "dt_bias", heads)),
              _ptr(_f32vec(a_log, "A_log", heads)), _ptr(_f32vec(d_skip, "D", heads)), _ptr(state),
              _ptr(_i32(cu_seqlens, "cu_seqlens")), _ptr(_i32(seq_ctx, "seq_ctx")), _ptr(_i32(seq_slot, "seq_slot")),
              int(n_seqs), T, _ptr(y), split, heads, v_dim, n_state, groups, _dtype_code(xbc), _stream())
    return y


def gated_group_norm(y: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, eps: float, groups: int) -> torch.Tensor:
    """``v = y * silu(z)``, each of the row's ``groups`` equal parts divided by its own ``sqrt(mean(v^2) + eps)``,
    times ``weight``. ``y`` float32 [T, C], or [parts, T, C] whose parts are added up first; ``z`` [T, C] in the
    storage type (rows may be strided); returns [T, C] in ``z``'s type."""
    _cuda(y, z, weight)
    if y.dim() == 2:
        y = y.unsqueeze(0)
    parts, T, C = y.shape
    if y.dtype != torch.float32 or not y.is_contiguous() or z.stride(1) != 1 or tuple(z.shape) != (T, C):
        raise KernelError("gated_group_norm: y float32 [parts, T, C] contiguous, z [T, C] with contiguous columns")
    out = torch.empty(T, C, dtype=z.dtype, device=y.device)
    _lib.call("tk_gated_group_norm", _ptr(y), parts, _ptr(z), z.stride(0), _ptr(_f32vec(weight, "norm weight", C)), float(eps),
              _ptr(out), T, C, int(groups), _dtype_code(z), _stream())
    return out


def qkv_maps_write(qkv: torch.Tensor, positions: torch.Tensor, tok_seq: torch.Tensor, block_table: torch.Tensor | None,
                   pool: torch.Tensor | None, heads: int, kv_heads: int, dim: int, v_dim: int, maps: int) -> torch.Tensor:
    """From rows ``[q | k | v]`` (q: ``heads`` heads of ``maps`` parts of ``dim``; k: ``kv_heads`` heads likewise;
    v: ``kv_heads`` heads of ``v_dim``) the queries [T, heads * maps, maps * dim], each map a head of the key's
    width with zeros outside its part, and the keys and values into ``pool`` [pages, 2, kv_heads, P, row] at
    each token's position (``pool`` None: queries only). Positions enter nowhere."""
    _cuda(qkv, positions, tok_seq, block_table, pool)
    T = qkv.shape[0]
    need = heads * maps * dim + (kv_heads * (maps * dim + v_dim) if pool is not None else 0)
    if qkv.stride(1) != 1 or qkv.shape[1] < need:
        raise KernelError(f"qkv_maps_write: rows of at least {need} contiguous columns")
    q = torch.empty(T, heads * maps, maps * dim, dtype=qkv.dtype, device=qkv.device)
    P = dp = bt = 0
    if pool is not None:
        if (pool.dtype != qkv.dtype or not pool.is_contiguous() or pool.dim() != 5 or pool.shape[1] != 2
                or pool.shape[2] != kv_heads):
            raise KernelError(f"qkv_maps_write: the pool is {qkv.dtype} [pages, 2, {kv_heads}, P, row]")
        P, dp, bt = pool.shape[3], pool.shape[4], _i32(block_table, "block_table").stride(0)
    _lib.call("tk_qkv_maps_write", _ptr(qkv), qkv.stride(0), _ptr(_i32(positions, "positions")),
              _ptr(_i32(tok_seq, "tok_seq")), _ptr(block_table), bt, _ptr(q), _ptr(pool), T, heads, kv_heads, dim, v_dim,
              maps, P, dp, _dtype_code(qkv), _stream())
    return q


def diff_combine(a: torch.Tensor, lam: float, coef: float, eps: float) -> torch.Tensor:
    """``a`` [T, 2 H, V], a head's two maps' outputs side by side -> [T, H, V]: ``o = a_1 - lam a_2``, divided by
    ``sqrt(mean(o^2) + eps)`` over the head's values, times ``coef`` (32-bit, one rounding)."""
    _cuda(a)
    T, H2, V = a.shape
    if not a.is_contiguous() or H2 % 2:
        raise KernelError("diff_combine: a is contiguous [T, 2 H, V]")
    out = torch.empty(T, H2 // 2, V, dtype=a.dtype, device=a.device)
    _lib.call("tk_diff_combine", _ptr(a), _ptr(out), T * (H2 // 2), V, float(lam), float(coef), float(eps),
              _dtype_code(a), _stream())
    return out


def stream32_group_norm(stream: torch.Tensor | None, x: torch.Tensor | None, gate: torch.Tensor | None,
                        weight: torch.Tensor | None, eps: float, groups: int, out_dtype: torch.dtype,
                        in_place: bool = False):
    """``stream' = stream + x * sigmoid(gate)`` in 32-bit (``x`` without ``gate``: the plain add; ``stream`` None:
    ``x`` starts it), ``y = stream'`` with each of the row's ``groups`` equal parts divided by its own ``sqrt(mean
    + eps)``, times ``weight``, rounded once to ``out_dtype``. Returns ``(y, stream')``; ``y`` None without
    ``weight``. ``in_place``: ``stream`` is updated instead of copied."""
    _cuda(stream, x, gate, weight)
    src = x if x is not None else stream
    rows, width = src.shape
    if stream is not None and (stream.dtype != torch.float32 or not stream.is_contiguous()):
        raise KernelError("stream32_group_norm: the stream is contiguous float32")
    for t in (x, gate):
        if t is not None and (t.stride(1) != 1 or tuple(t.shape) != (rows, width)):
            raise KernelError("stream32_group_norm: x and gate are [rows, width] with contiguous columns")
    if x is not None and gate is not None and gate.dtype != x.dtype:
        raise KernelError("stream32_group_norm: x and gate are of one type")
    kind = x if x is not None else torch.empty(0, dtype=out_dtype)
    if kind.dtype != out_dtype:
        raise KernelError("stream32_group_norm: x and the normed rows are of one type")
    new = stream if (in_place and stream is not None) else torch.empty(rows, width, dtype=torch.float32, device=src.device)
    y = torch.empty(rows, width, dtype=out_dtype, device=src.device) if weight is not None else None
    _lib.call("tk_stream32_group_norm", _ptr(stream), _ptr(x), x.stride(0) if x is not None else 0, _ptr(gate),
              gate.stride(0) if gate is not None else 0, _ptr(_f32vec(weight, "norm weight", width)), float(eps),
              _ptr(new), _ptr(y), rows, width, int(groups), F32 if out_dtype == torch.float32 else BF16, _stream())
    return y, new
