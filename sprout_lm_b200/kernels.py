"""ctypes binding of the sm_100a kernel library.

Every function takes torch CUDA tensors, checks dtype, contiguity and sizes on the host,
and launches on torch's current stream.  There is no fallback: if the library cannot be
built or loaded, or no CUDA device is present, calls raise.
"""
from __future__ import annotations

import ctypes
import functools
import os
import threading
from ctypes import c_float, c_int, c_void_p

import torch

from .csrc.build import BuildError, library_path

F32, BF16 = 0, 1
LAUNCHES = 0          # kernels launched through this module (one per call); benchmarks read the difference
STATUS_BITS = {1: "a block-table entry outside the page pool", 2: "a token id outside the vocabulary",
               4: "non-finite logits", 8: "a bounded device-side wait ran out", 16: "a position outside the rotary table",
               32: "a kernel's shared memory was not aligned for its tiles"}


class KernelError(RuntimeError):
    pass


_P, _I, _F, _L = c_void_p, c_int, c_float, ctypes.c_longlong
_SIGNATURES = {
    "sprout_embed": [_P, _I, _P, _P, _I, _I, _I, _F, _P, _P],
    "sprout_rmsnorm": [_P, _P, _P, _I, _P, _I, _I, _F, _P],
    "sprout_swiglu": [_P, _P, _I, _I, _I, _I, _P],
    "sprout_rope_append": [_P, _P, _P, _I, _P, _P, _P, _I, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "sprout_gemm_simple": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "sprout_attention_simple": [_P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "sprout_sample": [_P, _I, _P, _P, _P, _P, _I, _I, _P, _P],
    "sprout_advance_decode": [_P, _P, _P, _P, _P, _P, _I, _I, _P],
    "sprout_feed_tokens": [_P, _P, _P, _I, _I, _I, _P],
    "sprout_attention_decode": [_P, _I, _P, _P, _P, _I, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "sprout_attention_decode_fused": [_P, _P, _P, _P, _I, _I, _I, _P, _P, _P, _I, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _I, _F, _P, _P],
    "sprout_attention_decode_resident": [_P, _P, _P, _P, _I, _I, _I, _P, _I, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _I, _F, _P, _P],
    "sprout_attention_decode_resident_cap": [_I, _I, _I, _I],
    "sprout_attention_prefill": [_P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, ctypes.c_longlong, _P, _P, _P],
    "sprout_attention_prefill_tc_supported": [_I, _I, _I],
    "sprout_gemm_bf16": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "sprout_gemm_bf16_unscaled": [_P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P],
    "sprout_ffn_decode": [_P, _P, _P, _P, _P, _I, _I, _I, _F, _P],
    "sprout_ffn_decode_supported": [_I, _I, _I],
    "sprout_wait_probe": [_P, _P],
    "sprout_linear_decode": [_P, _I, _P, _P, _F, _P, _P, _I, _I, _I, _I, _P, _P],
    "sprout_linear_decode_supported": [_I, _I, _I],
    "sprout_scale_cast": [_P, _P, _P, _I, _F, _L, _P],
    "sprout_sum_norm": [_P, _P, _P, _P, _P, _I, _I, _I, _F, _F, _P, _P, _I, _P],
    "sprout_polynorm": [_P, _I, _P, _I, _P, _I, _I, _F, _P],
    "sprout_latent_kv_append": [_P, _I, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _P, _I, _I, _I, _I, _I, _I, _F, _P, _P],
    "sprout_latent_query_tail": [_P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "sprout_headwise_gemm": [_P, _L, _L, _P, _P, _L, _L, _I, _I, _I, _I, _I, _P],
    "sprout_latent_attention_simple": [_P, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _P, _P],
    "sprout_latent_attention_mma": [_P, _P, _P, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _F, _P, _P],
    "sprout_latent_attention_mma_supported": [_I, _I],
    "sprout_depth_average": [_P, _P, _P, _I, _L, _P],
    "sprout_softcap": [_P, _F, _L, _P],
    "sprout_layernorm": [_P, _P, _P, _P, _I, _P, _I, _I, _F, _P],
    "sprout_norm_add": [_P, _P, _P, _P, _P, _I, _I, _I, _F, _P],
    "sprout_gated_rmsnorm": [_P, _P, _P, _I, _P, _I, _I, _I, _F, _P],
    "sprout_relu2": [_P, _P, _I, _L, _P],
    "sprout_glu_clamped": [_P, _P, _I, _I, _I, _F, _F, _P],
    "sprout_rope_maps_append": [_P, _I, _I, _P, _P, _P, _I, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _F, _I, _P, _P, _F, _P, _P],
    "sprout_multimap_attention_simple": [_P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _F, _F, _F, _F, _I, _I, _P, _P, _I, _I, _F, _P, _P],
    "sprout_multimap_attention_mma": [_P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _F, _F, _F, _F, _I, _P, _I, _I, _P, _P, _I, _I, _F, _P, _P],
    "sprout_multimap_attention_mma_supported": [_I, _I, _I],
    "sprout_decay_chunks": [_P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "sprout_decay_chunks_supported": [_I, _I, _I],
    "sprout_decay_scan": [_P, _I, _I, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _P, _P],
    "sprout_gated_scan": [_P, _I, _P, _I, _P, _I, _P, _I, _I, _I, _P, _P, _P, _F, _F, _I, _I, _I, _I, _I, _I, _P, _P, _P, _I, _P, _P,
                          _I, _I, _I, _P, _P, _P, _P, _I, _I, _P],
    "sprout_causal_conv": [_P, _I, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P],
    "sprout_gated_group_norm": [_P, _P, _I, _P, _I, _P, _I, _I, _I, _I, _F, _I, _I, _P],
    "sprout_scaled_sum": [_P, _P, _F, _P, _F, _L, _P],
    "sprout_moe_route": [_P, _I, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P, _I, _I, _I, _P],
    "sprout_exp_gates": [_P, _P, _I, _P, _P, _F, _I, _I, _P, _P, _P, _I, _P, _P, _P, _P, _P],
    "sprout_exp_memory_out": [_P, _I, _P, _P, _I, _I, _P, _P, _I, _I, _I, _I, _F, _F, _P],
    "sprout_unit_act": [_P, _I, _P, _I, _I, _I, _I, _I, _I, _P, _I, _P],
    "sprout_side_input_few": [_P, _P, _P, _P, _P, _I, _I, _P, _I, _I, _I, _I, _I, _F, _P, _P, _P],
    "sprout_side_gate": [_P, _I, _P, _I, _I, _P, _I, _P, _I, _I, _I, _P, _P],
    "sprout_rms_add": [_P, _P, _P, _I, _I, _F, _P],
    "sprout_add_rows": [_P, _P, _P, _I, _I, _P],
    "sprout_gated_rows_add": [_P, _P, _P, _I, _I, _I, _P],
    "sprout_narrow_rows": [_P, _P, _L, _P],
    "sprout_moe_arrange": [_P, _P, _P, _P, _P, _I, _I, _P],
    "sprout_moe_up_plain": [_P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _F, _P],
    "sprout_moe_down_plain": [_P, _I, _P, _P, _P, _I, _I, _I, _I, _P],
    "sprout_moe_combine": [_P, _P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _P],
    "sprout_moe_mma_supported": [_I, _I, _I],
    "sprout_moe_experts_mma": [_P, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _F, _P],
}

_lock = threading.Lock()
_lib = None


def load_library(verbose: bool = True):
    """The loaded kernel library, built on first use."""
    global _lib
    with _lock:
        if _lib is None:
            # SPROUT_KERNEL_LIBRARY names an already built library (an instrumented build, say)
            path = os.environ.get("SPROUT_KERNEL_LIBRARY") or library_path(build=True, verbose=verbose)
            lib = ctypes.CDLL(str(path))
            lib.sprout_last_error.restype = ctypes.c_char_p
            lib.sprout_abi_version.restype = c_int
            lib.sprout_sample_scratch_bytes.restype = ctypes.c_longlong
            lib.sprout_sample_scratch_bytes.argtypes = [c_int]
            lib.sprout_attention_decode_scratch_floats.restype = ctypes.c_longlong
            lib.sprout_attention_decode_scratch_floats.argtypes = [c_int, c_int, c_int, c_int]
            lib.sprout_attention_decode_ctas_per_sm.restype = c_int
            lib.sprout_attention_decode_ctas_per_sm.argtypes = [c_int, c_int, c_int]
            for name, argtypes in _SIGNATURES.items():
                fn = getattr(lib, name)
                fn.argtypes = argtypes
                fn.restype = c_int
            lib.sprout_set_pdl.argtypes = [c_int]
            lib.sprout_set_pdl.restype = None
            lib.sprout_sm_count.argtypes = []
            lib.sprout_sm_count.restype = c_int
            if os.environ.get("SPROUT_PDL", "1") == "0":
                lib.sprout_set_pdl(0)
            _lib = lib
    return _lib


def set_pdl(enabled: bool) -> None:
    """Programmatic dependent launch of all kernels on (the default) or off."""
    load_library().sprout_set_pdl(1 if enabled else 0)


_sm_counts: dict = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of ``device`` (the current one by default), asked once."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    if index is None:
        index = torch.cuda.current_device()
    count = _sm_counts.get(index)
    if count is None:
        count = _sm_counts[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return count


def library_file() -> str:
    return str(library_path(build=True, verbose=False))


def _dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported element type {dtype}; the kernels take float32 and bfloat16")


def _ptr(tensor, name, dtype=None, allow_none=False):
    if tensor is None:
        if allow_none:
            return None
        raise KernelError(f"{name} is missing")
    if not tensor.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor; there is no CPU path")
    if dtype is not None and tensor.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {tensor.dtype}")
    return tensor.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle.  The raw query is ten times cheaper than building a Stream
    object, and this runs once per kernel launch."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _run(name, *args):
    global LAUNCHES
    lib = _lib or load_library()
    if name not in _SIGNATURES:
        raise KernelError(f"{name}: no declared signature")         # an undeclared call would pass pointers as 32-bit integers
    LAUNCHES += 1
    code = getattr(lib, name)(*args)
    if code != 0:
        raise KernelError(lib.sprout_last_error().decode())


def _rows_contiguous(t, name):
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{name} must be 2-D with unit inner stride, got shape {tuple(t.shape)} strides {t.stride()}")


# ---------------------------------------------------------------------------------- wrappers

def embed(table, tokens, out, status, scale: float = 1.0):
    """out[t] = table[tokens[t]] widened to float32, times ``scale``."""
    _rows_contiguous(table, "table")
    if not table.is_contiguous() or not out.is_contiguous():
        raise KernelError("embed: table and out must be contiguous")
    T, H = out.shape
    if tokens.numel() != T or table.shape[1] != H:
        raise KernelError("embed: shapes do not fit")
    _run("sprout_embed", _ptr(table, "table"), _dtype_code(table.dtype), _ptr(tokens, "tokens", torch.int32),
         _ptr(out, "out", torch.float32), T, H, table.shape[0], float(scale), _ptr(status, "status", torch.int32), _stream())


def rmsnorm(x, gain, out, eps, rows=None):
    """out[r] = rmsnorm(x[rows[r]] or x[r]) * gain; x float32, out float32 or bfloat16."""
    if not x.is_contiguous() or not out.is_contiguous() or x.dim() != 2 or out.dim() != 2:
        raise KernelError("rmsnorm: x and out must be contiguous 2-D")
    R, H = out.shape
    if x.shape[1] != H or gain.numel() != H or (rows is None and x.shape[0] != R) or (rows is not None and rows.numel() != R):
        raise KernelError("rmsnorm: shapes do not fit")
    _run("sprout_rmsnorm", _ptr(x, "x", torch.float32), _ptr(gain, "gain", torch.float32), _ptr(out, "out"),
         _dtype_code(out.dtype), _ptr(rows, "rows", torch.int32, allow_none=True), R, H, float(eps), _stream())


def swiglu(gate_up, out, block: int = 8):
    """out = silu(gate) * up for rows that interleave gate and up in blocks of ``block`` columns
    (8: the tensor-core products' fused matrix; the intermediate size itself: gate rows first, then
    up rows)."""
    if not gate_up.is_contiguous() or not out.is_contiguous() or gate_up.dtype != out.dtype:
        raise KernelError("swiglu: tensors must be contiguous and of one dtype")
    T, I = out.shape
    if tuple(gate_up.shape) != (T, 2 * I):
        raise KernelError("swiglu: gate_up must be [tokens, 2 * intermediate]")
    _run("sprout_swiglu", _ptr(gate_up, "gate_up"), _ptr(out, "out"), _dtype_code(out.dtype), T, I, int(block), _stream())


def rope_append(qkv, positions, seq_of_token, block_table, cos_table, sin_table, k_cache, v_cache,
                heads, kv_heads, head_dim, page_tokens, write_cache, status, acc=None, bias=None,
                interleaved=False):
    """Rotate q and k of every token by its position; store rotated k and v in the paged cache.

    The tables are float32 [max_positions, rotary_dim / 2]: the first ``rotary_dim`` elements of a
    head turn (all of it when the tables are head_dim / 2 wide), in half-split pairs
    (d, d + rotary_dim / 2) or, with ``interleaved``, in pairs (2d, 2d + 1); the rest pass through.

    k_cache and v_cache are [pages, kv_heads, page_tokens, head_dim].  With ``acc`` (float32
    [tokens, width], row stride = width) the projections are read from there plus ``bias``
    instead of from ``qkv``, which then receives the rotated q; ``acc`` is left zeroed."""
    T = qkv.shape[0]
    if not qkv.is_contiguous() or qkv.shape[1] != (heads + 2 * kv_heads) * head_dim:
        raise KernelError("rope_append: qkv must be contiguous [tokens, (heads + 2 kv_heads) * head_dim]")
    if positions.numel() != T or seq_of_token.numel() != T:
        raise KernelError("rope_append: one position and one sequence index per token")
    if (cos_table is None) != (sin_table is None):
        raise KernelError("rope_append: cos and sin tables go together")
    if cos_table is not None and (cos_table.shape != sin_table.shape or cos_table.dim() != 2
                                  or not 0 < cos_table.shape[1] <= head_dim // 2
                                  or not cos_table.is_contiguous() or not sin_table.is_contiguous()):
        raise KernelError("rope_append: cos/sin tables must be contiguous [max_positions, rotary_dim / 2] with rotary_dim <= head_dim")
    rotary_dim = 2 * cos_table.shape[1] if cos_table is not None else 0
    num_pages = 1
    if write_cache:
        for name, cache in (("k_cache", k_cache), ("v_cache", v_cache)):
            if cache.dtype != qkv.dtype or not cache.is_contiguous() or tuple(cache.shape[1:]) != (kv_heads, page_tokens, head_dim):
                raise KernelError(f"rope_append: {name} must be contiguous [pages, kv_heads, page_tokens, head_dim] of {qkv.dtype}")
        num_pages = k_cache.shape[0]
    _rows_contiguous(block_table, "block_table")
    if acc is not None and (acc.dtype != torch.float32 or acc.dim() != 2 or acc.shape[0] < T
                            or acc.shape[1] != qkv.shape[1] or not acc.is_contiguous()):
        raise KernelError("rope_append: acc must be contiguous float32 [>= tokens, width]")
    if bias is not None and (acc is None or bias.numel() != qkv.shape[1]):
        raise KernelError("rope_append: a bias goes with acc and has one entry per column")
    _run("sprout_rope_append", _ptr(qkv, "qkv"), _ptr(acc, "acc", torch.float32, True),
         _ptr(bias, "bias", torch.float32, True), _dtype_code(qkv.dtype), _ptr(positions, "positions", torch.int32),
         _ptr(seq_of_token, "seq_of_token", torch.int32), _ptr(block_table, "block_table", torch.int32),
         block_table.stride(0), _ptr(cos_table, "cos", torch.float32, True), _ptr(sin_table, "sin", torch.float32, True),
         cos_table.shape[0] if cos_table is not None else 0, _ptr(k_cache, "k_cache", allow_none=not write_cache),
         _ptr(v_cache, "v_cache", allow_none=not write_cache), T, heads, kv_heads, head_dim, rotary_dim,
         1 if interleaved else 0, page_tokens, num_pages, 1 if write_cache else 0,
         _ptr(status, "status", torch.int32), _stream())


def gemm_simple(a, weight, out, bias=None, residual=None):
    """out = a @ weight.T (+ bias) (+ residual) with float32 accumulation on CUDA cores."""
    _rows_contiguous(a, "a")
    _rows_contiguous(out, "out")
    if not weight.is_contiguous() or weight.dim() != 2:
        raise KernelError("gemm_simple: weight must be contiguous [N, K]")
    M, K = a.shape
    N = weight.shape[0]
    if weight.shape[1] != K or tuple(out.shape) != (M, N) or weight.dtype != a.dtype:
        raise KernelError(f"gemm_simple: shapes/dtypes do not fit: a {tuple(a.shape)} {a.dtype}, "
                          f"weight {tuple(weight.shape)} {weight.dtype}, out {tuple(out.shape)}")
    if bias is not None and bias.numel() != N:
        raise KernelError("gemm_simple: bias must have N entries")
    if residual is not None and (tuple(residual.shape) != (M, N) or residual.stride(0) != out.stride(0)):
        raise KernelError("gemm_simple: residual must have out's shape and row stride")
    _run("sprout_gemm_simple", _ptr(a, "a"), _ptr(weight, "weight"), _ptr(bias, "bias", torch.float32, True),
         _ptr(residual, "residual", torch.float32, True), _ptr(out, "out"), _dtype_code(a.dtype),
         _dtype_code(out.dtype), M, N, K, a.stride(0), out.stride(0), _stream())


def attention_simple(q, k_cache, v_cache, block_table, seq_of_token, positions, out, heads, kv_heads, head_dim, status):
    """Paged causal attention with float32 arithmetic; q and out are [tokens, heads * head_dim] views."""
    _rows_contiguous(q, "q")
    _rows_contiguous(out, "out")
    _rows_contiguous(block_table, "block_table")
    T = q.shape[0]
    if q.shape[1] != heads * head_dim or tuple(out.shape) != (T, heads * head_dim):
        raise KernelError("attention_simple: q and out must be [tokens, heads * head_dim]")
    if k_cache.shape != v_cache.shape or tuple(k_cache.shape[1:]) != (kv_heads, k_cache.shape[2], head_dim) \
            or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise KernelError("attention_simple: caches must be contiguous [pages, kv_heads, page_tokens, head_dim]")
    if not (q.dtype == out.dtype == k_cache.dtype == v_cache.dtype):
        raise KernelError("attention_simple: q, out and the caches must share one dtype")
    _run("sprout_attention_simple", _ptr(q, "q"), q.stride(0), _ptr(k_cache, "k_cache"), _ptr(v_cache, "v_cache"),
         _ptr(block_table, "block_table", torch.int32), block_table.stride(0),
         _ptr(seq_of_token, "seq_of_token", torch.int32), _ptr(positions, "positions", torch.int32),
         _ptr(out, "out"), out.stride(0), _dtype_code(q.dtype), T, heads, kv_heads, head_dim, k_cache.shape[2],
         k_cache.shape[0], _ptr(status, "status", torch.int32), _stream())


def gemm_bf16(a, weight, out, status, bias=None, residual=None, orientation=0, split_k=1, swiglu=False, gate_activation="silu"):
    """out = a @ weight.T (+ bias) (+ residual) on the tcgen05 tensor cores; a and weight bfloat16.

    ``residual`` must be ``out`` itself (float32): the product is added in place.  orientation 0
    lets the kernel choose (weight rows on the MMA's M axis for up to 128 tokens), 1 forces
    tokens on M, 2 weights on M.  ``split_k`` > 1 divides K among CTAs (weights on M with a
    residual only; the partial sums are added with atomics).  ``swiglu``: weight rows interleave
    gate and up in blocks of 8 and ``out`` is bfloat16 [M, N/2] = act(gate) * up, act = ``gate_activation``: "silu" or
    "gelu_tanh" (the tanh form of gelu)."""
    if gate_activation not in ("silu", "gelu_tanh"):
        raise KernelError(f"gemm_bf16: the gated epilogue has silu and gelu_tanh, not {gate_activation!r}")
    _rows_contiguous(a, "a")
    _rows_contiguous(out, "out")
    if not weight.is_contiguous() or weight.dim() != 2:
        raise KernelError("gemm_bf16: weight must be contiguous [N, K]")
    M, K = a.shape
    N = weight.shape[0]
    if weight.shape[1] != K or tuple(out.shape) != (M, N // 2 if swiglu else N) or a.dtype != torch.bfloat16 \
            or weight.dtype != torch.bfloat16:
        raise KernelError(f"gemm_bf16: shapes/dtypes do not fit: a {tuple(a.shape)} {a.dtype}, "
                          f"weight {tuple(weight.shape)} {weight.dtype}, out {tuple(out.shape)}")
    if bias is not None and bias.numel() != N:
        raise KernelError("gemm_bf16: bias must have N entries")
    if residual is not None and residual.data_ptr() != out.data_ptr():
        raise KernelError("gemm_bf16: the residual is added in place: pass out itself")
    _run("sprout_gemm_bf16", _ptr(a, "a"), _ptr(weight, "weight"), _ptr(bias, "bias", torch.float32, True),
         _ptr(out, "out"), _dtype_code(out.dtype), (3 if gate_activation == "gelu_tanh" else 2) if swiglu else (1 if residual is not None else 0), M, N, K, a.stride(0),
         out.stride(0), orientation, split_k, _ptr(status, "status", torch.int32), _stream())


def gemm_bf16_unscaled_supported(tokens: int, out_features: int, in_features: int, split_k: int) -> bool:
    lib = _lib or load_library()
    lib.sprout_gemm_bf16_unscaled_supported.argtypes = [c_int, c_int, c_int, c_int]
    lib.sprout_gemm_bf16_unscaled_supported.restype = c_int
    return bool(lib.sprout_gemm_bf16_unscaled_supported(tokens, out_features, in_features, split_k))


def gemm_bf16_unscaled(x, gain, weight, out, status, split_k=1):
    """out (float32 [M, N]) += bfloat16(x * gain) @ weight.T for up to 256 tokens: the product of an
    RMSNorm's output without the norm's scale (x float32 [M, K] are the rows before the norm, gain
    its float32 gains).  Whoever reads the sums multiplies row m by 1 / sqrt(mean(x[m]^2) + eps)
    (``attention_decode_fused`` / ``attention_decode_resident`` with ``norm_x``).  The tokens' tiles
    are made inside the kernel: no kernel stands between the residual stream and the product."""
    _rows_contiguous(x, "x")
    _rows_contiguous(out, "out")
    M, K = x.shape
    N = weight.shape[0]
    if x.dtype != torch.float32 or out.dtype != torch.float32 or weight.dtype != torch.bfloat16 or not weight.is_contiguous() \
            or weight.shape[1] != K or tuple(out.shape) != (M, N) or gain.dtype != torch.float32 or gain.numel() != K:
        raise KernelError(f"gemm_bf16_unscaled: shapes/dtypes do not fit: x {tuple(x.shape)} {x.dtype}, weight {tuple(weight.shape)} "
                          f"{weight.dtype}, out {tuple(out.shape)} {out.dtype}")
    _run("sprout_gemm_bf16_unscaled", _ptr(x, "x", torch.float32), x.stride(0), _ptr(gain, "gain", torch.float32), _ptr(weight, "weight"),
         _ptr(out, "out", torch.float32), M, N, K, out.stride(0), split_k, _ptr(status, "status", torch.int32), _stream())


def linear_decode_supported(tokens: int, out_features: int, in_features: int) -> bool:
    """Whether ``linear_decode`` takes these sizes: 1..16 tokens, sizes that are multiples of 16, a
    matrix small enough for light CTAs."""
    lib = _lib or load_library()
    return bool(lib.sprout_linear_decode_supported(tokens, out_features, in_features))


def linear_decode(weight, out, status, a=None, norm=None):
    """out += input @ weight.T for up to 16 tokens, added with atomics into the float32 ``out``
    [tokens, N] (the residual stream, or a zeroed workspace).  The input is ``a`` (bfloat16
    [tokens, K]) or ``norm = (x, gain, eps)``: the RMSNorm of the float32 rows ``x``, computed
    inside the kernel."""
    _rows_contiguous(out, "out")
    if weight.dim() != 2 or not weight.is_contiguous() or weight.dtype != torch.bfloat16 or out.dtype != torch.float32:
        raise KernelError("linear_decode: weight must be contiguous bfloat16 [N, K], out float32")
    N, K = weight.shape
    T = out.shape[0]
    if out.shape[1] != N:
        raise KernelError(f"linear_decode: out {tuple(out.shape)} does not fit weight {tuple(weight.shape)}")
    if norm is not None:
        x, gain, eps = norm
        if tuple(x.shape) != (T, K) or not x.is_contiguous() or gain.numel() != K:
            raise KernelError("linear_decode: x must be contiguous [tokens, K] and gain have K entries")
        _run("sprout_linear_decode", None, 0, _ptr(x, "x", torch.float32), _ptr(gain, "gain", torch.float32), float(eps),
             _ptr(weight, "weight"), _ptr(out, "out"), out.stride(0), T, N, K, _ptr(status, "status", torch.int32), _stream())
        return
    _rows_contiguous(a, "a")
    if tuple(a.shape) != (T, K) or a.dtype != torch.bfloat16:
        raise KernelError(f"linear_decode: a must be bfloat16 [{T}, {K}], got {tuple(a.shape)} {a.dtype}")
    _run("sprout_linear_decode", _ptr(a, "a"), a.stride(0), None, None, 0.0, _ptr(weight, "weight"), _ptr(out, "out"),
         out.stride(0), T, N, K, _ptr(status, "status", torch.int32), _stream())


FFN_PLAN_FIELDS = ("ctas", "cluster", "tiles1", "base_tiles1", "max_tiles1", "boxes1", "box1_bytes", "tiles2", "max_tiles2",
                   "box_rows2", "row_boxes2", "max_ktiles", "max_ksteps", "col_boxes2", "box2_bytes", "stride1", "stride_x",
                   "off_w2", "off_act", "off_xchg", "off_bar", "smem_bytes")
LINEAR_PLAN_FIELDS = ("tiles", "ksteps", "row_groups", "k_splits", "max_tiles", "max_ksteps", "boxes", "box_bytes", "off_act",
                      "off_gain", "off_stage", "off_bar", "smem_bytes")


def small_batch_plan(kind: str, tokens: int, rows: int, cols: int, ctas: int | None = None, cluster: int = 1) -> dict | None:
    """How a small-batch kernel would lay a launch out on ``ctas`` CTAs (host arithmetic of the
    kernel library, no GPU needed), or None where it refuses the sizes.  ``kind`` "ffn": rows is
    the hidden size, cols the intermediate size, ``cluster`` the CTAs of a thread-block cluster
    (``ctas`` None: the shape the current device would get); "linear": a [rows, cols] matrix."""
    lib = _lib or load_library()
    out_type = ctypes.POINTER(c_int)
    if kind == "ffn":
        fn = lib.sprout_ffn_decode_plan
        fn.argtypes = [c_int, c_int, c_int, c_int, c_int, out_type]
        fn.restype = c_int
        out = (c_int * len(FFN_PLAN_FIELDS))()
        if not fn(tokens, rows, cols, 0 if ctas is None else ctas, cluster, out):
            return None
        return dict(zip(FFN_PLAN_FIELDS, out))
    if ctas is None:
        ctas = lib.sprout_sm_count()       # the current device's; a B200's 148 where there is none
    fn = lib.sprout_linear_decode_plan
    fn.argtypes = [c_int, c_int, c_int, c_int, out_type]
    fn.restype = c_int
    out = (c_int * len(LINEAR_PLAN_FIELDS))()
    if not fn(tokens, rows, cols, ctas, out):
        return None
    return dict(zip(LINEAR_PLAN_FIELDS, out))


FFN_PHASES = ("entry", "weights requested", "earlier kernels done", "norm", "weights there",
              "gate/up, SwiGLU, activation exchanged", "cluster met", "down rows there", "down done")


def ffn_decode_phase_stamps() -> dict | None:
    """Microseconds from a CTA's entry to the end of each phase of the last ``ffn_decode`` launch,
    for its first and its last CTA, from a library built with ``SPROUT_BUILD_FLAGS=-DFFN_STAMPS``
    (None from an ordinary build).  Synchronises the device."""
    lib = _lib or load_library()
    if not hasattr(lib, "sprout_ffn_stamps"):
        return None
    torch.cuda.synchronize()
    raw = (ctypes.c_ulonglong * 32)()
    lib.sprout_ffn_stamps(raw)
    return {which: {name: (raw[16 * c + i] - raw[16 * c]) / 1000.0 for i, name in enumerate(FFN_PHASES)}
            for c, which in enumerate(("first CTA", "last CTA"))}


ATTENTION_PHASES = ("entry", "first keys and values requested", "earlier kernels done", "q, new key and value ready",
                    "products and softmax", "warps merged", "cluster met", "splits merged, output stored", "cluster left")


def attention_decode_phase_stamps() -> dict | None:
    """Microseconds from entry to the end of each phase of the last split-key decode attention
    launch of a head size up to 64 (its first CTA), from a library built with
    ``SPROUT_BUILD_FLAGS=-DATTN_STAMPS`` (None from an ordinary build, or when no such launch has
    run).  Synchronises the device."""
    lib = _lib or load_library()
    if not hasattr(lib, "sprout_attention_stamps"):
        return None
    torch.cuda.synchronize()
    raw = (ctypes.c_ulonglong * 16)()
    lib.sprout_attention_stamps(raw)
    if not raw[0]:
        return None
    return {name: (raw[i] - raw[0]) / 1000.0 for i, name in enumerate(ATTENTION_PHASES)}


def decode_timeline() -> dict | None:
    """When the kernels of the last decode layer ran, from a library built with
    ``SPROUT_BUILD_FLAGS=-DSPROUT_TIMELINE`` (None from an ordinary build): per kernel the entry of
    its first CTA, the latest return of a CTA's wait for the earlier kernels and the latest exit,
    in microseconds after the first of these times.  The last product (the output head) stands
    for the kernel after the last layer.  Synchronises the device."""
    lib = _lib or load_library()
    if not hasattr(lib, "sprout_timeline_ffn_decode"):
        return None
    torch.cuda.synchronize()
    records = {}
    for label, reader, slot in (("norm + q/k/v", "linear_decode", 0), ("attention", "attention_bf16", 0), ("attention, wide heads", "attention_bf16_wide", 0),
                                ("output projection", "linear_decode", 1), ("feed-forward", "ffn_decode", 0),
                                ("q/k/v product", "gemm_tcgen05", 0), ("attention, resident", "attention_decode_resident", 0),
                                ("output product", "gemm_tcgen05", 1), ("gate/up product", "gemm_tcgen05", 2),
                                ("down product", "gemm_tcgen05", 3), ("head product", "gemm_tcgen05", 4)):
        raw = (ctypes.c_ulonglong * 32)()
        getattr(lib, "sprout_timeline_" + reader)(raw)
        records[label] = [raw[4 * slot], raw[4 * slot + 1], raw[4 * slot + 2]]
    # the records of kernels that this step did not run are older than the step: drop what lies more than 5 ms before the newest
    newest = max(v[2] for v in records.values())
    records = {label: v for label, v in records.items() if v[0] and newest - v[0] < 5_000_000}
    origin = min(v[0] for v in records.values() if v[0])
    return {label: {"entry": (v[0] - origin) / 1000.0, "waited": (v[1] - origin) / 1000.0, "exit": (v[2] - origin) / 1000.0}
            for label, v in records.items() if v[0]}


def wait_probe(status):
    """Launch a one-warp kernel that waits (bounded, about a second and a half) on a barrier on
    which nothing arrives, gives up, sets the status word's wait bit and returns: for tests of the
    bound that every TMA and tcgen05 kernel's waits share."""
    _run("sprout_wait_probe", _ptr(status, "status", torch.int32), _stream())


def ffn_decode_supported(tokens: int, hidden: int, intermediate: int) -> bool:
    """Whether ``ffn_decode`` takes these sizes: 1..16 tokens, sizes that are multiples of 16, and a
    layer small enough for every CTA to hold its share of the two matrices in shared memory."""
    lib = _lib or load_library()
    return bool(lib.sprout_ffn_decode_supported(tokens, hidden, intermediate))


def ffn_decode(x, gain, eps, w_gate_up, w_down, status):
    """x += W_down (silu(W_gate h) * W_up h) with h = rmsnorm(x, gain, eps), for up to 16 tokens,
    in one kernel (norm, both products, activation and residual sum; the activation is exchanged
    among the CTAs of a thread-block cluster and never goes to memory).

    ``x`` float32 [tokens, hidden], changed in place; ``w_gate_up`` bfloat16 [2 * intermediate,
    hidden] with gate and up rows interleaved in blocks of 8; ``w_down`` bfloat16 [hidden,
    intermediate]."""
    if x.dim() != 2 or not x.is_contiguous() or not w_gate_up.is_contiguous() or not w_down.is_contiguous():
        raise KernelError("ffn_decode: x and the weights must be contiguous")
    T, H = x.shape
    inter = w_down.shape[1]
    if tuple(w_gate_up.shape) != (2 * inter, H) or w_down.shape[0] != H or gain.numel() != H:
        raise KernelError(f"ffn_decode: shapes do not fit: x {tuple(x.shape)}, gate/up {tuple(w_gate_up.shape)}, "
                          f"down {tuple(w_down.shape)}")
    _run("sprout_ffn_decode", _ptr(x, "x", torch.float32), _ptr(gain, "gain", torch.float32),
         _ptr(w_gate_up, "w_gate_up", torch.bfloat16), _ptr(w_down, "w_down", torch.bfloat16),
         _ptr(status, "status", torch.int32), T, H, inter, float(eps), _stream())


def _check_paged(q, k_cache, v_cache, block_table, out, heads, head_dim, name):
    _rows_contiguous(q, "q")
    _rows_contiguous(out, "out")
    _rows_contiguous(block_table, "block_table")
    T = q.shape[0]
    if q.shape[1] != heads * head_dim or tuple(out.shape) != (T, heads * head_dim):
        raise KernelError(f"{name}: q and out must be [tokens, heads * head_dim]")
    if k_cache.shape != v_cache.shape or k_cache.dim() != 4 or k_cache.shape[3] != head_dim \
            or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise KernelError(f"{name}: caches must be contiguous [pages, kv_heads, page_tokens, head_dim]")
    if not (q.dtype == out.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16):
        raise KernelError(f"{name}: q, out and the caches must be bfloat16")


def decode_split_plan(requests: int, kv_heads: int, max_keys: int, head_dim: int = 64,
                      live_keys: int | None = None, sms: int | None = None) -> tuple[int, int, bool]:
    """(keys per split, splits, whether scratch memory is needed) for decode attention over at
    most ``max_keys`` keys (the block tables' width), of which about ``live_keys`` are expected
    to hold keys (a replayed graph's tables are wider than its contexts; splits beyond a
    request's length cost next to nothing).  A CTA takes its split in passes of 128 keys, one
    after the other; up to 8 splits of a (request, key/value head) merge inside a thread-block
    cluster, more go through scratch memory and a merge kernel.

    The pick minimises a small model of the kernel's time, fitted to measurements on a B200: the
    CTAs run in waves of as many as the SMs hold at once (the device's own count for the kernel as
    built; fewer for clusters, whose CTAs hold more shared memory and must be placed together); the
    launch costs a fixed start, every wave its passes (the longer of a pass's latency and the time
    to bring the wave's keys and values in), every further wave a little more; a merge costs a
    little inside a cluster and more through memory, growing with the splits.  So a small batch
    gets many short splits in a cluster (latency), a large one few long ones, and a launch of
    several waves goes through memory even where its splits would fit a cluster."""
    live = max_keys if live_keys is None else max(1, min(max_keys, live_keys))
    if sms is None:
        sms = sm_count() if torch.cuda.is_available() else 148      # host-side inspection without a device: a B200's count
    return _decode_split_plan(requests * kv_heads, -(-max_keys // 128), -(-live // 128), head_dim, sms,
                              decode_ctas_per_sm(head_dim), decode_ctas_per_sm(head_dim, True))


@functools.lru_cache(maxsize=64)
def decode_ctas_per_sm(head_dim: int, cluster: bool = False) -> int:
    """CTAs of the split-key decode kernel that an SM holds at once (``cluster``: of the variant
    launched in clusters, whose CTAs also hold what the splits send one another): the device's own
    answer for the kernel as built (registers and shared memory), or, without a device, what its
    shared memory and its register bounds give on a B200."""
    if torch.cuda.is_available() and head_dim % 16 == 0 and head_dim <= 128:
        count = int(load_library().sprout_attention_decode_ctas_per_sm(head_dim, 1, int(cluster)))
        if count > 0:
            return count
    stride = head_dim if head_dim == 128 or (head_dim == 64 and not cluster) else head_dim + 8    # swizzled rows, or rows padded by 16 bytes
    shared = 16 * (head_dim + 8) * 2 + 2 * 128 * stride * 2 + 128 * 8 + 16    # the tensor-core kernel's, per CTA
    if cluster:
        shared += (8 * head_dim + 8) * 8 + 256 * 4
    by_registers = (4 if cluster else 5) if head_dim <= 64 else 3 if head_dim == 128 else 4      # by its registers
    return max(1, min(by_registers, (228 * 1024) // (shared + 1024)))


@functools.lru_cache(maxsize=4096)
def _decode_split_plan(pairs: int, total_passes: int, live_passes: int, head_dim: int, sms: int, per_sm: int,
                       per_sm_cluster: int | None = None) -> tuple[int, int, bool]:
    slots = sms * per_sm
    cluster_slots = sms * (per_sm_cluster or per_sm)
    total_passes = max(1, total_passes)
    best, best_cost, last = (128 * total_passes, 1, False), None, None
    for passes in range(1, total_passes + 1):
        splits = -(-total_passes // passes)
        live_splits = -(-live_passes // passes)
        if (splits, live_splits) == last:
            continue                       # the same splits, as many of them with keys, longer passes: never better
        last = (splits, live_splits)
        # a pass takes 1.6 to 2.3 us (by the head size) when little is in flight, 3.5 us once about
        # 16 MB are (the latency under load), and never less than the wave's bytes at 6.3 TB/s
        idle_us = 1.0 + head_dim / 100.0
        for through_memory in (False, True):
            if (through_memory and splits == 1) or (not through_memory and splits > 8):
                continue
            # the CTAs that hold a slot: a cluster is placed whole, of independent CTAs those that find keys
            ctas = pairs * (live_splits if through_memory else splits)
            # a cluster needs room for all its CTAs at once in one part of the GPU: larger clusters pack worse
            room = slots if through_memory or splits == 1 else max(1, int(cluster_slots * (1.0 - 0.06 * (splits - 1))))
            # a last wave that is not full costs less than a full one: half-way between the two counts
            waves = max(1.0, (-(-ctas // room) + ctas / room) / 2)
            wave_mb = min(ctas, room) * 128 * head_dim * 4 / 1e6
            pass_us = max(idle_us + (3.5 - idle_us) * min(1.0, wave_mb / 16.0), wave_mb / 6.3)
            merge_us = 0.0 if splits == 1 else 3.5 + 0.085 * splits if through_memory else 1.0
            # the first wave pays the launch's start; CTAs of later waves start as others leave
            cost = 2.2 + waves * min(passes, live_passes) * pass_us + (waves - 1.0) * 1.0 + merge_us
            if best_cost is None or cost < best_cost:
                best, best_cost = (128 * passes, splits, through_memory), cost
    return best


def attention_decode(q, k_cache, v_cache, block_table, context_lens, out, heads, kv_heads, head_dim, status,
                     split_keys=None, scratch=None, live_keys=None):
    """One query token per request over its pages (bfloat16, float32 softmax): keys are split
    among CTAs; up to 8 splits merge inside a thread-block cluster, more (or a given
    ``scratch``) go through float32 scratch memory and a merge kernel."""
    _check_paged(q, k_cache, v_cache, block_table, out, heads, head_dim, "attention_decode")
    R = q.shape[0]
    max_keys = block_table.shape[1] * k_cache.shape[2]
    if split_keys is None:
        split_keys, splits, through_memory = decode_split_plan(R, kv_heads, max_keys, head_dim, live_keys)
    else:
        splits = max(1, -(-max_keys // split_keys))
        through_memory = splits > 8
    need = load_library().sprout_attention_decode_scratch_floats(R, heads, head_dim, splits)
    if through_memory and scratch is None:
        scratch = torch.empty(need, dtype=torch.float32, device=q.device)
    if scratch is not None and (scratch.dtype != torch.float32 or scratch.numel() < need):
        raise KernelError(f"attention_decode: scratch must hold {need} float32 values")
    _run("sprout_attention_decode", _ptr(q, "q"), q.stride(0), _ptr(k_cache, "k_cache"), _ptr(v_cache, "v_cache"),
         _ptr(block_table, "block_table", torch.int32), block_table.stride(0),
         _ptr(context_lens, "context_lens", torch.int32), _ptr(out, "out"), out.stride(0),
         _ptr(scratch, "scratch", torch.float32, True), R, heads, kv_heads, head_dim, k_cache.shape[2],
         k_cache.shape[0], split_keys, splits, _ptr(status, "status", torch.int32), _stream())


RESIDENT_STEP = 256          # the resident kernel's room for keys grows in steps of this many


@functools.lru_cache(maxsize=256)
def resident_cap(heads: int, kv_heads: int, head_dim: int, page_tokens: int) -> int:
    """The longest context that ``attention_decode_resident`` takes for these sizes (0: none)."""
    return int(load_library().sprout_attention_decode_resident_cap(heads, kv_heads, head_dim, page_tokens))


def decode_attention_plan(requests: int, heads: int, kv_heads: int, head_dim: int, page_tokens: int, max_keys: int,
                          planned_keys: int | None = None) -> tuple:
    """How a step of one token per request runs its attention over contexts of up to
    ``planned_keys`` keys (block tables ``max_keys`` wide): ``("resident", room)`` where a request's
    whole context fits one CTA's shared memory (room: keys, in steps of 256), else ``("split", keys
    per split, splits, through memory)`` as ``decode_split_plan`` lays it out."""
    planned = max(1, min(max_keys, planned_keys if planned_keys else max_keys))
    # One CTA per (request, key/value head) pulls its whole context alone: that pays once there are
    # enough of them to keep the SMs' copy engines busy, and as long as they all fit the SMs at once
    # (they are one to an SM).  Measured alone at the 0.5B sizes, 640 keys each, split plan against
    # resident: 8 requests 4.6 / 5.4 us, 32: 8.0 / 5.5, 64: 11.1 / 7.7, 128: 14.4 / 14.3, 256: 19.2 / 28.9.
    sms = sm_count() if torch.cuda.is_available() else 148
    # At head size 128 a second wave of them loses to the split kernel, which holds three CTAs per SM
    # there (7B sizes, 64 requests of 384 keys: 15.6 against 10.9 us; 32 requests: 8.2 against 13.4).
    most = 2 * sms if head_dim == 64 else sms
    if RESIDENT_ENABLED and head_dim in (64, 128) and (3 * sms) // 8 <= requests * kv_heads <= most:
        cap = resident_cap(heads, kv_heads, head_dim, page_tokens)
        room = min(cap, -(-planned // RESIDENT_STEP) * RESIDENT_STEP)
        if planned <= room:
            return ("resident", room)
    return ("split",) + decode_split_plan(requests, kv_heads, max_keys, head_dim, planned)


RESIDENT_ENABLED = os.environ.get("SPROUT_RESIDENT_ATTENTION", "1") != "0"


def _norm_scale(norm_x, requests: int, name: str):
    """(pointer, width, eps) of the rows whose inverse RMS scales a request's sums; ``norm_x`` is
    (x float32 [requests, width] contiguous, eps) or None."""
    if norm_x is None:
        return None, 0, 0.0
    x, eps = norm_x
    if x.dtype != torch.float32 or x.dim() != 2 or x.shape[0] != requests or not x.is_contiguous() or not eps > 0:
        raise KernelError(f"{name}: the scale needs contiguous float32 rows [requests, width] and a positive eps")
    return _ptr(x, "norm_x", torch.float32), x.shape[1], float(eps)


def attention_decode_resident(k_cache, v_cache, block_table, context_lens, out, heads, kv_heads, head_dim, status, room,
                              q=None, acc=None, bias=None, cos_table=None, sin_table=None, interleaved=False, norm_x=None):
    """Decode attention with every request's whole context (at most ``room`` keys) in one CTA's
    shared memory, fetched by TMA before the wait for the step's earlier kernels.  With ``acc``
    (and ``bias``, rotation tables) the fused form of ``attention_decode_fused``: the new token's
    q, k, v come as float32 sums, k and v are appended to the cache, the sums are cleared; with
    ``q`` the cache already holds the new token.  ``out`` is bfloat16 [requests, heads * head_dim]."""
    R = out.shape[0]
    width = (heads + 2 * kv_heads) * head_dim
    if (acc is None) == (q is None):
        raise KernelError("attention_decode_resident: give either q or the float32 sums")
    if acc is not None and (acc.dtype != torch.float32 or tuple(acc.shape) != (R, width) or not acc.is_contiguous()):
        raise KernelError("attention_decode_resident: acc must be contiguous float32 [requests, (heads + 2 kv_heads) * head_dim]")
    if q is not None:
        _rows_contiguous(q, "q")
        if q.dtype != torch.bfloat16 or tuple(q.shape) != (R, heads * head_dim):
            raise KernelError("attention_decode_resident: q must be bfloat16 [requests, heads * head_dim]")
    if out.dtype != torch.bfloat16 or out.shape[1] != heads * head_dim or out.stride(1) != 1:
        raise KernelError("attention_decode_resident: out must be bfloat16 [requests, heads * head_dim]")
    if k_cache.shape != v_cache.shape or k_cache.dim() != 4 or k_cache.shape[3] != head_dim or k_cache.shape[1] != kv_heads \
            or k_cache.dtype != torch.bfloat16 or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise KernelError("attention_decode_resident: caches must be contiguous bfloat16 [pages, kv_heads, page_tokens, head_dim]")
    if bias is not None and bias.numel() != width:
        raise KernelError("attention_decode_resident: bias must have one entry per column of acc")
    if (cos_table is None) != (sin_table is None):
        raise KernelError("attention_decode_resident: cos and sin tables go together")
    if cos_table is not None and (cos_table.shape != sin_table.shape or cos_table.dim() != 2
                                  or not 0 < cos_table.shape[1] <= head_dim // 2
                                  or not cos_table.is_contiguous() or not sin_table.is_contiguous()):
        raise KernelError("attention_decode_resident: cos/sin tables must be contiguous [max_positions, rotary_dim / 2]")
    _rows_contiguous(block_table, "block_table")
    _run("sprout_attention_decode_resident", _ptr(acc, "acc", torch.float32, True), _ptr(bias, "bias", torch.float32, True),
         _ptr(cos_table, "cos", torch.float32, True), _ptr(sin_table, "sin", torch.float32, True),
         cos_table.shape[0] if cos_table is not None else 0, 2 * cos_table.shape[1] if cos_table is not None else 0,
         1 if interleaved else 0, _ptr(q, "q", torch.bfloat16, True), q.stride(0) if q is not None else 0,
         _ptr(k_cache, "k_cache"), _ptr(v_cache, "v_cache"), _ptr(block_table, "block_table", torch.int32),
         block_table.stride(0), _ptr(context_lens, "context_lens", torch.int32), _ptr(out, "out"), out.stride(0),
         R, heads, kv_heads, head_dim, k_cache.shape[2], k_cache.shape[0], int(room),
         *_norm_scale(norm_x if acc is not None else None, R, "attention_decode_resident"), _ptr(status, "status", torch.int32), _stream())


def decode_fusable(requests: int, heads: int, kv_heads: int, head_dim: int, max_keys: int) -> bool:
    """Whether the decode step's attention can take the projection's tail (bias, rotation, cache
    append) into its own kernel: the tensor-core kernel's sizes."""
    return head_dim <= 128 and head_dim % 16 == 0 and heads // kv_heads <= 16


def attention_decode_fused(acc, bias, cos_table, sin_table, k_cache, v_cache, block_table, context_lens, out,
                           heads, kv_heads, head_dim, status, live_keys=None, interleaved=False, scratch=None, norm_x=None):
    """Decode attention with the q/k/v projection's tail folded in.  ``acc`` holds, for each
    request's new token, the float32 sums [requests, (heads + 2 kv_heads) * head_dim] of a split-K
    product; the kernel adds ``bias``, rotates q and k by the position context_lens - 1 (tables
    [max_positions, rotary_dim / 2] and ``interleaved`` as for ``rope_append``; None: no rotation),
    appends k and v to the paged cache, attends over context_lens keys and leaves ``acc`` zeroed.
    ``out`` is bfloat16 [requests, heads * head_dim].  ``scratch``: float32 memory for the splits'
    partial results where the plan merges through memory (allocated here when not given).
    ``norm_x`` = (x, eps): the sums are those of ``gemm_bf16_unscaled`` (a normalised input without
    its scale); request r's sums are multiplied by 1 / sqrt(mean(x[r]^2) + eps) first."""
    R = out.shape[0]
    width = (heads + 2 * kv_heads) * head_dim
    if acc.dtype != torch.float32 or tuple(acc.shape) != (R, width) or not acc.is_contiguous():
        raise KernelError("attention_decode_fused: acc must be contiguous float32 [requests, (heads + 2 kv_heads) * head_dim]")
    if out.dtype != torch.bfloat16 or out.shape[1] != heads * head_dim or out.stride(1) != 1:
        raise KernelError("attention_decode_fused: out must be bfloat16 [requests, heads * head_dim]")
    if k_cache.shape != v_cache.shape or k_cache.dim() != 4 or k_cache.shape[3] != head_dim or k_cache.shape[1] != kv_heads \
            or k_cache.dtype != torch.bfloat16 or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise KernelError("attention_decode_fused: caches must be contiguous bfloat16 [pages, kv_heads, page_tokens, head_dim]")
    if bias is not None and bias.numel() != width:
        raise KernelError("attention_decode_fused: bias must have one entry per column of acc")
    _rows_contiguous(block_table, "block_table")
    max_keys = block_table.shape[1] * k_cache.shape[2]
    split_keys, splits, through_memory = decode_split_plan(R, kv_heads, max_keys, head_dim, live_keys)
    if not decode_fusable(R, heads, kv_heads, head_dim, max_keys):
        raise KernelError("attention_decode_fused: these sizes need the separate kernels (see decode_fusable)")
    if cos_table is not None and (cos_table.shape != sin_table.shape or cos_table.dim() != 2
                                  or not 0 < cos_table.shape[1] <= head_dim // 2
                                  or not cos_table.is_contiguous() or not sin_table.is_contiguous()):
        raise KernelError("attention_decode_fused: cos/sin tables must be contiguous [max_positions, rotary_dim / 2]")
    if through_memory:            # many splits or a large batch: independent CTAs and a merge kernel
        need = load_library().sprout_attention_decode_scratch_floats(R, heads, head_dim, splits)
        if scratch is None or scratch.numel() < need:
            scratch = torch.empty(need, dtype=torch.float32, device=out.device)
    else:
        scratch = None
    _run("sprout_attention_decode_fused", _ptr(acc, "acc"), _ptr(bias, "bias", torch.float32, True),
         _ptr(cos_table, "cos", torch.float32, True), _ptr(sin_table, "sin", torch.float32, True),
         cos_table.shape[0] if cos_table is not None else 0, 2 * cos_table.shape[1] if cos_table is not None else 0,
         1 if interleaved else 0, _ptr(k_cache, "k_cache"), _ptr(v_cache, "v_cache"),
         _ptr(block_table, "block_table", torch.int32), block_table.stride(0),
         _ptr(context_lens, "context_lens", torch.int32), _ptr(out, "out"), out.stride(0),
         _ptr(scratch, "scratch", torch.float32, True), R, heads, kv_heads, head_dim,
         k_cache.shape[2], k_cache.shape[0], split_keys, splits, *_norm_scale(norm_x, R, "attention_decode_fused"),
         _ptr(status, "status", torch.int32), _stream())


PREFILL_VARIANTS = {"auto": 0, "mma_sync": 1, "tcgen05": 2}
# which prefill attention kernel the engine's steps use (measurements compare them)
PREFILL_VARIANT = os.environ.get("SPROUT_PREFILL_ATTENTION", "auto")
_prefill_scratch: dict = {}      # (device, head_dim) -> (float32 scratch, int32 counters) of the tcgen05 prefill kernel


def _prefill_workspace(device, head_dim):
    key = (device, head_dim)
    held = _prefill_scratch.get(key)
    if held is None:
        lib = load_library()
        lib.sprout_attention_prefill_scratch_floats.restype = ctypes.c_longlong
        lib.sprout_attention_prefill_scratch_floats.argtypes = [c_int]
        lib.sprout_attention_prefill_counters.restype = c_int
        lib.sprout_attention_prefill_counters.argtypes = []
        held = (torch.empty(lib.sprout_attention_prefill_scratch_floats(head_dim), dtype=torch.float32, device=device),
                torch.zeros(lib.sprout_attention_prefill_counters(), dtype=torch.int32, device=device))
        _prefill_scratch[key] = held
    return held


def attention_prefill(q, k_cache, v_cache, block_table, q_start, positions, out, heads, kv_heads, head_dim, status,
                      variant="auto"):
    """Tensor-core flash attention of the step's queries (portions of prompts, single tokens) over
    their requests' pages (bfloat16, float32 softmax).  ``variant``: "tcgen05" (S and P V in tensor
    memory, K and V pages by TMA; head_dim 64 or 128, pages of 8..64 or a multiple of 128 tokens),
    "mma_sync" (every head_dim up to 128 in steps of 16, every page size), or "auto": tcgen05
    where it takes the sizes and the requests bring 128 (token, head) rows each on average."""
    _check_paged(q, k_cache, v_cache, block_table, out, heads, head_dim, "attention_prefill")
    scratch = counters = None
    if variant != "mma_sync" and head_dim in (64, 128):
        scratch, counters = _prefill_workspace(q.device, head_dim)
    _run("sprout_attention_prefill", _ptr(q, "q"), q.stride(0), _ptr(k_cache, "k_cache"), _ptr(v_cache, "v_cache"),
         _ptr(block_table, "block_table", torch.int32), block_table.stride(0), _ptr(q_start, "q_start", torch.int32),
         _ptr(positions, "positions", torch.int32), _ptr(out, "out"), out.stride(0), q.shape[0], q_start.numel() - 1,
         heads, kv_heads, head_dim, k_cache.shape[2], k_cache.shape[0], PREFILL_VARIANTS[variant],
         _ptr(scratch, "scratch", torch.float32, True), scratch.numel() if scratch is not None else 0,
         _ptr(counters, "counters", torch.int32, True), _ptr(status, "status", torch.int32), _stream())


def paged_attention(q, cache, ctx, out, heads, kv_heads, head_dim, status):
    """Causal attention of the step's queries over their requests' pages (``cache`` is a
    CacheView).  float32 runs the plain kernel (the true 32-bit path); bfloat16 runs the split-key
    kernel when every request brings one token and the tensor-core kernel otherwise."""
    if q.dtype == torch.bfloat16:
        if ctx.max_q_len == 1 and heads // kv_heads <= 16:
            max_keys = cache.block_table.shape[1] * cache.k.shape[2]
            plan = decode_attention_plan(q.shape[0], heads, kv_heads, head_dim, cache.k.shape[2], max_keys,
                                         ctx.planned_context or ctx.max_context)
            if plan[0] == "resident":
                return attention_decode_resident(cache.k, cache.v, cache.block_table, ctx.context_lens, out, heads, kv_heads,
                                                 head_dim, status, plan[1], q=q)
            return attention_decode(q, cache.k, cache.v, cache.block_table, ctx.context_lens, out,
                                    heads, kv_heads, head_dim, status, live_keys=ctx.planned_context or ctx.max_context)
        if head_dim <= 128:
            variant = PREFILL_VARIANT
            if variant == "tcgen05" and not load_library().sprout_attention_prefill_tc_supported(head_dim, cache.k.shape[2], out.stride(0)):
                variant = "mma_sync"
            return attention_prefill(q, cache.k, cache.v, cache.block_table, ctx.q_start, ctx.positions, out,
                                     heads, kv_heads, head_dim, status, variant=variant)
    attention_simple(q, cache.k, cache.v, cache.block_table, ctx.seq_of_token, ctx.positions, out,
                     heads, kv_heads, head_dim, status)


def sample(logits, out, status, temperature=None, uniform=None):
    """out[r] = argmax(logits[r]) where temperature[r] == 0 (or no temperature is given), else a
    draw from softmax(logits[r] / temperature[r]) at the uniform number uniform[r]."""
    _rows_contiguous(logits, "logits")
    R, V = logits.shape
    if out.numel() != R:
        raise KernelError("sample: one output per row")
    scratch = torch.empty(load_library().sprout_sample_scratch_bytes(R), dtype=torch.uint8, device=logits.device)
    _run("sprout_sample", _ptr(logits, "logits", torch.float32), logits.stride(0),
         _ptr(temperature, "temperature", torch.float32, True), _ptr(uniform, "uniform", torch.float32, True),
         _ptr(out, "out", torch.int32), _ptr(scratch, "scratch"), R, V, _ptr(status, "status", torch.int32), _stream())


def advance_decode(token_ids, positions, context_lens, sampled, history, step_counter):
    """Feed a decode step's sampled tokens back as the next step's inputs, on the device."""
    R = token_ids.numel()
    if history.dim() != 2 or history.shape[1] != R or not history.is_contiguous():
        raise KernelError("advance_decode: history must be contiguous [max_steps, requests]")
    _run("sprout_advance_decode", _ptr(token_ids, "token_ids", torch.int32), _ptr(positions, "positions", torch.int32),
         _ptr(context_lens, "context_lens", torch.int32), _ptr(sampled, "sampled", torch.int32),
         _ptr(history, "history", torch.int32), _ptr(step_counter, "step_counter", torch.int32), R,
         history.shape[0], _stream())


def feed_tokens(token_ids, rows, fed, vocab: int):
    """token_ids[r] = fed[rows[r]] where rows[r] >= 0: a step launched before its predecessor has
    been read back takes the predecessor's sampled tokens on the device."""
    if rows.numel() != token_ids.numel():
        raise KernelError("feed_tokens: one row index per token")
    _run("sprout_feed_tokens", _ptr(token_ids, "token_ids", torch.int32), _ptr(rows, "rows", torch.int32),
         _ptr(fed, "fed", torch.int32), token_ids.numel(), fed.numel(), vocab, _stream())


# ---------------------------------------------------------------------------------- sum-then-norm streams, latent attention

def scale_cast(x, y, h, alpha: float):
    """y = alpha * x (float32) and, when ``h`` is given, h = x in h's dtype."""
    if not (x.is_contiguous() and y.is_contiguous()) or x.shape != y.shape or (h is not None and (h.shape != x.shape or not h.is_contiguous())):
        raise KernelError("scale_cast: x, y and h must be contiguous and of one shape")
    _run("sprout_scale_cast", _ptr(x, "x", torch.float32), _ptr(y, "y", torch.float32), _ptr(h, "h", allow_none=True),
         _dtype_code(h.dtype) if h is not None else F32, float(alpha), x.numel(), _stream())


def sum_norm(y, gain, x, eps: float, y2=None, h=None, alpha: float = 1.0, history=None, weights=None, n: int = 0):
    """x = rmsnorm(y) * gain (float32; ``x`` may be ``y``); optionally y2 = alpha * x (may be ``y``)
    and h = x in h's dtype, for the sublayer that follows.  With ``history`` (float32 [entries, rows, hidden]) and
    ``weights``: the normed rows become entry n + 1 of the history and x, y2 and h are made from
    sum_{j <= n + 1} weights[j] * history[j] instead (``depth_average`` folded in)."""
    if y.dim() != 2 or not y.is_contiguous() or not x.is_contiguous() or x.shape != y.shape or gain.numel() != y.shape[1]:
        raise KernelError("sum_norm: y and x must be contiguous [rows, hidden], gain [hidden]")
    for name, t in (("y2", y2), ("h", h)):
        if t is not None and (t.shape != y.shape or not t.is_contiguous()):
            raise KernelError(f"sum_norm: {name} must be contiguous and have y's shape")
    if history is not None and (history.dim() != 3 or not history.is_contiguous() or tuple(history.shape[1:]) != tuple(y.shape)
                                or weights is None or not 0 <= n + 1 < history.shape[0] or weights.numel() < n + 2
                                or (h is not None and y2 is None)):
        raise KernelError("sum_norm: history must be contiguous [entries, rows, hidden] with n + 1 inside it and n + 2 weights")
    _run("sprout_sum_norm", _ptr(y, "y", torch.float32), _ptr(gain, "gain", torch.float32), _ptr(x, "x", torch.float32),
         _ptr(y2, "y2", torch.float32, True), _ptr(h, "h", allow_none=True), _dtype_code(h.dtype) if h is not None else F32,
         y.shape[0], y.shape[1], float(eps), float(alpha), _ptr(history, "history", torch.float32, True),
         _ptr(weights, "weights", torch.float32, True), int(n), _stream())


def polynorm(z, out, coefficients, eps: float):
    """out = a N(z) + b N(z^2) + c N(z^3) + e per row, N(v) = v / sqrt(mean(v^2) + eps);
    ``coefficients`` is a float32 device tensor (a, b, c, e)."""
    if z.dim() != 2 or not z.is_contiguous() or not out.is_contiguous() or out.shape != z.shape or coefficients.numel() != 4:
        raise KernelError("polynorm: z and out must be contiguous [rows, width], four coefficients")
    _run("sprout_polynorm", _ptr(z, "z"), _dtype_code(z.dtype), _ptr(out, "out"), _dtype_code(out.dtype),
         _ptr(coefficients, "coefficients", torch.float32), z.shape[0], z.shape[1], float(eps), _stream())


def _rotary(cos_table, sin_table, limit: int, name: str):
    if (cos_table is None) != (sin_table is None):
        raise KernelError(f"{name}: cos and sin tables go together")
    if cos_table is None:
        return None, None, 0, 0
    if cos_table.shape != sin_table.shape or cos_table.dim() != 2 or not 0 < 2 * cos_table.shape[1] <= limit \
            or not cos_table.is_contiguous() or not sin_table.is_contiguous():
        raise KernelError(f"{name}: cos/sin tables must be contiguous [max_positions, rotary_dim / 2] with rotary_dim <= {limit}")
    return _ptr(cos_table, "cos", torch.float32), _ptr(sin_table, "sin", torch.float32), cos_table.shape[0], 2 * cos_table.shape[1]


def latent_kv_append(src, weight, positions, seq_of_token, block_table, cos_table, sin_table, interleaved, cache, rank: int,
                     eps: float, status):
    """Row t of ``src`` (float32 [tokens, >= rank + rot], unit inner stride) is [latent | shared key part]:
    the latent is RMS-normed and multiplied by ``weight``, the key part's first ``rotary_dim`` elements
    are rotated by the token's position, and the row is stored in ``cache``
    [pages, 1, page_tokens, rank + rot] at the token's place."""
    _rows_contiguous(src, "src")
    _rows_contiguous(block_table, "block_table")
    if cache.dim() != 4 or cache.shape[1] != 1 or not cache.is_contiguous() or cache.shape[3] < rank:
        raise KernelError("latent_kv_append: the cache must be contiguous [pages, 1, page_tokens, rank + rot]")
    rot = cache.shape[3] - rank
    T = src.shape[0]
    if src.shape[1] < rank + rot or weight.numel() != rank or positions.numel() != T or seq_of_token.numel() != T:
        raise KernelError("latent_kv_append: shapes do not fit")
    cos, sin, table_positions, rotary_dim = _rotary(cos_table, sin_table, max(rot, 1), "latent_kv_append")
    _run("sprout_latent_kv_append", _ptr(src, "src", torch.float32), src.stride(0), _ptr(weight, "weight", torch.float32),
         _ptr(positions, "positions", torch.int32), _ptr(seq_of_token, "seq_of_token", torch.int32),
         _ptr(block_table, "block_table", torch.int32), block_table.stride(0), cos, sin, table_positions, rotary_dim,
         1 if interleaved else 0, _ptr(cache, "cache"), _dtype_code(cache.dtype), T, rank, rot, cache.shape[2], cache.shape[0],
         float(eps), _ptr(status, "status", torch.int32), _stream())


def latent_query_tail(q, qlat, positions, cos_table, sin_table, interleaved, heads: int, dim: int, rot: int, rank: int, status):
    """qlat[t, h, rank:] = q[t, h, dim:] with its first ``rotary_dim`` elements rotated by the token's position;
    q is [tokens, heads * (dim + rot)], qlat [tokens, heads * (rank + rot)]."""
    T = q.shape[0]
    if not q.is_contiguous() or not qlat.is_contiguous() or q.dtype != qlat.dtype or tuple(q.shape) != (T, heads * (dim + rot)) \
            or tuple(qlat.shape) != (T, heads * (rank + rot)) or positions.numel() != T:
        raise KernelError("latent_query_tail: shapes do not fit")
    cos, sin, table_positions, rotary_dim = _rotary(cos_table, sin_table, max(rot, 1), "latent_query_tail")
    _run("sprout_latent_query_tail", _ptr(q, "q"), _ptr(qlat, "qlat"), _dtype_code(q.dtype), _ptr(positions, "positions", torch.int32),
         cos, sin, table_positions, rotary_dim, 1 if interleaved else 0, T, heads, dim, rot, rank,
         _ptr(status, "status", torch.int32), _stream())


def headwise_gemm(a, weight, out, heads: int, a_head_stride: int, out_head_stride: int):
    """out[t, h, :n] = weight[h] @ a[t, h, :k] for every head: ``weight`` is contiguous [heads, n, k];
    head h's input starts at column h * a_head_stride of ``a``'s rows, its output at column
    h * out_head_stride of ``out``'s rows.  float32 accumulation in ascending k."""
    _rows_contiguous(a, "a")
    _rows_contiguous(out, "out")
    if weight.dim() != 3 or weight.shape[0] != heads or not weight.is_contiguous() or a.dtype != weight.dtype or out.dtype != a.dtype:
        raise KernelError("headwise_gemm: weight must be contiguous [heads, n, k] of the activations' dtype")
    n, k = weight.shape[1], weight.shape[2]
    if a.shape[0] != out.shape[0] or (heads - 1) * a_head_stride + k > a.shape[1] or (heads - 1) * out_head_stride + n > out.shape[1]:
        raise KernelError("headwise_gemm: the heads do not fit the rows")
    _run("sprout_headwise_gemm", _ptr(a, "a"), a.stride(0), a_head_stride, _ptr(weight, "weight"), _ptr(out, "out"), out.stride(0),
         out_head_stride, _dtype_code(a.dtype), a.shape[0], heads, n, k, _stream())


def latent_attention_simple(qlat, cache, block_table, seq_of_token, positions, sink, out, heads: int, rank: int, scale: float, status):
    """Causal attention of every (token, head) row of ``qlat`` [tokens, heads * width] over the rows of
    its request in ``cache`` [pages, 1, page_tokens, width]: score = scale * (row . key row), value = the
    key row's first ``rank`` elements; ``sink`` (float32 [heads] or None) adds exp(sink[h]) to the softmax
    denominator.  out [tokens, heads * rank].  float32 arithmetic; the true 32-bit path."""
    T = qlat.shape[0]
    width = cache.shape[3]
    if cache.dim() != 4 or cache.shape[1] != 1 or not cache.is_contiguous() or cache.dtype != qlat.dtype or out.dtype != qlat.dtype \
            or not qlat.is_contiguous() or not out.is_contiguous() or tuple(qlat.shape) != (T, heads * width) \
            or tuple(out.shape) != (T, heads * rank) or (sink is not None and sink.numel() != heads):
        raise KernelError("latent_attention_simple: shapes or dtypes do not fit")
    _rows_contiguous(block_table, "block_table")
    _run("sprout_latent_attention_simple", _ptr(qlat, "qlat"), _ptr(cache, "cache"), _ptr(block_table, "block_table", torch.int32),
         block_table.stride(0), _ptr(seq_of_token, "seq_of_token", torch.int32), _ptr(positions, "positions", torch.int32),
         _ptr(sink, "sink", torch.float32, True), _ptr(out, "out"), _dtype_code(qlat.dtype), T, heads, width, rank,
         cache.shape[2], cache.shape[0], float(scale), _ptr(status, "status", torch.int32), _stream())


def latent_attention_mma_supported(width: int, rank: int) -> bool:
    """Whether the tensor-core latent attention kernels take rows of ``width`` with a latent of ``rank``
    (multiples of 16 whose stages fit shared memory)."""
    lib = _lib or load_library()
    return bool(lib.sprout_latent_attention_mma_supported(int(width), int(rank)))


def latent_split_plan(requests: int, heads: int, rank: int, planned_keys: int, width: int = 0) -> tuple[int, int]:
    """(ranges, keys per range) for a step of one token per request: as many CTAs as the SMs hold at once
    (one per SM for wide rows, whose two stages fill its shared memory), ranges of a multiple of 64 keys, at
    most 64 of them.  It follows the contexts' length alone, so a captured step is replayed for steps that
    plan alike."""
    groups, along_y = -(-heads // 16), 1 if rank <= 512 else -(-rank // 512)
    row_bytes = (max(width, rank) + 8) * 2
    blocks = 1 if rank <= 128 else 2 if rank <= 256 else 4             # of 128 value columns, four warps each
    shared = 16 * row_bytes + max(128 * row_bytes, blocks * 4 * 16 * 128 * 4)
    per_sm = max(1, min(4 // blocks, 232448 // (shared + 18432)))       # by registers (128 a thread) and by shared memory
    stages = max(1, -(-planned_keys // 64))
    # a range is worth its fixed costs (query rows, exchange, partial sums through memory) from four stages on
    splits = max(1, min(per_sm * sm_count() // max(1, requests * groups * along_y), stages // 4, 64))
    split_keys = -(-stages // splits) * 64
    return max(1, -(-planned_keys // split_keys)), split_keys


def latent_attention_mma(qlat, cache, block_table, q_start, positions, context_lens, sink, out, heads: int, rank: int,
                         scale: float, status, requests: int, splits: int = 0, split_keys: int = 0):
    """The tensor-core form of ``latent_attention_simple`` (bfloat16).  ``splits`` 0: rows of any mix of
    portions and single tokens, 64 to a CTA.  ``splits`` >= 1: one token per request, its keys divided into
    ranges of ``split_keys`` that are merged through float32 scratch."""
    T = qlat.shape[0]
    width = cache.shape[3]
    if cache.dim() != 4 or cache.shape[1] != 1 or not cache.is_contiguous() or cache.dtype != torch.bfloat16 \
            or qlat.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or not qlat.is_contiguous() or not out.is_contiguous() \
            or tuple(qlat.shape) != (T, heads * width) or tuple(out.shape) != (T, heads * rank) \
            or (sink is not None and sink.numel() != heads) or q_start.numel() != requests + 1 or positions.numel() != T:
        raise KernelError("latent_attention_mma: shapes or dtypes do not fit")
    _rows_contiguous(block_table, "block_table")
    scratch = None
    if splits:
        if T != requests or context_lens is None or context_lens.numel() != requests:
            raise KernelError("latent_attention_mma: split keys need one token and one context length per request")
        scratch = torch.empty(requests * splits * heads * (rank + 2), dtype=torch.float32, device=qlat.device)
    _run("sprout_latent_attention_mma", _ptr(qlat, "qlat"), _ptr(cache, "cache"), _ptr(block_table, "block_table", torch.int32),
         block_table.stride(0), _ptr(q_start, "q_start", torch.int32), _ptr(positions, "positions", torch.int32),
         _ptr(context_lens, "context_lens", torch.int32, True), _ptr(sink, "sink", torch.float32, True), _ptr(out, "out"),
         _ptr(scratch, "scratch", torch.float32, True), T, requests, heads, width, rank, cache.shape[2], cache.shape[0],
         int(splits), int(split_keys), float(scale), _ptr(status, "status", torch.int32), _stream())
    if splits:
        global LAUNCHES
        LAUNCHES += 1                       # the merge kernel


LATENT_ATTENTION = os.environ.get("SPROUT_LATENT_ATTENTION", "auto")      # "simple": the float32-arithmetic kernel for every step


def latent_attention(qlat, cache, ctx, sink, out, heads: int, rank: int, scale: float, status):
    """Latent attention of the step's rows over their requests' pages (``cache`` is a CacheView whose
    key buffer holds the rows).  float32 runs the plain kernel (the true 32-bit path), and so do sizes the
    tensor-core kernels do not take; bfloat16 runs the split-key kernel when every request brings one
    token and the whole-rows kernel otherwise."""
    width = cache.k.shape[3]
    if qlat.dtype != torch.bfloat16 or LATENT_ATTENTION == "simple" or not latent_attention_mma_supported(width, rank):
        return latent_attention_simple(qlat, cache.k, cache.block_table, ctx.seq_of_token, ctx.positions, sink, out, heads, rank,
                                       scale, status)
    splits = split_keys = 0
    if ctx.max_q_len == 1:
        splits, split_keys = latent_split_plan(ctx.num_seqs, heads, rank, ctx.planned_context or ctx.max_context, width)
    latent_attention_mma(qlat, cache.k, cache.block_table, ctx.q_start, ctx.positions, ctx.context_lens, sink, out, heads, rank,
                         scale, status, ctx.num_seqs, splits, split_keys)


def depth_average(history, x, weights, n: int):
    """history[n + 1] = x, then x = sum over j <= n + 1 of weights[j] * history[j]; history is float32
    [entries, rows, width], x float32 [rows, width], weights float32 with at least n + 2 entries."""
    if history.dim() != 3 or not history.is_contiguous() or not x.is_contiguous() or tuple(history.shape[1:]) != tuple(x.shape) \
            or not 0 <= n + 1 < history.shape[0] or weights.numel() < n + 2:
        raise KernelError("depth_average: shapes do not fit")
    _run("sprout_depth_average", _ptr(history, "history", torch.float32), _ptr(x, "x", torch.float32),
         _ptr(weights, "weights", torch.float32), int(n), x.numel(), _stream())


def softcap(x, cap: float):
    """x = cap * tanh(x / cap) in place (float32)."""
    if not x.is_contiguous():
        raise KernelError("softcap: x must be contiguous")
    _run("sprout_softcap", _ptr(x, "x", torch.float32), float(cap), x.numel(), _stream())


# ---------------------------------------------------------------------------------- layers wrapped in two norms, activations

def layernorm(x, gain, out, eps: float, rows=None, bias=None):
    """out[r] = (x[r] - mean) / sqrt(var + eps) * gain (+ bias) of row r (or of row rows[r]); x float32, out float32 or
    bfloat16."""
    if x.dim() != 2 or out.dim() != 2 or not x.is_contiguous() or not out.is_contiguous():
        raise KernelError("layernorm: x and out must be contiguous 2-D")
    R, H = out.shape
    if x.shape[1] != H or gain.numel() != H or (rows is None and x.shape[0] != R) or (rows is not None and rows.numel() != R):
        raise KernelError("layernorm: shapes do not fit")
    if bias is not None and bias.numel() != H:
        raise KernelError("layernorm: the bias has one entry per column")
    _run("sprout_layernorm", _ptr(x, "x", torch.float32), _ptr(gain, "gain", torch.float32),
         _ptr(bias, "bias", torch.float32, allow_none=True), _ptr(out, "out"),
         _dtype_code(out.dtype), _ptr(rows, "rows", torch.int32, allow_none=True), R, H, float(eps), _stream())


def norm_add(y, gain, x, eps: float, next_gain=None, h=None):
    """x += layernorm(y) * gain (float32, in place); with ``next_gain`` and ``h`` also h = layernorm(x) * next_gain of
    the new x, in h's dtype: the norm after a sublayer, the residual sum and the norm before the next sublayer."""
    if y.dim() != 2 or not y.is_contiguous() or not x.is_contiguous() or x.shape != y.shape or gain.numel() != y.shape[1]:
        raise KernelError("norm_add: y and x must be contiguous [rows, width], gain [width]")
    if (next_gain is None) != (h is None) or (h is not None and (h.shape != x.shape or not h.is_contiguous()
                                                                   or next_gain.numel() != y.shape[1])):
        raise KernelError("norm_add: the next norm's gain and its output go together and have x's width")
    _run("sprout_norm_add", _ptr(y, "y", torch.float32), _ptr(gain, "gain", torch.float32), _ptr(x, "x", torch.float32),
         _ptr(next_gain, "next_gain", torch.float32, True), _ptr(h, "h", allow_none=True),
         _dtype_code(h.dtype) if h is not None else F32, y.shape[0], y.shape[1], float(eps), _stream())


def gated_rmsnorm(o, gain, gate, out, eps: float):
    """out = o / sqrt(mean(o^2) + eps) * gain * sigmoid(gate); o float32 [rows, width], gate a view [rows, width] with
    unit inner stride of out's dtype."""
    _rows_contiguous(gate, "gate")
    if o.dim() != 2 or not o.is_contiguous() or not out.is_contiguous() or out.shape != o.shape or gate.shape != o.shape \
            or gate.dtype != out.dtype or gain.numel() != o.shape[1]:
        raise KernelError("gated_rmsnorm: shapes or dtypes do not fit")
    _run("sprout_gated_rmsnorm", _ptr(o, "o", torch.float32), _ptr(gain, "gain", torch.float32), _ptr(gate, "gate"),
         gate.stride(0), _ptr(out, "out"), _dtype_code(out.dtype), o.shape[0], o.shape[1], float(eps), _stream())


def relu2(z, out):
    """out = max(z, 0)^2 element by element."""
    if not z.is_contiguous() or not out.is_contiguous() or z.shape != out.shape or z.dtype != out.dtype:
        raise KernelError("relu2: z and out must be contiguous and alike")
    _run("sprout_relu2", _ptr(z, "z"), _ptr(out, "out"), _dtype_code(z.dtype), z.numel(), _stream())


def glu_clamped(gate_up, out, limit: float, alpha: float):
    """out = g sigmoid(alpha g) (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit); rows of ``gate_up``
    hold the gate values first and the up values after them."""
    R, ff = out.shape
    if not gate_up.is_contiguous() or not out.is_contiguous() or tuple(gate_up.shape) != (R, 2 * ff) or gate_up.dtype != out.dtype:
        raise KernelError("glu_clamped: gate_up must be contiguous [rows, 2 ff] of out's dtype")
    _run("sprout_glu_clamped", _ptr(gate_up, "gate_up"), _ptr(out, "out"), _dtype_code(out.dtype), R, ff, float(limit),
         float(alpha), _stream())


# ---------------------------------------------------------------------------------- attention with one or two maps per head

def rope_maps_append(rows, positions, seq_of_token, block_table, cos_table, sin_table, k_cache, v_cache, q_vectors: int,
                     kv_heads: int, maps: int, dim: int, vdim: int, page_tokens: int, write: bool, status,
                     unit_eps: float = 0.0, value_from_key: bool = False, q_weight=None, k_weight=None, weight_eps: float = 0.0):
    """Rotate the first ``2 * cos_table.shape[1]`` elements of every query vector (in place) and key vector by the token's
    position, half-split pairs; append keys ([pages, kv_heads, page_tokens, maps * dim]) and values
    ([pages, kv_heads, page_tokens, vdim]) when ``write``.  A row holds q_vectors * dim query elements, then (when
    ``write``) kv_heads * maps * dim key elements and kv_heads * vdim value elements.  With ``unit_eps`` > 0 every query
    and key vector is divided by its root mean square over ``dim`` after the rotation; with ``value_from_key`` the rows hold
    no value elements and the cached value row is the key row as projected (before rotation and norm).  ``q_weight`` /
    ``k_weight`` (float32 [dim]): before the rotation every query / key vector is divided by its root mean square over
    ``dim`` (``weight_eps`` inside the root) and multiplied by the weight."""
    _rows_contiguous(rows, "rows")
    for weight in (q_weight, k_weight):
        if weight is not None and (weight.dtype != torch.float32 or weight.numel() != dim or not weight.is_contiguous()):
            raise KernelError("rope_maps_append: a norm weight is float32 [dim]")
    _rows_contiguous(block_table, "block_table")
    T = rows.shape[0]
    cos_ptr, sin_ptr, max_positions, rot = _rotary(cos_table, sin_table, dim, "rope_maps_append")
    if write:
        if k_cache.dtype != rows.dtype or not k_cache.is_contiguous() or tuple(k_cache.shape[1:]) != (kv_heads, page_tokens, maps * dim):
            raise KernelError("rope_maps_append: k_cache must be contiguous [pages, kv_heads, page_tokens, maps * dim]")
        if v_cache.dtype != rows.dtype or not v_cache.is_contiguous() or tuple(v_cache.shape[1:]) != (kv_heads, page_tokens, vdim):
            raise KernelError("rope_maps_append: v_cache must be contiguous [pages, kv_heads, page_tokens, vdim]")
    _run("sprout_rope_maps_append", _ptr(rows, "rows"), rows.stride(0), _dtype_code(rows.dtype),
         _ptr(positions, "positions", torch.int32), _ptr(seq_of_token, "seq_of_token", torch.int32),
         _ptr(block_table, "block_table", torch.int32), block_table.stride(0), cos_ptr, sin_ptr, max_positions,
         _ptr(k_cache, "k_cache", allow_none=not write), _ptr(v_cache, "v_cache", allow_none=not write), T, q_vectors,
         kv_heads, maps, dim, rot, vdim, page_tokens, k_cache.shape[0] if write else 1, 1 if write else 0,
         float(unit_eps), 1 if value_from_key else 0, _ptr(q_weight, "q_weight", torch.float32, True),
         _ptr(k_weight, "k_weight", torch.float32, True), float(weight_eps), _ptr(status, "status", torch.int32), _stream())


MASK_KINDS = {"causal": 0, "window": 1, "chunk": 2}


def _mask_code(mask) -> tuple[int, int, int]:
    """(kind, size, kept first positions) of ``mask``: None or ("causal", None), ("window", n) or ("window", n, first): a
    query sees itself and the n - 1 positions before it, and the first ``first`` positions of its sequence; ("chunk", n):
    a query sees the positions of its own chunk of n, counted from position 0, up to itself."""
    if mask is None:
        return 0, 0, 0
    kind, size = mask[0], mask[1]
    keep = int(mask[2]) if len(mask) > 2 else 0
    if kind not in MASK_KINDS or (kind != "causal" and (not isinstance(size, int) or size <= 0)) or keep < 0 \
            or (keep and kind != "window"):
        raise KernelError(f"attention: unknown mask {mask!r}")
    return MASK_KINDS[kind], int(size or 0), keep


def _gate_args(gate, tokens: int, heads: int, dtype, name: str):
    if gate is None:
        return None, 0
    if gate.dim() != 2 or gate.stride(1) != 1 or gate.shape[0] != tokens or gate.shape[1] != heads or gate.dtype != dtype:
        raise KernelError(f"{name}: the gate must be a [tokens, heads] view with unit inner stride, of q's dtype")
    return gate.data_ptr(), gate.stride(0)


def multimap_attention_simple(q, cache, ctx, out, heads: int, kv_heads: int, maps: int, dim: int, vdim: int, scale: float,
                              lam: float, norm_eps: float, out_scale: float, status, mask=None, sink=None, gate=None,
                              softcap: float = 0.0):
    """Causal attention with ``maps`` (1 or 2) softmax maps per head over shared values, float32 arithmetic:
    out = (a_0 - lam a_1) [/ rms when norm_eps > 0] * out_scale per head.  q [tokens, heads * maps * dim] (a view with
    unit inner stride), out [tokens, heads * vdim].  ``mask`` says what a query sees (``_mask_code``), ``sink`` (float32
    [heads]) adds exp(sink_h) to every softmax denominator of head h, ``gate`` ([tokens, heads]) multiplies head h's output
    by sigmoid(gate); ``softcap`` > 0 turns every scaled score s into softcap * tanh(s / softcap)."""
    _rows_contiguous(q, "q")
    mask_kind, mask_size, mask_keep = _mask_code(mask)
    gate_ptr, gate_stride = _gate_args(gate, q.shape[0], heads, q.dtype, "multimap_attention")
    if sink is not None and (sink.dtype != torch.float32 or sink.numel() != heads):
        raise KernelError("multimap_attention: one float32 sink per head")
    _rows_contiguous(out, "out")
    k_cache, v_cache = cache.k, cache.v
    if k_cache.dtype != q.dtype or v_cache.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelError("multimap_attention: q, the cache and out must have one dtype")
    if tuple(k_cache.shape[1:]) != (kv_heads, cache.page_tokens, maps * dim) or tuple(v_cache.shape[1:]) != (kv_heads, cache.page_tokens, vdim):
        raise KernelError("multimap_attention: the cache's shape does not fit the heads")
    if q.shape[1] != heads * maps * dim or out.shape[1] != heads * vdim or out.shape[0] != q.shape[0]:
        raise KernelError("multimap_attention: q or out has the wrong width")
    _run("sprout_multimap_attention_simple", _ptr(q, "q"), q.stride(0), _ptr(k_cache, "k_cache"), _ptr(v_cache, "v_cache"),
         _ptr(cache.block_table, "block_table", torch.int32), cache.block_table.stride(0),
         _ptr(ctx.seq_of_token, "seq_of_token", torch.int32), _ptr(ctx.positions, "positions", torch.int32), _ptr(out, "out"),
         out.stride(0), _dtype_code(q.dtype), q.shape[0], heads, kv_heads, maps, dim, vdim, cache.page_tokens,
         k_cache.shape[0], float(scale), float(lam), float(norm_eps), float(out_scale), mask_kind, mask_size,
         _ptr(sink, "sink", torch.float32, True), gate_ptr, gate_stride, mask_keep, float(softcap),
         _ptr(status, "status", torch.int32), _stream())


# ---------------------------------------------------------------------------------- linear attention with decay and state

def decay_scan(rows, q_start, state_slots, state, decay, out, heads: int, dim: int, vdim: int, silu: bool, status):
    """Per request and head, token by token: S = decay_h S + k v^T, o = S^T q, with q, k, v (after silu when ``silu``)
    taken from ``rows`` [tokens, >= heads * (2 dim + vdim)] laid out [q | k | v]; ``state`` float32
    [slots, heads, dim, vdim] is read and written at the requests' slots; out float32 [tokens, heads * vdim]."""
    _rows_contiguous(rows, "rows")
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (heads, dim, vdim):
        raise KernelError("decay_scan: state must be contiguous float32 [slots, heads, dim, vdim]")
    if not out.is_contiguous() or tuple(out.shape) != (rows.shape[0], heads * vdim) or decay.numel() != heads:
        raise KernelError("decay_scan: out must be contiguous float32 [tokens, heads * vdim], one decay per head")
    _run("sprout_decay_scan", _ptr(rows, "rows"), rows.stride(0), _dtype_code(rows.dtype), _ptr(q_start, "q_start", torch.int32),
         _ptr(state_slots, "state_slots", torch.int32), _ptr(state, "state", torch.float32), state.shape[0],
         _ptr(decay, "decay", torch.float32), _ptr(out, "out", torch.float32), state_slots.numel(), heads, dim, vdim,
         1 if silu else 0, _ptr(status, "status", torch.int32), _stream())


# ---------------------------------------------------------------------------------- routed feed-forward

def moe_route(h, router, correction, ids, weights, counts, experts: int, top: int, scale: float, groups=None,
              renormalize: bool = True, extra_out=None):
    """Per token: softmax of the float32 router product, ``top`` largest of score + correction (lowest index first among
    equals; ``correction`` None: the scores alone), weights = taken scores / (their sum + 1e-20) * scale, or the taken
    scores * scale when not ``renormalize``.  ``groups`` = (count, keep): the outputs form ``count`` equal groups of
    neighbours, a group's score is its largest score, only outputs of the ``keep`` best groups can be taken.  ``extra_out``
    (float32 [tokens, n]): the router matrix's last n rows are not part of the softmax; their products are written there.
    ids int32 [tokens, top] (from ``experts`` on: identity experts), weights float32 [tokens, top]; counts int32 [experts] +=
    rows per real expert."""
    _rows_contiguous(h, "h")
    extra = 0 if extra_out is None else extra_out.shape[1]
    outputs, width = router.shape[0] - extra, router.shape[1]
    T = h.shape[0]
    group_count, group_keep = (int(groups[0]), int(groups[1])) if groups else (1, 1)
    if extra and (extra_out.dtype != torch.float32 or not extra_out.is_contiguous() or extra_out.shape[0] != T):
        raise KernelError("moe_route: extra_out must be contiguous float32 [tokens, extra]")
    if not router.is_contiguous() or h.shape[1] != width or (correction is not None and correction.numel() != outputs) or tuple(ids.shape) != (T, top) \
            or tuple(weights.shape) != (T, top) or not ids.is_contiguous() or not weights.is_contiguous() or counts.numel() < max(experts, 1):
        raise KernelError("moe_route: shapes do not fit")
    _run("sprout_moe_route", _ptr(h, "h"), h.stride(0), _dtype_code(h.dtype), _ptr(router, "router", torch.float32),
         _ptr(correction, "correction", torch.float32, True), _ptr(ids, "ids", torch.int32), _ptr(weights, "weights", torch.float32),
         _ptr(counts, "counts", torch.int32), T, width, outputs, experts, top, float(scale), extra,
         _ptr(extra_out, "extra_out", torch.float32, True), group_count, group_keep, 1 if renormalize else 0, _stream())


def moe_arrange(ids, counts, offsets, order, place_of, experts: int):
    """counts -> offsets [experts + 1] (counts are zeroed again); every (token, place) of a real expert gets a row in its
    expert's range: order[row] = token * top + place, place_of[token * top + place] = row (-1 for identity experts)."""
    entries = ids.numel()
    if offsets.numel() < experts + 1 or order.numel() < entries or place_of.numel() < entries:
        raise KernelError("moe_arrange: buffers too small")
    _run("sprout_moe_arrange", _ptr(ids, "ids", torch.int32), _ptr(counts, "counts", torch.int32),
         _ptr(offsets, "offsets", torch.int32), _ptr(order, "order", torch.int32), _ptr(place_of, "place_of", torch.int32),
         entries, experts, _stream())


def moe_up_plain(h, order, offsets, w_gate_up, act, experts: int, top: int, limit: float, alpha: float):
    """act[row] = glu_clamped(W_gate[e] a, W_up[e] a) for the arranged rows (a = h[order[row] // top], e the row's expert);
    w_gate_up [experts, 2 ff, width] with gate rows first; CUDA cores, float32 sums in ascending k.  ``limit`` <= 0: experts
    without a gate, act[row] = gelu(W_up[e] a) (the exact form) with w_gate_up [experts, ff, width]."""
    _rows_contiguous(h, "h")
    R, ff = act.shape
    if not w_gate_up.is_contiguous() or tuple(w_gate_up.shape) != (experts, (2 if limit > 0 else 1) * ff, h.shape[1]) or w_gate_up.dtype != h.dtype \
            or act.dtype != h.dtype or not act.is_contiguous():
        raise KernelError("moe_up: shapes or dtypes do not fit")
    _run("sprout_moe_up_plain", _ptr(h, "h"), h.stride(0), _dtype_code(h.dtype), _ptr(order, "order", torch.int32),
         _ptr(offsets, "offsets", torch.int32), _ptr(w_gate_up, "w_gate_up"), _ptr(act, "act"), R, experts, top, h.shape[1], ff,
         float(limit), float(alpha), _stream())


def moe_down_plain(act, offsets, w_down, rows_out, experts: int):
    """rows_out[row] = W_down[e] act[row] (float32) for the arranged rows; w_down [experts, width, ff]."""
    R, ff = act.shape
    width = rows_out.shape[1]
    if not w_down.is_contiguous() or tuple(w_down.shape) != (experts, width, ff) or w_down.dtype != act.dtype \
            or rows_out.dtype != torch.float32 or not rows_out.is_contiguous() or rows_out.shape[0] != R or not act.is_contiguous():
        raise KernelError("moe_down: shapes or dtypes do not fit")
    _run("sprout_moe_down_plain", _ptr(act, "act"), _dtype_code(act.dtype), _ptr(offsets, "offsets", torch.int32),
         _ptr(w_down, "w_down"), _ptr(rows_out, "rows_out", torch.float32), R, experts, width, ff, _stream())


def moe_combine(y, h, ids, weights, place_of, rows, top: int):
    """y[t] += sum over the token's places of weight * (h[t] for an identity expert, else rows[place_of])."""
    _rows_contiguous(h, "h")
    T, width = y.shape
    if not y.is_contiguous() or y.dtype != torch.float32 or h.shape != y.shape or (rows is not None and rows.shape[1] != width):
        raise KernelError("moe_combine: shapes do not fit")
    _run("sprout_moe_combine", _ptr(y, "y", torch.float32), _ptr(h, "h"), h.stride(0), _dtype_code(h.dtype),
         _ptr(ids, "ids", torch.int32), _ptr(weights, "weights", torch.float32), _ptr(place_of, "place_of", torch.int32),
         _ptr(rows, "rows", torch.float32, True), T, width, top, _stream())


def multimap_key_split(requests: int, kv_heads: int, group: int, max_q_len: int, planned_keys: int, sms: int | None = None) -> int:
    """Into how many CTAs a step of single tokens divides a request's 64-key tiles: enough to give every SM a CTA, at
    most 8, at most the tiles there are; 1 for steps with longer portions.  (Measured at 64 requests of 2,048 keys:
    with 256 CTAs already, two shares each cost 115 us against 97 undivided; with 128 CTAs, 80 against 93.)"""
    if max_q_len * group > 16:
        return 1
    tiles = max(1, -(-planned_keys // 64))
    ctas = max(1, requests * kv_heads)
    return max(1, min(8, tiles, -(-(sms or sm_count()) // ctas)))


def visible_keys(mask, context: int) -> int:
    """The most keys a query of a context of ``context`` positions sees under ``mask``, in whole 64-key tiles' reach."""
    kind, size, keep = _mask_code(mask)
    return context if kind == 0 else min(context, size + 63 + (-(-keep // 64) * 64 if keep else 0))


def multimap_attention(q, cache, ctx, out, heads: int, kv_heads: int, maps: int, dim: int, vdim: int, scale: float, lam: float,
                       norm_eps: float, out_scale: float, status, mask=None, sink=None, gate=None, softcap: float = 0.0):
    """Attention with one or two maps per head: the tensor-core kernel in bfloat16 for the sizes it is built for
    (``SPROUT_MULTIMAP_ATTENTION=simple`` keeps the float32-arithmetic kernel), else the float32-arithmetic kernel."""
    if q.dtype == torch.bfloat16 and os.environ.get("SPROUT_MULTIMAP_ATTENTION", "mma") != "simple" \
            and (_lib or load_library()).sprout_multimap_attention_mma_supported(maps, dim, vdim) \
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.stride(0) % 2 == 0:
        global LAUNCHES
        _rows_contiguous(q, "q")
        _rows_contiguous(out, "out")
        k_cache, v_cache = cache.k, cache.v
        if tuple(k_cache.shape[1:]) != (kv_heads, cache.page_tokens, maps * dim) or tuple(v_cache.shape[1:]) != (kv_heads, cache.page_tokens, vdim) \
                or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype or out.dtype != q.dtype:
            raise KernelError("multimap_attention: the cache's shape or dtype does not fit the heads")
        if q.shape[1] != heads * maps * dim or out.shape[1] != heads * vdim or out.shape[0] != q.shape[0]:
            raise KernelError("multimap_attention: q or out has the wrong width")
        requests = ctx.q_start.numel() - 1
        group = heads // kv_heads
        tiles = (q.shape[0] * group + 63) // 64 + requests
        max_q_len = int(getattr(ctx, "max_q_len", 0) or q.shape[0])
        planned = int(getattr(ctx, "planned_context", 0) or getattr(ctx, "max_context", 0) or 0)
        ksplit = multimap_key_split(requests, kv_heads, group, max_q_len, visible_keys(mask, planned)) if planned else 1
        mask_kind, mask_size, mask_keep = _mask_code(mask)
        gate_ptr, gate_stride = _gate_args(gate, q.shape[0], heads, q.dtype, "multimap_attention")
        if sink is not None and (sink.dtype != torch.float32 or sink.numel() != heads):
            raise KernelError("multimap_attention: one float32 sink per head")
        partial = None
        if ksplit > 1:
            partial = torch.empty(requests * kv_heads * ksplit * 16 * maps * (2 + vdim), dtype=torch.float32, device=q.device)
            LAUNCHES += 1           # the merge kernel behind the same call
        _run("sprout_multimap_attention_mma", _ptr(q, "q"), q.stride(0), _ptr(k_cache, "k_cache"), _ptr(v_cache, "v_cache"),
             _ptr(cache.block_table, "block_table", torch.int32), cache.block_table.stride(0),
             _ptr(ctx.q_start, "q_start", torch.int32), _ptr(ctx.positions, "positions", torch.int32), _ptr(out, "out"),
             out.stride(0), requests, tiles, max_q_len, heads, kv_heads, maps, dim, vdim,
             cache.page_tokens, k_cache.shape[0], float(scale),
             float(lam), float(norm_eps), float(out_scale), ksplit, _ptr(partial, "partial", torch.float32, True),
             mask_kind, mask_size, _ptr(sink, "sink", torch.float32, True), gate_ptr, gate_stride, mask_keep, float(softcap),
             _ptr(status, "status", torch.int32), _stream())
        return
    multimap_attention_simple(q, cache, ctx, out, heads, kv_heads, maps, dim, vdim, scale, lam, norm_eps, out_scale, status,
                              mask=mask, sink=sink, gate=gate, softcap=softcap)


CHUNKED_FROM = 8            # a step whose longest portion has at least this many tokens runs the chunked decay kernel


def decay_attention(rows, ctx, state, decay, out, heads: int, dim: int, vdim: int, silu: bool, status, chunked: bool = True):
    """Linear attention with decay over the step's tokens, from and into the requests' state slots: prompt portions
    of bfloat16 rows run 64 tokens at a time on tensor cores when the key size is one the kernel is built for
    (``SPROUT_DECAY_ATTENTION=scan`` keeps the token-by-token kernel, ``=chain`` the form in which a CTA walks its
    request's chunks in order), everything else token by token in float32.
    The chunked path replaces q, k and v in ``rows`` by their activation; ``chunked=False`` (decays outside (0, 1],
    whose powers it could not take) keeps the token-by-token kernel."""
    if chunked and rows.dtype == torch.bfloat16 and getattr(ctx, "max_q_len", 1) >= CHUNKED_FROM and os.environ.get("SPROUT_DECAY_ATTENTION", "chunks") != "scan" \
            and rows.stride(1) == 1 and rows.data_ptr() % 16 == 0 \
            and (_lib or load_library()).sprout_decay_chunks_supported(dim, vdim, rows.stride(0)):
        _rows_contiguous(rows, "rows")
        buffer = state.buffer
        if buffer.dtype != torch.float32 or not buffer.is_contiguous() or tuple(buffer.shape[1:]) != (heads, dim, vdim):
            raise KernelError("decay_attention: state must be contiguous float32 [slots, heads, dim, vdim]")
        if not out.is_contiguous() or tuple(out.shape) != (rows.shape[0], heads * vdim) or decay.numel() != heads:
            raise KernelError("decay_attention: out must be contiguous float32 [tokens, heads * vdim], one decay per head")
        global LAUNCHES
        requests = state.slots.numel()
        sums, max_chunks = None, 0
        if os.environ.get("SPROUT_DECAY_ATTENTION", "chunks") != "chain":
            # all chunks at once: scratch for every chunk's own sums, which the scan turns into the state before the chunk
            max_chunks = rows.shape[0] // 64 + requests
            sums = torch.empty((max_chunks, heads, dim, vdim), dtype=torch.float32, device=rows.device)
            LAUNCHES += 2
        _run("sprout_decay_chunks", _ptr(rows, "rows"), rows.stride(0), _ptr(ctx.q_start, "q_start", torch.int32),
             _ptr(state.slots, "state_slots", torch.int32), _ptr(buffer, "state", torch.float32), buffer.shape[0],
             _ptr(decay, "decay", torch.float32), _ptr(out, "out", torch.float32), _ptr(sums, "sums", torch.float32, True),
             max_chunks, rows.shape[0], requests, heads, dim, vdim, 1 if silu else 0, _ptr(status, "status", torch.int32), _stream())
        if silu:
            LAUNCHES += 1           # the activation pass behind the same call
        return
    decay_scan(rows, ctx.q_start, state.slots, state.buffer, decay, out, heads, dim, vdim, silu, status)


def moe_experts(h, order, offsets, w_gate_up, w_down, act, rows_out, experts: int, top: int, limit: float, alpha: float):
    """The routed experts' two products over the arranged rows: on tensor cores in bfloat16 when the sizes are
    multiples of 8 (``SPROUT_MOE=plain`` keeps the CUDA-core products), else on CUDA cores."""
    global LAUNCHES
    width, ff = h.shape[1], act.shape[1]
    if h.dtype == torch.bfloat16 and h.stride(1) == 1 and os.environ.get("SPROUT_MOE", "mma") != "plain" \
            and (_lib or load_library()).sprout_moe_mma_supported(width, ff, h.stride(0)) \
            and all(t.data_ptr() % 16 == 0 for t in (h, w_gate_up, w_down, act, rows_out)):
        _run("sprout_moe_experts_mma", _ptr(h, "h"), h.stride(0), _ptr(order, "order", torch.int32),
             _ptr(offsets, "offsets", torch.int32), _ptr(w_gate_up, "w_gate_up", torch.bfloat16),
             _ptr(w_down, "w_down", torch.bfloat16), _ptr(act, "act", torch.bfloat16), _ptr(rows_out, "rows_out", torch.float32),
             act.shape[0], experts, top, width, ff, float(limit), float(alpha), _stream())
        LAUNCHES += 1               # two kernels behind one call
        return
    moe_up_plain(h, order, offsets, w_gate_up, act, experts, top, limit, alpha)
    moe_down_plain(act, offsets, w_down, rows_out, experts)


# ---------------------------------------------------------------------------------- recurrences with a decay made from the input

SCAN_CHUNK = 64             # tokens of a chunk of the gated scan
SCAN_CHUNKED_FROM = 128     # a step whose longest portion has at least this many tokens walks chunks side by side


def _scan_view(t, name: str, width: int, dtype):
    if t.dim() != 2 or t.stride(1) != 1 or t.shape[1] != width or t.dtype != dtype:
        raise KernelError(f"gated_scan: {name} must be a [tokens, {width}] view with unit inner stride of {dtype}, got "
                          f"{tuple(t.shape)} {t.dtype}")
    return t.data_ptr(), t.stride(0)


def gated_scan(q, k, v, z, bias, ctx, state, out, heads: int, groups: int, dim: int, vdim: int, status, per_head: bool = False,
               tau: float = 1.0, q_scale: float = 1.0, a_log=None, skip=None, given=None, ones_col: bool = False):
    """Per request and head, token by token: S = diag(a) S + (c k) v^T, o = S^T (q_scale q) + skip_h v, the state float32
    [slots, heads, dim, vdim] read and written at the requests' slots (``state``: a ``StateView``-like with ``buffer`` and
    ``slots``).  q, k [tokens, groups * dim] (heads of a group share them), v [tokens, heads * vdim], views with unit inner
    stride of one dtype.  Per key channel (default): z [tokens, heads * dim] (of that dtype or float32), a = sigmoid(z + bias)^(1 / tau), c = 1.
    ``per_head``: z [tokens, heads], dt = softplus(z + bias), a = exp(-exp(a_log) dt) for all of the head's channels, c = dt.
    ``given`` = (a, c), float32 [tokens, heads] each: the decay and the factor on k per head, ready-made (z and bias are None).
    ``ones_col``: the value rows are narrower than the state, v [tokens, heads * v_cols] with v_cols < vdim, and the state's
    column v_cols is fed the constant 1 as a value (the columns after it 0): that column of the state is then the sum of the
    decayed c k, and that column of the output its product with q_scale q, a normaliser.
    out float32 [tokens, heads * vdim].  A step whose longest portion has ``SCAN_CHUNKED_FROM`` tokens or more cuts the
    portions into chunks of ``SCAN_CHUNK`` tokens that are walked side by side (``SPROUT_GATED_SCAN=whole`` keeps one walk
    per request): scratch for every token's decay and every chunk's sums."""
    tokens, dtype = v.shape[0], v.dtype
    v_cols = v.shape[1] // heads if ones_col else vdim
    if ones_col and not v_cols < vdim:
        raise KernelError("gated_scan: the column of ones needs a state wider than the value rows")
    q_ptr, q_stride = _scan_view(q, "q", groups * dim, dtype)
    k_ptr, k_stride = _scan_view(k, "k", groups * dim, dtype)
    v_ptr, v_stride = _scan_view(v, "v", heads * v_cols, dtype)
    if given is not None:
        per_head = True
        z_f32, z_ptr, z_stride = True, None, 0
        for t in given:
            if t.dtype != torch.float32 or not t.is_contiguous() or t.numel() != tokens * heads:
                raise KernelError("gated_scan: ready-made decays are contiguous float32 [tokens, heads]")
    else:
        z_f32 = z.dtype == torch.float32                # the decay's input may be float32 beside bfloat16 projections
        z_ptr, z_stride = _scan_view(z, "z", heads if per_head else heads * dim, torch.float32 if z_f32 else dtype)
    buffer = state.buffer
    if buffer.dtype != torch.float32 or not buffer.is_contiguous() or tuple(buffer.shape[1:]) != (heads, dim, vdim):
        raise KernelError("gated_scan: state must be contiguous float32 [slots, heads, dim, vdim]")
    if not out.is_contiguous() or out.dtype != torch.float32 or tuple(out.shape) != (tokens, heads * vdim):
        raise KernelError("gated_scan: out must be contiguous float32 [tokens, heads * vdim]")
    if given is None and (bias.numel() != (heads if per_head else heads * dim) or (per_head and (a_log is None or a_log.numel() != heads))) \
            or (skip is not None and skip.numel() != heads):
        raise KernelError("gated_scan: the decay's constants do not fit the heads")
    global LAUNCHES
    requests = state.slots.numel()
    da = dc = sums = prods = None
    max_chunks = 0
    if getattr(ctx, "max_q_len", 1) >= SCAN_CHUNKED_FROM and os.environ.get("SPROUT_GATED_SCAN", "chunks") != "whole":
        max_chunks = tokens // SCAN_CHUNK + requests
        if given is None:
            da = torch.empty(tokens * (heads if per_head else heads * dim), dtype=torch.float32, device=v.device)
            dc = torch.empty(tokens * heads, dtype=torch.float32, device=v.device) if per_head else None
        sums = torch.empty((max_chunks, heads, dim, vdim), dtype=torch.float32, device=v.device)
        prods = torch.empty((max_chunks, heads, dim), dtype=torch.float32, device=v.device)
        LAUNCHES += 3 if given is None else 2               # decays, chunk sums and the carry behind the same call
    if given is not None:
        da, dc = given
    _run("sprout_gated_scan", q_ptr, q_stride, k_ptr, k_stride, v_ptr, v_stride, z_ptr, z_stride, 1 if z_f32 else 0,
         _dtype_code(dtype), _ptr(bias, "bias", torch.float32, True), _ptr(a_log, "a_log", torch.float32, True), _ptr(skip, "skip", torch.float32, True),
         1.0 / float(tau), float(q_scale), 2 if given is not None else 1 if per_head else 0, state.slots.numel(), heads, groups, dim, vdim,
         _ptr(ctx.q_start, "q_start", torch.int32), _ptr(state.slots, "state_slots", torch.int32),
         _ptr(buffer, "state", torch.float32), buffer.shape[0], _ptr(out, "out", torch.float32),
         _ptr(status, "status", torch.int32), tokens, SCAN_CHUNK, max_chunks, _ptr(da, "decays", torch.float32, True),
         _ptr(dc, "steps", torch.float32, True), _ptr(sums, "sums", torch.float32, True), _ptr(prods, "products", torch.float32, True),
         v_cols, 1 if ones_col else 0, _stream())


def causal_conv(rows, weight, bias, out, ctx, state, status, silu: bool = True):
    """out[t, c] = act(bias[c] + sum_j weight[c, j] x[t - (taps - 1 - j), c]) per request, zeros before its first token;
    ``rows`` and ``out`` are [tokens, channels] views with unit inner stride of one dtype, weight float32 [channels, taps];
    the state float32 [slots, taps - 1, channels] holds each request's last taps - 1 inputs and is brought up to date."""
    channels, taps = weight.shape
    buffer = state.buffer
    if rows.dim() != 2 or rows.stride(1) != 1 or out.stride(1) != 1 or rows.shape != out.shape or rows.shape[1] != channels \
            or rows.dtype != out.dtype:
        raise KernelError("causal_conv: rows and out must be [tokens, channels] views of one dtype")
    if weight.dtype != torch.float32 or not weight.is_contiguous() or (bias is not None and bias.numel() != channels):
        raise KernelError("causal_conv: weight must be contiguous float32 [channels, taps], one bias per channel")
    if buffer.dtype != torch.float32 or not buffer.is_contiguous() or tuple(buffer.shape[1:]) != (taps - 1, channels):
        raise KernelError("causal_conv: state must be contiguous float32 [slots, taps - 1, channels]")
    _run("sprout_causal_conv", rows.data_ptr(), rows.stride(0), _ptr(weight, "weight", torch.float32),
         _ptr(bias, "bias", torch.float32, True), out.data_ptr(), out.stride(0), _dtype_code(rows.dtype),
         _ptr(ctx.q_start, "q_start", torch.int32), _ptr(state.slots, "state_slots", torch.int32),
         _ptr(buffer, "state", torch.float32), buffer.shape[0], state.slots.numel(), int(ctx.max_q_len), channels, taps,
         1 if silu else 0, _ptr(status, "status", torch.int32), _stream())


def gated_group_norm(o, gate, weight, out, eps: float, groups: int = 1, gate_first: bool = False, silu: bool = True):
    """Rows of ``o`` (float32 [rows, width]) in ``groups`` equal parts, each divided by its root mean square (eps inside
    the root), times ``weight`` (float32; it repeats every weight.numel() elements: a weight per head, or one for the whole
    row), times act(gate), act = silu or sigmoid; with ``gate_first`` the gate is applied before the norm.  ``gate`` is a
    [rows, width] view with unit inner stride of out's dtype."""
    _rows_contiguous(gate, "gate")
    rows, width = o.shape
    if not o.is_contiguous() or o.dtype != torch.float32 or not out.is_contiguous() or out.shape != o.shape \
            or gate.shape != o.shape or gate.dtype != out.dtype or width % weight.numel() or width % groups:
        raise KernelError("gated_group_norm: shapes or dtypes do not fit")
    _run("sprout_gated_group_norm", _ptr(o, "o", torch.float32), _ptr(gate, "gate"), gate.stride(0),
         _ptr(weight, "weight", torch.float32), weight.numel(), _ptr(out, "out"), _dtype_code(out.dtype), rows, width,
         int(groups), float(eps), 1 if gate_first else 0, 1 if silu else 0, _stream())


def scaled_sum(x, y1, a: float, y2=None, b: float = 0.0):
    """x += a * y1 (+ b * y2), float32, element by element."""
    if x.dtype != torch.float32 or not x.is_contiguous() or y1.shape != x.shape or not y1.is_contiguous() \
            or (y2 is not None and (y2.shape != x.shape or not y2.is_contiguous())):
        raise KernelError("scaled_sum: contiguous float32 tensors of one shape")
    _run("sprout_scaled_sum", _ptr(x, "x", torch.float32), _ptr(y1, "y1", torch.float32), float(a),
         _ptr(y2, "y2", torch.float32, True), float(b), x.numel(), _stream())


# ---------------------------------------------------------------------------------- a matrix memory with exponential gates

def exp_gates(zi, zf, bias_i, bias_f, cap: float, ctx, top_state, slots, status):
    """The gates of a matrix memory with exponential gates and a running maximum, for every token of the step: with
    i = cap tanh((zi + bias_i) / cap) and f = logsigmoid(cap tanh((zf + bias_f) / cap)) (``cap`` <= 0: no cap) per head, and m
    the running maximum carried in ``top_state`` (float32 [slots, heads], zero for a new request):
    m_t = max(f_t + m_(t-1), i_t), a_t = exp(f_t + m_(t-1) - m_t), c_t = exp(i_t - m_t).  zi, zf: float32 [tokens, heads] views
    with one row stride.  Returns (a, c, m), float32 [tokens, heads] each; ``top_state`` is brought up to date."""
    tokens, heads = zi.shape
    if zi.dtype != torch.float32 or zf.dtype != torch.float32 or zi.stride(1) != 1 or zf.stride(1) != 1 or zf.shape != zi.shape \
            or zi.stride(0) != zf.stride(0):
        raise KernelError("exp_gates: the gates' inputs are float32 [tokens, heads] views of equal strides")
    if top_state.dtype != torch.float32 or not top_state.is_contiguous() or tuple(top_state.shape[1:]) != (heads,):
        raise KernelError("exp_gates: the running maxima are contiguous float32 [slots, heads]")
    a, c, m = (torch.empty((tokens, heads), dtype=torch.float32, device=zi.device) for _ in range(3))
    _run("sprout_exp_gates", zi.data_ptr(), zf.data_ptr(), zi.stride(0), _ptr(bias_i, "bias_i", torch.float32, True),
         _ptr(bias_f, "bias_f", torch.float32, True), float(cap), slots.numel(), heads, _ptr(ctx.q_start, "q_start", torch.int32),
         _ptr(slots, "state_slots", torch.int32), _ptr(top_state, "top_state", torch.float32), top_state.shape[0],
         _ptr(a, "a", torch.float32), _ptr(c, "c", torch.float32), _ptr(m, "m", torch.float32), _ptr(status, "status", torch.int32),
         _stream())
    return a, c, m


def exp_memory_out(o, m, gate, weight, out, heads: int, vdim: int, eps: float, out_scale: float = 1.0):
    """The scan's rows into the mixer's gated, normed output: o float32 [tokens, heads * cols] holds per head ``vdim`` outputs
    and then n . q; out[t, h] = (o / (max(|n . q|, exp(-m)) + 1e-6)) / rms * weight[h] * sigmoid(gate[t, h]) * out_scale, rms over
    the head's ``vdim`` values (eps inside the root).  gate: a [tokens, heads * vdim] view (float32, or out's dtype)."""
    tokens = o.shape[0]
    cols = o.shape[1] // heads
    _rows_contiguous(gate, "gate")
    if o.dtype != torch.float32 or not o.is_contiguous() or cols <= vdim or m.numel() != tokens * heads or weight.numel() != heads * vdim \
            or tuple(out.shape) != (tokens, heads * vdim) or not out.is_contiguous() or gate.shape[1] != heads * vdim \
            or gate.dtype not in (torch.float32, out.dtype):
        raise KernelError("exp_memory_out: shapes or dtypes do not fit")
    _run("sprout_exp_memory_out", _ptr(o, "o", torch.float32), cols, _ptr(m, "m", torch.float32), gate.data_ptr(), gate.stride(0),
         1 if gate.dtype == torch.float32 else 0, _ptr(weight, "weight", torch.float32), _ptr(out, "out"), _dtype_code(out.dtype),
         tokens, heads, vdim, float(eps), float(out_scale), _stream())


# ---------------------------------------------------------------------------------- rows of feed-forwards and of inputs to the stream

ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "gelu_erf": 2}


def unit_act(rows, out, activation: str, gated: bool, row_logits=None):
    """out = act(gate) * up for rows [gate: ff | up: ff] (``gated``), or act(rows) for rows of ff elements; ``rows`` and
    ``out`` are views with unit inner stride of one dtype.  ``row_logits`` (a float32 view with one number per row): row r is
    also multiplied by sigmoid(row_logits[r])."""
    _rows_contiguous(rows, "rows")
    _rows_contiguous(out, "out")
    ff = out.shape[1]
    if activation not in ACTIVATIONS or rows.dtype != out.dtype or rows.shape[0] != out.shape[0] or rows.shape[1] < (2 if gated else 1) * ff:
        raise KernelError("unit_act: shapes, dtypes or the activation's name do not fit")
    if row_logits is not None and (row_logits.dtype != torch.float32 or row_logits.shape[0] != out.shape[0]):
        raise KernelError("unit_act: one float32 logit per row")
    _run("sprout_unit_act", rows.data_ptr(), rows.stride(0), out.data_ptr(), out.stride(0), _dtype_code(out.dtype), out.shape[0], ff,
         ACTIVATIONS[activation], 1 if gated else 0, None if row_logits is None else row_logits.data_ptr(),
         0 if row_logits is None else row_logits.stride(0), _stream())


SIDE_FEW_TOKENS = 32        # up to this many tokens the per-layer token input runs as two light launches
SIDE_FEW_MAX_DIM = 512


def side_input_few(x, w_gate, w_proj, weight, table, first: int, token_ids, eps: float, status):
    """x[t] += rmsnorm(W_proj (gelu_tanh(W_gate x[t]) * table[token_ids[t], first : first + dim])) * weight for a handful
    of tokens in two launches (the gated row; the projection with norm and sum): x float32 [tokens, width], w_gate [dim, width], w_proj [width, dim] and table [vocab, columns]
    contiguous of one dtype (the stream and the intermediate results are rounded to it as the separate kernels round them)."""
    tokens, width = x.shape
    dim = w_gate.shape[0]
    if x.dtype != torch.float32 or not x.is_contiguous() or tuple(w_gate.shape) != (dim, width) or tuple(w_proj.shape) != (width, dim) \
            or not w_gate.is_contiguous() or not w_proj.is_contiguous() or not table.is_contiguous() or w_gate.dtype != w_proj.dtype \
            or table.dtype != w_gate.dtype or weight.numel() != width or token_ids.numel() != tokens:
        raise KernelError("side_input_few: shapes or dtypes do not fit")
    global LAUNCHES
    g = torch.empty((tokens, dim), dtype=torch.float32, device=x.device)
    _run("sprout_side_input_few", _ptr(x, "x", torch.float32), _ptr(w_gate, "w_gate"), _ptr(w_proj, "w_proj"),
         _ptr(weight, "weight", torch.float32), _ptr(table, "table"), table.shape[1], int(first), _ptr(token_ids, "token_ids", torch.int32),
         table.shape[0], _dtype_code(w_gate.dtype), tokens, width, dim, float(eps), _ptr(g, "g", torch.float32),
         _ptr(status, "status", torch.int32), _stream())
    LAUNCHES += 1               # two kernels behind one call


def side_gate(z, table, first: int, token_ids, out, status):
    """out[t, j] = gelu_tanh(z[t, j]) * table[token_ids[t], first + j]; z a view with unit inner stride, table contiguous
    [vocab, columns], out contiguous [tokens, dim], all of one dtype."""
    _rows_contiguous(z, "z")
    tokens, dim = out.shape
    if z.dtype != out.dtype or table.dtype != out.dtype or not table.is_contiguous() or not out.is_contiguous() \
            or z.shape[0] != tokens or z.shape[1] < dim or first < 0 or first + dim > table.shape[1] or token_ids.numel() != tokens:
        raise KernelError("side_gate: shapes or dtypes do not fit")
    _run("sprout_side_gate", z.data_ptr(), z.stride(0), _ptr(table, "table"), table.shape[1], int(first),
         _ptr(token_ids, "token_ids", torch.int32), table.shape[0], _ptr(out, "out"), _dtype_code(out.dtype), tokens, dim,
         _ptr(status, "status", torch.int32), _stream())


def rms_add(y, weight, x, eps: float):
    """x += y / sqrt(mean(y^2) + eps) * weight, row by row; float32."""
    if y.dtype != torch.float32 or x.dtype != torch.float32 or y.shape != x.shape or not y.is_contiguous() or not x.is_contiguous() \
            or weight.numel() != x.shape[1]:
        raise KernelError("rms_add: contiguous float32 rows of one shape and a weight per column")
    _run("sprout_rms_add", _ptr(y, "y", torch.float32), _ptr(weight, "weight", torch.float32), _ptr(x, "x", torch.float32),
         x.shape[0], x.shape[1], float(eps), _stream())


def add_rows(x, vec, other=None):
    """x[t] += vec (+ other[t]); float32."""
    if x.dtype != torch.float32 or not x.is_contiguous() or vec.numel() != x.shape[1] or not vec.is_contiguous() \
            or (other is not None and (other.shape != x.shape or not other.is_contiguous() or other.dtype != torch.float32)):
        raise KernelError("add_rows: contiguous float32 rows and a vector of their width")
    _run("sprout_add_rows", _ptr(x, "x", torch.float32), _ptr(other, "other", torch.float32, True), _ptr(vec, "vec", torch.float32),
         x.shape[0], x.shape[1], _stream())


def gated_rows_add(x, y, logits):
    """x[t] += sigmoid(logits[t]) * y[t]; x, y contiguous float32 [tokens, width], logits a float32 view with one number per row."""
    if x.dtype != torch.float32 or y.dtype != torch.float32 or x.shape != y.shape or not x.is_contiguous() or not y.is_contiguous() \
            or logits.dtype != torch.float32 or logits.shape[0] != x.shape[0]:
        raise KernelError("gated_rows_add: shapes or dtypes do not fit")
    _run("sprout_gated_rows_add", _ptr(x, "x", torch.float32), _ptr(y, "y", torch.float32), logits.data_ptr(), logits.stride(0),
         x.shape[0], x.shape[1], _stream())


def narrow_rows(x):
    """The float32 rows ``x`` as a new bfloat16 tensor (round to nearest even)."""
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("narrow_rows: contiguous float32 rows")
    out = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
    _run("sprout_narrow_rows", _ptr(x, "x", torch.float32), _ptr(out, "out", torch.bfloat16), x.numel(), _stream())
    return out


def describe_status(word: int) -> str:
    return "; ".join(text for bit, text in STATUS_BITS.items() if word & bit) or "ok"


__all__ = ["KernelError", "BuildError", "load_library", "library_file", "embed", "rmsnorm", "swiglu",
           "rope_append", "gemm_simple", "gemm_bf16", "attention_simple", "attention_decode", "attention_decode_fused", "attention_decode_resident", "decode_attention_plan", "decode_fusable", "attention_prefill",
           "paged_attention", "sample", "advance_decode", "feed_tokens", "describe_status"]
