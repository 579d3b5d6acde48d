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


_P, _I, _F = c_void_p, c_int, c_float
_SIGNATURES = {
    "sprout_embed": [_P, _I, _P, _P, _I, _I, _I, _P, _P],
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

def embed(table, tokens, out, status):
    """out[t] = table[tokens[t]] widened to float32."""
    _rows_contiguous(table, "table")
    if not table.is_contiguous() or not out.is_contiguous():
        raise KernelError("embed: table and out must be contiguous")
    T, H = out.shape
    if tokens.numel() != T or table.shape[1] != H:
        raise KernelError("embed: shapes do not fit")
    _run("sprout_embed", _ptr(table, "table"), _dtype_code(table.dtype), _ptr(tokens, "tokens", torch.int32),
         _ptr(out, "out", torch.float32), T, H, table.shape[0], _ptr(status, "status", torch.int32), _stream())


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


def gemm_bf16(a, weight, out, status, bias=None, residual=None, orientation=0, split_k=1, swiglu=False):
    """out = a @ weight.T (+ bias) (+ residual) on the tcgen05 tensor cores; a and weight bfloat16.

    ``residual`` must be ``out`` itself (float32): the product is added in place.  orientation 0
    lets the kernel choose (weight rows on the MMA's M axis for up to 128 tokens), 1 forces
    tokens on M, 2 weights on M.  ``split_k`` > 1 divides K among CTAs (weights on M with a
    residual only; the partial sums are added with atomics).  ``swiglu``: weight rows interleave
    gate and up in blocks of 8 and ``out`` is bfloat16 [M, N/2] = silu(gate) * up."""
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
         _ptr(out, "out"), _dtype_code(out.dtype), 2 if swiglu else (1 if residual is not None else 0), M, N, K, a.stride(0),
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


def describe_status(word: int) -> str:
    return "; ".join(text for bit, text in STATUS_BITS.items() if word & bit) or "ok"


__all__ = ["KernelError", "BuildError", "load_library", "library_file", "embed", "rmsnorm", "swiglu",
           "rope_append", "gemm_simple", "gemm_bf16", "attention_simple", "attention_decode", "attention_decode_fused", "attention_decode_resident", "decode_attention_plan", "decode_fusable", "attention_prefill",
           "paged_attention", "sample", "advance_decode", "feed_tokens", "describe_status"]
