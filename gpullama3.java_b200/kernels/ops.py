"""Python faces of the CUDA kernels: each function checks its tensors and calls one exported C
function on torch's current stream.  There is no other implementation behind these names: on a
machine without a GPU or without the compiled libraries they raise."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p

import torch

from .build import KernelBuildError, library

F32, BF16 = 0, 1
PAGE_TOKENS = 64  # must equal b200::kPageTokens
# what the plain kernels, which take every size the others refuse, are built for
HEAD_DIM_STEP, MAX_HEAD_DIM = 16, 512   # attention_generic.cu
MAX_ROTARY_DIM = 512                    # rope_cache.cu

_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    """A kernel refused its arguments or its launch failed."""


_ERRORS = {
    10001: "bad argument",
    10002: "unsupported size",
    10003: "scratch too small",
    10004: "the call needs more scratch than the built-in array of the no-allocation entry point holds",
}

_functions: dict[str, ctypes._CFuncPtr] = {}

# C signatures: library, then argument types (the trailing stream is added for all)
_SIGNATURES = {
    "b200_embed_gather": ("embedding", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float]),
    "b200_rmsnorm": ("norm", [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_float]),
    "b200_rope_cache_write": ("rope_cache", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                             c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int]),
    "b200_attention_paged": ("attention_generic", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                                   c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                                   c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int]),
    "b200_gemm_generic": ("gemm_generic", [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int,
                                           c_int, c_int, c_int, c_int, c_float, c_float]),
    "b200_gemm_generic_batched": ("gemm_generic", [c_void_p, c_int, c_int, ctypes.c_longlong, c_void_p, c_int, c_int,
                                                   ctypes.c_longlong, c_void_p, c_int, c_int, ctypes.c_longlong, c_int, c_int,
                                                   c_int, c_int]),
    "b200_gemm_decode": ("gemm_decode", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                         c_int, c_float, c_float]),
    "b200_gemm_decode_linked": ("gemm_decode", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                                c_int, c_int, c_void_p, c_int, c_float, c_int, c_void_p, c_int, c_void_p,
                                                c_int, c_void_p]),
    "b200_gemm_tcgen05": ("gemm_tcgen05", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                           c_int, c_int, c_int, c_int, c_float, c_float]),
    "b200_gemm_tcgen05_grouped": ("gemm_tcgen05", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                                   c_void_p, c_int, c_float, c_float]),
    "b200_gemm_tcgen05_qkv_rope": ("gemm_tcgen05", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p,
                                                    c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                                    c_int, c_int, c_int]),
    "b200_rope_angles": ("rope_cache", [c_void_p, c_void_p, c_void_p, c_int, c_int]),
    "b200_gemm_skinny": ("gemm_skinny_tcgen05", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                                 c_int, c_int, c_int]),
    "b200_attention_decode": ("attention_decode", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                                   c_void_p, c_void_p, ctypes.c_longlong, c_int, c_int, c_int, c_int,
                                                   c_int, c_int, c_int]),
    "b200_attention_decode_terms": ("attention_decode", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                                         c_void_p, c_void_p, ctypes.c_longlong, c_int, c_int, c_int, c_int,
                                                         c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int]),
    "b200_attention_prefill": ("attention_prefill", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                     c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                     c_void_p, c_void_p, c_void_p, c_int]),
    "b200_attention_decode_rope": ("attention_decode", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                                        c_void_p, c_void_p, ctypes.c_longlong, c_int, c_int, c_int,
                                                        c_int, c_int, c_int, c_void_p, c_int, c_int, c_int]),
    "b200_attention_prefill_tc": ("attention_prefill_tcgen05", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                                                c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                                                                c_int, c_int, c_int, c_int]),
    "b200_random_fill": ("random_init", [c_void_p, c_int, ctypes.c_longlong, ctypes.c_ulonglong, c_float, c_float]),
    "b200_streams_combine": ("streams", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int]),
    "b200_streams_read_norm": ("streams", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                                           c_float]),
    "b200_streams_step": ("streams", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                      c_int, c_int, c_float]),
    "b200_head_rows": ("head_rows", [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                     c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                     c_void_p, c_void_p]),
    "b200_softcap_rows": ("elementwise", [c_void_p, ctypes.c_longlong, c_float]),
    "b200_gated_rmsnorm": ("elementwise", [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                           c_float, c_int, c_int, c_int]),
    "b200_gate_rows": ("elementwise", [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int]),
    "b200_scale_rows": ("elementwise", [c_void_p, ctypes.c_longlong, c_float]),
    "b200_group_rmsnorm": ("sandwich", [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float]),
    "b200_sandwich_step": ("sandwich", [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                        c_int, c_int, c_float]),
    "b200_sandwich_step_conv": ("sandwich", [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                             c_int, c_int, c_float, c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_int,
                                             c_int]),
    "b200_add_row": ("sandwich", [c_void_p, c_void_p, c_int, c_int]),
    "b200_causal_conv": ("delta_rule", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, ctypes.c_longlong, c_void_p,
                                        c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                        c_int]),
    "b200_linear_scan": ("delta_rule", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                        c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                        c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_int, c_int]),
    "b200_moe_table_route": ("moe", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int]),
    "b200_layernorm": ("norm", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float]),
    "b200_causal_conv_silu": ("delta_rule", [c_void_p, c_int, c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_void_p,
                                             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int]),
    "b200_delta_rule_scan": ("delta_rule", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                            ctypes.c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                            c_int, c_int, c_int, c_int, c_float, c_float, c_int]),
    "b200_moe_route": ("moe", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                               c_int, c_int, c_float, c_void_p]),
    "b200_moe_rows": ("moe", [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                              c_int, c_int, c_int, c_float, c_float]),
    "b200_moe_group": ("moe", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "b200_moe_gather": ("moe", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int]),
    "b200_moe_combine": ("moe", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int]),
    "b200_differential_heads": ("elementwise", [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                                c_float, c_float]),
    "b200_gated_norm_step": ("gated_residual", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                                c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p, ctypes.c_longlong, c_int,
                                                c_void_p, c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_int, c_int, c_void_p]),
    "b200_depth_average": ("gated_residual", [c_void_p, ctypes.c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                              ctypes.c_longlong]),
    "b200_cast_rows": ("gated_residual", [c_void_p, c_void_p, c_int, ctypes.c_longlong]),
    "b200_bias_act_rows": ("gated_residual", [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int]),
    "b200_token_gate_rows": ("gated_residual", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int,
                                                c_int, c_int, c_int]),
    "b200_argmax_rows": ("sampling", [c_void_p, c_int, c_void_p, c_int, c_int]),
    "b200_sample_rows": ("sampling", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_void_p]),
}


def _fn(name: str):
    f = _functions.get(name)
    if f is None:
        lib_name, argtypes = _SIGNATURES[name]
        lib = library(lib_name)
        try:
            f = getattr(lib, name)
        except AttributeError as e:
            raise KernelBuildError(f"{name} is not exported by the {lib_name} kernel library") from e
        f.argtypes = list(argtypes) + [c_void_p]
        f.restype = c_int
        n_args = len(f.argtypes)

        def checked(*args, _f=f, _n=n_args, _name=name):
            if len(args) != _n:  # ctypes lets extra arguments through, which shifts the stream pointer
                raise TypeError(f"{_name} takes {_n} arguments, got {len(args)}")
            if _profile is None:
                return _f(*args)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            status = _f(*args)
            e1.record()
            _profile.append((_name, e0, e1))
            return status

        f = _functions[name] = checked
    return f


_profile: list | None = None   # (function, start event, end event) per launch while profiling is on


def profile_start() -> None:
    """From now on every launch issued through these functions is bracketed by CUDA events on its stream.  Launches
    replayed from a CUDA graph are not seen: profile with graphs off."""
    global _profile
    _profile = []


def profile_stop() -> dict[str, tuple[int, float]]:
    """Ends profiling; ``{function: (launches, total device ms)}``."""
    global _profile
    rows, _profile = _profile or [], None
    torch.cuda.synchronize()
    out: dict[str, tuple[int, float]] = {}
    for name, e0, e1 in rows:
        n, ms = out.get(name, (0, 0.0))
        out[name] = (n + 1, ms + e0.elapsed_time(e1))
    return out


_launches = 0
_launches_by_kernel: dict[str, int] = {}


def launch_count() -> int:
    """How many kernel launches this process has issued through these functions."""
    return _launches


def launches_by_kernel() -> dict[str, int]:
    """The same count per kernel function (a copy).  A launch recorded into a CUDA graph counts once, when it
    is recorded.  Decode attention that was told not to start early counts under ``<name>:late``."""
    return dict(_launches_by_kernel)


def _check(status: int, name: str) -> None:
    global _launches
    _launches += 1
    _launches_by_kernel[name] = _launches_by_kernel.get(name, 0) + 1
    if status != 0:
        what = _ERRORS.get(status)
        if what is None:
            what = f"CUDA error {status}"
        raise KernelError(f"{name}: {what}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_current_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """The current CUDA stream's handle.  Asked for at every launch (a graph capture changes it), so through the
    two plain C calls where this torch has them: building a ``torch.cuda.Stream`` object costs several microseconds,
    which a pass of a hundred short kernels feels."""
    if _raw_stream is not None and _current_device is not None:
        return _raw_stream(_current_device())
    return torch.cuda.current_stream().cuda_stream


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"kernels store float32 or bfloat16, not {dtype}") from None


def _dev(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels take CUDA tensors only; there is no CPU path")


# --------------------------------------------------------------------------- embedding, norm
def embed_gather(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t] = scale * table[tokens[t]] into the float32 residual stream.  tokens int32 [T]."""
    _dev(table, tokens, out)
    assert out.dtype == torch.float32 and tokens.dtype == torch.int32
    assert table.is_contiguous() and out.is_contiguous()
    n, dim = out.shape
    _check(_fn("b200_embed_gather")(table.data_ptr(), dtype_code(table.dtype), tokens.data_ptr(), out.data_ptr(),
                                    n, dim, table.shape[0], float(scale), _stream()), "embed_gather")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float, rows: torch.Tensor | None = None) -> None:
    """out[r] = weight * x[rows[r]] / sqrt(mean(x^2) + eps).  x float32 [T, dim]."""
    _dev(x, weight, out, rows)
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and weight.is_contiguous()
    n_rows, dim = out.shape
    assert x.shape[1] == dim and weight.numel() == dim
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.numel() == n_rows
    _check(_fn("b200_rmsnorm")(x.data_ptr(), weight.data_ptr(), dtype_code(weight.dtype), out.data_ptr(),
                               dtype_code(out.dtype), rows.data_ptr() if rows is not None else None, n_rows, dim,
                               float(eps), _stream()), "rmsnorm")


def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, out: torch.Tensor, eps: float,
              rows: torch.Tensor | None = None) -> None:
    """out[r] = (x[rows[r]] - mean) / sqrt(mean((x - mean)^2) + eps) * weight + bias.  x, weight, bias float32."""
    _dev(x, weight, bias, out, rows)
    assert x.dtype == weight.dtype == bias.dtype == torch.float32
    assert x.is_contiguous() and out.is_contiguous() and weight.is_contiguous() and bias.is_contiguous()
    n_rows, dim = out.shape
    assert x.shape[1] == dim and weight.numel() == dim and bias.numel() == dim
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.numel() == n_rows
    _check(_fn("b200_layernorm")(x.data_ptr(), weight.data_ptr(), bias.data_ptr(), out.data_ptr(), dtype_code(out.dtype),
                                 rows.data_ptr() if rows is not None else None, n_rows, dim, float(eps), _stream()),
           "layernorm")


# --------------------------------------------------------------------------- position encoding + cache write
def rope_cache_write(qkv: torch.Tensor, positions: torch.Tensor, seq_ids: torch.Tensor, page_table: torch.Tensor,
                     inv_freq: torch.Tensor, k_pool: torch.Tensor | None, v_pool: torch.Tensor | None, n_heads: int,
                     n_kv_heads: int, head_dim: int, rotary_dim: int, pairing: int, write_cache: bool = True) -> None:
    """Rotate the queries of ``qkv`` [T, (H + 2 KVH) D] in place; write rotated keys and the values
    into the cache pages of their positions."""
    _dev(qkv, positions, seq_ids, page_table, inv_freq, k_pool, v_pool)
    assert qkv.is_contiguous() and qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() >= max(rotary_dim // 2, 0)
    assert page_table.dtype == torch.int32 and page_table.dim() == 2 and page_table.is_contiguous()
    if write_cache:
        assert k_pool.dtype == qkv.dtype and v_pool.dtype == qkv.dtype
        assert k_pool.is_contiguous() and v_pool.is_contiguous()
        assert tuple(k_pool.shape[1:]) == (n_kv_heads, PAGE_TOKENS, head_dim)
        assert tuple(v_pool.shape[1:]) == (n_kv_heads, head_dim, PAGE_TOKENS)
    _check(_fn("b200_rope_cache_write")(
        qkv.data_ptr(), dtype_code(qkv.dtype), positions.data_ptr(), seq_ids.data_ptr(), page_table.data_ptr(),
        page_table.shape[1], inv_freq.data_ptr(), k_pool.data_ptr() if write_cache else None,
        v_pool.data_ptr() if write_cache else None, qkv.shape[0], n_heads, n_kv_heads, head_dim, rotary_dim, pairing,
        1 if write_cache else 0, _stream()), "rope_cache_write")


# --------------------------------------------------------------------------- attention
def attention_paged(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, positions: torch.Tensor,
                    seq_ids: torch.Tensor, page_table: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                    n_heads: int, n_kv_heads: int, head_dim: int, window: int = 0, n_splits: int = 1, *,
                    keep_first: int = 0, slopes: torch.Tensor | None = None, sinks: torch.Tensor | None = None,
                    gate: torch.Tensor | None = None) -> None:
    """Causal grouped-query attention of every token of ``q`` over the cached keys 0..position of
    its sequence.  q: rows of ``q_row_stride`` elements whose first H*D are the rotated queries.
    ``n_splits`` > 1 cuts every token's keys into that many spans, one CTA each, merged by a second kernel (a decode
    step: few tokens, long rows of keys).  ``keep_first``: positions below it stay visible behind the window;
    ``slopes`` float32 [H]: score -= slopes[h] * distance; ``sinks`` float32 [H]: exp(sinks[h]) joins the softmax's
    denominator; ``gate`` [T, >= H] of q's dtype: head outputs are multiplied by sigmoid(gate[t, h])."""
    _dev(q, out, positions, seq_ids, page_table, k_pool, v_pool)
    assert out.is_contiguous() and out.shape[1] == n_heads * head_dim and out.dtype == q.dtype == k_pool.dtype
    assert tuple(k_pool.shape[1:]) == (n_kv_heads, PAGE_TOKENS, head_dim)
    assert tuple(v_pool.shape[1:]) == (n_kv_heads, head_dim, PAGE_TOKENS)
    scratch = None
    if n_splits > 1:
        scratch = torch.empty(out.shape[0] * n_heads * n_splits * (head_dim + 2), dtype=torch.float32, device=q.device)
    _dev(slopes, sinks, gate)
    for t in (slopes, sinks):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == n_heads)
    assert gate is None or (gate.dtype == q.dtype and gate.stride(1) == 1 and gate.shape[1] >= n_heads)
    ptr = lambda t: t.data_ptr() if t is not None else None
    _check(_fn("b200_attention_paged")(
        q.data_ptr(), q_row_stride, out.data_ptr(), dtype_code(q.dtype), positions.data_ptr(), seq_ids.data_ptr(),
        page_table.data_ptr(), page_table.shape[1], k_pool.data_ptr(), v_pool.data_ptr(), out.shape[0], n_heads,
        n_kv_heads, head_dim, int(window), int(n_splits), scratch.data_ptr() if scratch is not None else None,
        int(keep_first), ptr(slopes), ptr(sinks), ptr(gate), gate.stride(0) if gate is not None else 0, _stream()),
        "attention_paged")


# --------------------------------------------------------------------------- matrix products
EPILOGUE_STORE, EPILOGUE_RESIDUAL_ADD, EPILOGUE_GATED_SILU, EPILOGUE_GATED_GELU_TANH, EPILOGUE_GATED_CLAMPED = 0, 1, 2, 3, 4
GATED_EPILOGUES = (EPILOGUE_GATED_SILU, EPILOGUE_GATED_GELU_TANH, EPILOGUE_GATED_CLAMPED)
# the gated epilogues' activations: silu(g) u, gelu_tanh(g) u, and the clamped form g' sigmoid(slope g') (u' + 1) with
# g' = min(g, limit), u' = clamp(u, -limit, limit), whose two numbers travel with the call (``gate_args``)
ACTIVATION_CODES = {"silu": 0, "gelu_tanh": 1, "clamped_sigmoid": 2}
GATED_EPILOGUE_OF = {"silu": EPILOGUE_GATED_SILU, "gelu_tanh": EPILOGUE_GATED_GELU_TANH, "clamped_sigmoid": EPILOGUE_GATED_CLAMPED}


def gemm_generic(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, epilogue: int = EPILOGUE_STORE,
                 gate_args: tuple[float, float] = (0.0, 0.0)) -> None:
    """c = a @ w.T (store), c += a @ w.T (residual add, c float32) or c = act(gate) * up with
    gate/up rows interleaved in w (act: SiLU, or GELU in its tanh form).  32-bit FMA accumulation, no tensor cores."""
    _dev(a, w, c)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    assert c.shape[0] == M and c.shape[1] == (N // 2 if epilogue in GATED_EPILOGUES else N)
    _check(_fn("b200_gemm_generic")(
        a.data_ptr(), dtype_code(a.dtype), a.stride(0), w.data_ptr(), dtype_code(w.dtype), w.stride(0), c.data_ptr(),
        dtype_code(c.dtype), c.stride(0), M, N, K, epilogue, float(gate_args[0]), float(gate_args[1]), _stream()),
        "gemm_generic")


def gemm_per_head(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor) -> None:
    """c[:, h n : (h + 1) n] = a[:, h k : (h + 1) k] @ w[h].T for every head h: a [T, H k], w [H, n, k], c [T, H n].
    One launch of the plain kernel (32-bit FMA accumulation) for all heads."""
    _dev(a, w, c)
    H, n, k = w.shape
    T = a.shape[0]
    assert w.is_contiguous() and a.stride(1) == 1 and c.stride(1) == 1
    assert tuple(a.shape) == (T, H * k) and tuple(c.shape) == (T, H * n)
    _check(_fn("b200_gemm_generic_batched")(a.data_ptr(), dtype_code(a.dtype), a.stride(0), k, w.data_ptr(),
                                            dtype_code(w.dtype), k, n * k, c.data_ptr(), dtype_code(c.dtype), c.stride(0), n,
                                            T, n, k, H, _stream()), "gemm_per_head")


def gemm_decode(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, epilogue: int = EPILOGUE_STORE,
                gate_args: tuple[float, float] = (0.0, 0.0)) -> bool:
    """The decode-step matrix product (bfloat16 operands, at most 64 tokens, K a multiple of 32).
    Returns False, having done nothing, for operands it does not take."""
    M, K = a.shape
    if (a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or M > 64 or K % 32 or a.stride(1) != 1
            or w.stride(1) != 1 or a.stride(0) % 8 or w.stride(0) % 8 or (a.data_ptr() | w.data_ptr()) & 15):
        return False
    _dev(a, w, c)
    N = w.shape[0]
    assert w.shape[1] == K and c.stride(1) == 1 and c.shape[0] == M
    assert c.shape[1] == (N // 2 if epilogue in GATED_EPILOGUES else N)
    _check(_fn("b200_gemm_decode")(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), c.data_ptr(),
                                   dtype_code(c.dtype), c.stride(0), M, N, K, epilogue, float(gate_args[0]),
                                   float(gate_args[1]), _stream()), "gemm_decode")
    return True


def gemm_decode_links(n_rows: int, w: torch.Tensor) -> bool:
    """Whether ``gemm_decode_linked`` takes a product of ``n_rows`` bfloat16 rows with ``w``."""
    return (w.dtype == torch.bfloat16 and n_rows <= 16 and w.shape[1] % 32 == 0 and w.stride(1) == 1
            and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0)


def gemm_decode_partials(n_rows: int, n_out: int) -> int:
    """How many partial sums of squares per row the residual product [n_rows, n_out] leaves."""
    lib = library("gemm_decode")
    return int(lib.b200_gemm_decode_ctas(n_rows, n_out))


def gemm_decode_linked(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, epilogue: int, *, row_factors=None,
                       emit=None) -> None:
    """``gemm_decode`` as one half, or both, of an RMSNorm split between two products (at most 16 rows).

    ``row_factors = (partials [M, P] float32, eps, dim)``: the rows of ``a`` are x * w of a norm; every
    sum of row t is multiplied by rsqrt(sum(partials[t]) / dim + eps) before the epilogue.
    ``emit = (norm_weight [N], act [M, N] bfloat16, partials [M, gemm_decode_partials(M, N)] float32)``
    (residual epilogue only): after c += a w^T, act = bfloat16(c * norm_weight) and partials hold each
    CTA's sum of c^2 per row."""
    M, K = a.shape
    N = w.shape[0]
    _dev(a, w, c)
    assert a.dtype == torch.bfloat16 and gemm_decode_links(M, w) and a.stride(1) == 1 and a.stride(0) % 8 == 0
    assert w.shape[1] == K and c.stride(1) == 1 and c.shape[0] == M and a.data_ptr() % 16 == 0
    assert c.shape[1] == (N // 2 if epilogue in GATED_EPILOGUES else N)
    in_p, n_in, eps, dim = None, 0, 0.0, 0
    if row_factors is not None:
        part, eps, dim = row_factors
        assert part.dtype == torch.float32 and part.is_contiguous() and part.shape[0] == M
        in_p, n_in = part.data_ptr(), part.shape[1]
    out_w, out_w_dtype, out_act, ld_act, out_p = None, 0, None, 0, None
    if emit is not None:
        nw, act, part_out = emit
        assert epilogue == EPILOGUE_RESIDUAL_ADD and nw.numel() == N and nw.is_contiguous()
        assert act.dtype == torch.bfloat16 and act.shape == (M, N) and act.stride(1) == 1
        assert part_out.dtype == torch.float32 and part_out.is_contiguous()
        assert tuple(part_out.shape) == (M, gemm_decode_partials(M, N))
        out_w, out_w_dtype, out_act, ld_act, out_p = nw.data_ptr(), dtype_code(nw.dtype), act.data_ptr(), act.stride(0), part_out.data_ptr()
    _check(_fn("b200_gemm_decode_linked")(
        a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), c.data_ptr(), dtype_code(c.dtype), c.stride(0), M, N, K,
        epilogue, in_p, n_in, float(eps), int(dim), out_w, out_w_dtype, out_act, ld_act, out_p, _stream()),
        "gemm_decode_linked")


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, epilogue: int = EPILOGUE_STORE,
                 tile_width: int = 0, k_spans: int = 0, cta_pair: int = 0,
                 gate_args: tuple[float, float] = (0.0, 0.0)) -> bool:
    """The prefill matrix product on tcgen05 tensor cores (bfloat16 operands, rows 16-byte aligned).
    ``tile_width``: 256, 128 or 64 output columns per tile; 0 lets the shape decide (narrower tiles when the
    widest would leave SMs without one).  ``k_spans``: 2 or 4 cuts K among the CTAs of a cluster, which add their
    partial tiles in a fixed order (few tiles, long K); 1 never; 0 lets the shape decide.  ``cta_pair``: 1 computes
    tiles of 256 rows by pairs of CTAs that each load half of the weight stage (tile_width 256 or 128); -1 never;
    0 lets the shape decide.
    Returns False, having done nothing, for operands it does not take."""
    M, K = a.shape
    lda, a_inner = a.stride()
    ldw, w_inner = w.stride()
    pa, pw = a.data_ptr(), w.data_ptr()
    if (a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or K % 8 or K < 8 or a_inner != 1 or w_inner != 1
            or lda % 8 or ldw % 8 or (pa | pw) & 15):
        return False
    if epilogue in GATED_EPILOGUES and c.dtype != torch.bfloat16:
        return False
    _dev(a, w, c)
    N, Kw = w.shape
    ldc, c_inner = c.stride()
    assert Kw == K and c_inner == 1 and c.shape == (M, N // 2 if epilogue in GATED_EPILOGUES else N)
    _check(_fn("b200_gemm_tcgen05")(pa, lda, pw, ldw, c.data_ptr(), dtype_code(c.dtype), ldc, M, N, K, epilogue,
                                    tile_width, k_spans, cta_pair, float(gate_args[0]), float(gate_args[1]), _stream()),
           "gemm_tcgen05")
    return True


MAX_GEMM_GROUPS = 256   # gemm_tcgen05.cu


def gemm_tcgen05_grouped(a: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor, c: torch.Tensor,
                         epilogue: int = EPILOGUE_STORE, gate_args: tuple[float, float] = (0.0, 0.0)) -> bool:
    """One product per group in one launch on tcgen05 tensor cores: c[p] = a[p] @ w[g].T for the rows p = offsets[g] ..
    offsets[g + 1] - 1 (offsets int32 [G + 1] on the device, read there).  a [P, K] and w [G, N, K] bfloat16; c [P, N]
    float32 (store) or [P, N / 2] bfloat16 (gated epilogues).  Returns False, having done nothing, for operands it
    does not take."""
    P, K = a.shape
    G, N, Kw = w.shape
    if (a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or G > MAX_GEMM_GROUPS or K % 8 or K < 8 or a.stride(1) != 1
            or a.stride(0) % 8 or not w.is_contiguous() or (a.data_ptr() | w.data_ptr()) & 15):
        return False
    gated = epilogue in GATED_EPILOGUES
    if (gated and (c.dtype != torch.bfloat16 or N % 2)) or (not gated and (epilogue != EPILOGUE_STORE or c.dtype != torch.float32)):
        return False
    _dev(a, w, offsets, c)
    assert Kw == K and offsets.dtype == torch.int32 and offsets.numel() == G + 1 and c.stride(1) == 1
    assert tuple(c.shape) == (P, N // 2 if gated else N)
    status = _fn("b200_gemm_tcgen05_grouped")(a.data_ptr(), a.stride(0), w.data_ptr(), c.data_ptr(), dtype_code(c.dtype),
                                              c.stride(0), P, N, K, G, offsets.data_ptr(), epilogue, float(gate_args[0]),
                                              float(gate_args[1]), _stream())
    if status == _UNSUPPORTED:
        return False
    _check(status, "gemm_tcgen05_grouped")
    return True


def rope_angles(positions: torch.Tensor, inv_freq: torch.Tensor, half: int) -> torch.Tensor:
    """float32 [half, T, 2]: cosine and sine of position * frequency for every pair of a head and every token of a
    pass, evaluated as the rotation kernels evaluate them (pair-major: the tokens of a warp read neighbours)."""
    _dev(positions, inv_freq)
    assert positions.dtype == torch.int32 and inv_freq.dtype == torch.float32 and inv_freq.numel() >= half > 0
    out = torch.empty((half, positions.numel(), 2), dtype=torch.float32, device=positions.device)
    _check(_fn("b200_rope_angles")(positions.data_ptr(), inv_freq.data_ptr(), out.data_ptr(), positions.numel(), half, _stream()),
           "rope_angles")
    return out


_UNSUPPORTED = 10002   # kErrUnsupportedSize: the kernel leaves these operands to another one


def gemm_tcgen05_qkv_rope(a: torch.Tensor, w: torch.Tensor, qkv: torch.Tensor, positions: torch.Tensor,
                          seq_ids: torch.Tensor, page_table: torch.Tensor, angles: torch.Tensor,
                          k_pool: torch.Tensor | None, v_pool: torch.Tensor | None, n_heads: int, n_kv_heads: int,
                          head_dim: int, pairing: int, write_cache: bool = True) -> bool:
    """The query/key/value projection of a prompt pass on tcgen05 tensor cores with the rotation and the cache
    write in its epilogue: ``qkv`` [T, (H + 2 KVH) D] receives the rotated queries (its key and value columns stay
    unwritten), rotated keys and the values go to the cache pages of their positions.  ``angles``: ``rope_angles`` of
    the pass.  Returns False, having done nothing, for shapes it does not take (head sizes other than 64 and 128, a
    product of few tiles): the caller then runs the product and ``rope_cache_write``."""
    M, K = a.shape
    N = (n_heads + 2 * n_kv_heads) * head_dim
    if (a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or qkv.dtype != torch.bfloat16 or head_dim not in (64, 128)
            or K % 8 or K < 8 or a.stride(1) != 1 or w.stride(1) != 1 or a.stride(0) % 8 or w.stride(0) % 8
            or qkv.stride(0) % 8 or (a.data_ptr() | w.data_ptr() | qkv.data_ptr()) & 15):
        return False
    _dev(a, w, qkv, positions, seq_ids, page_table, angles, k_pool, v_pool)
    assert tuple(w.shape) == (N, K) and tuple(qkv.shape) == (M, N) and qkv.stride(1) == 1
    assert positions.dtype == seq_ids.dtype == page_table.dtype == torch.int32 and page_table.dim() == 2 and page_table.is_contiguous()
    assert positions.numel() == M and seq_ids.numel() == M
    assert angles.dtype == torch.float32 and angles.is_contiguous() and tuple(angles.shape) == (head_dim // 2, M, 2)
    if write_cache:
        assert k_pool.dtype == v_pool.dtype == torch.bfloat16 and k_pool.is_contiguous() and v_pool.is_contiguous()
        assert tuple(k_pool.shape[1:]) == (n_kv_heads, PAGE_TOKENS, head_dim)
        assert tuple(v_pool.shape[1:]) == (n_kv_heads, head_dim, PAGE_TOKENS)
    status = _fn("b200_gemm_tcgen05_qkv_rope")(
        a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), qkv.data_ptr(), qkv.stride(0), M, K, positions.data_ptr(),
        seq_ids.data_ptr(), page_table.data_ptr(), page_table.shape[1], angles.data_ptr(),
        k_pool.data_ptr() if write_cache else None, v_pool.data_ptr() if write_cache else None, n_heads, n_kv_heads,
        head_dim, pairing, 1 if write_cache else 0, _stream())
    if status == _UNSUPPORTED:
        return False
    _check(status, "gemm_tcgen05_qkv_rope")
    return True


def gemm_tcgen05_k_spans(M: int, N: int, K: int) -> int:
    """Into how many spans ``gemm_tcgen05`` cuts K for this shape when it is left the choice (1: it does not)."""
    return int(library("gemm_tcgen05").b200_gemm_tcgen05_k_spans(M, N, K))


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, epilogue: int = EPILOGUE_STORE,
                k_splits: int | None = None) -> bool:
    """The few-token matrix product on tcgen05 tensor cores (bfloat16 operands, at most 128 tokens,
    rows 16-byte aligned).  Returns False, having done nothing, for operands it does not take."""
    M, K = a.shape
    if (a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or M > 128 or K % 8 or K < 8 or a.stride(1) != 1
            or w.stride(1) != 1 or a.stride(0) % 8 or w.stride(0) % 8 or (a.data_ptr() | w.data_ptr()) & 15):
        return False
    if epilogue in (EPILOGUE_GATED_GELU_TANH, EPILOGUE_GATED_CLAMPED) or (epilogue == EPILOGUE_GATED_SILU and c.dtype != torch.bfloat16):
        return False
    _dev(a, w, c)
    N = w.shape[0]
    assert w.shape[1] == K and c.stride(1) == 1 and c.shape[0] == M
    assert c.shape[1] == (N // 2 if epilogue in GATED_EPILOGUES else N)
    fn = _fn("b200_gemm_skinny")
    if k_splits is None:
        k_splits = library("gemm_skinny_tcgen05").b200_gemm_skinny_splits(M, N, K, _sm_count(a.device))
    _check(fn(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), c.data_ptr(), dtype_code(c.dtype), c.stride(0), M, N,
              K, epilogue, k_splits, _stream()), "gemm_skinny")
    return True


_sm_counts: dict = {}


def _sm_count(device) -> int:
    n = _sm_counts.get(device)
    if n is None:
        n = _sm_counts[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return n


def gemm_skinny_status() -> int:
    lib = library("gemm_skinny_tcgen05")
    lib.b200_gemm_skinny_status.restype = c_int
    return int(lib.b200_gemm_skinny_status())


def gemm_tcgen05_status() -> int:
    """0 when every wait inside the tensor-core GEMM completed since the last call; synchronises."""
    lib = library("gemm_tcgen05")
    lib.b200_gemm_tcgen05_status.restype = c_int
    return int(lib.b200_gemm_tcgen05_status())


def attention_decode_supported(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int) -> bool:
    return dtype == torch.bfloat16 and head_dim in (32, 64, 96, 128) and n_heads // n_kv_heads <= 16


_ctas_per_sm: dict = {}


def resident_ctas(device, head_dim: int = 64, group: int = 4, fused: bool = True) -> int:
    """The number of CTAs of decode attention the GPU holds at once, which is what the spans are planned for: the
    occupancy the driver reports for the kernel of these sizes (heads of 64 hold four per SM, heads of 128 two)
    times the SMs.  Four per SM for sizes that kernel does not take."""
    key = (head_dim, group > 8, fused)
    per_sm = _ctas_per_sm.get(key)
    if per_sm is None:
        query = library("attention_decode").b200_attention_decode_ctas_per_sm
        query.argtypes, query.restype = [c_int, c_int, c_int], c_int
        per_sm = _ctas_per_sm[key] = query(head_dim, group, 1 if fused else 0) or 4
    return per_sm * _sm_count(torch.device(device))


def attention_decode_splits(n_seqs: int, n_kv_heads: int, max_kv_len: int, resident_ctas: int) -> int:
    """How many spans each sequence's keys are cut into.  The grid (spans x kv heads x sequences)
    should fill the GPU in one wave (``resident_ctas``) without spilling into a second one.  Up to 16 spans a
    span may be as short as two blocks of 32 keys (a short context at a small batch is otherwise a handful of CTAs
    walking their keys one block after the other: batch 1 at 1,024 keys 0.705 -> 0.677 ms per step with 8 spans
    instead of 4); beyond 16 a span keeps at least 8 blocks so that its start-up and the merge pay (batch 1 at
    4,096 keys: 16 spans 0.713 ms, 32 spans 0.717, 64 spans 0.771)."""
    blocks = max(1, (max_kv_len + 31) // 32)
    cap = max(1, resident_ctas // max(1, n_seqs * n_kv_heads))
    want = max(1, min(cap, 64, max(blocks // 8, min(16, blocks // 2))))
    p = 1
    while p * 2 <= want:
        p *= 2
    return p


def attention_decode_early_start(n_seqs: int, n_kv_heads: int, max_kv_len: int, n_splits: int) -> bool:
    """Whether the decode attention may be scheduled while the kernel before it still runs.  A grid
    that fills the GPU with long spans (48 blocks of 32 keys or more) should find it empty instead:
    started early, its CTAs settle unevenly among the predecessor's and the fullest SMs finish late
    (batch 64 at 4,096 keys: 203 against 142 us per layer)."""
    blocks_per_span = (max_kv_len + 31) // 32 // max(1, n_splits)
    return not (n_seqs * n_kv_heads * n_splits >= 256 and blocks_per_span >= 48)


def attention_decode_rope_supported(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int,
                                    pairing: int) -> bool:
    """Whether the decode kernel can also do the step's rotation and cache write."""
    return (attention_decode_supported(dtype, n_heads, n_kv_heads, head_dim) and rotary_dim == head_dim
            and (pairing == 0 or head_dim in (64, 128)))


def attention_decode_rope(qkv: torch.Tensor, out: torch.Tensor, kv_lens: torch.Tensor, page_table: torch.Tensor,
                          k_pool: torch.Tensor, v_pool: torch.Tensor, inv_freq: torch.Tensor, n_heads: int,
                          n_kv_heads: int, head_dim: int, pairing: int, window: int, n_splits: int,
                          write_cache: bool = True, scratch: torch.Tensor | None = None,
                          early_start: bool = True) -> None:
    """Decode attention that rotates the step's queries itself and, with ``write_cache``, stores the
    step's rotated key and its value at position kv_lens[i] - 1 of sequence i.  ``qkv``: the raw
    projections [n_seqs, (n_heads + 2 n_kv_heads) head_dim] (left untouched)."""
    _dev(qkv, out, kv_lens, page_table, k_pool, v_pool, inv_freq)
    n_seqs = out.shape[0]
    assert qkv.dtype == out.dtype == k_pool.dtype == torch.bfloat16 and out.is_contiguous() and qkv.is_contiguous()
    assert qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim and inv_freq.dtype == torch.float32
    assert tuple(k_pool.shape[1:]) == (n_kv_heads, PAGE_TOKENS, head_dim)
    assert tuple(v_pool.shape[1:]) == (n_kv_heads, head_dim, PAGE_TOKENS)
    need = n_seqs * n_heads * n_splits * (head_dim + 2) if n_splits > 1 else 0
    if need and (scratch is None or scratch.numel() < need):
        scratch = torch.empty(need, dtype=torch.float32, device=qkv.device)
    _check(_fn("b200_attention_decode_rope")(
        qkv.data_ptr(), qkv.shape[1], out.data_ptr(), kv_lens.data_ptr(), page_table.data_ptr(), page_table.shape[1],
        k_pool.data_ptr(), v_pool.data_ptr(), scratch.data_ptr() if need else None, scratch.numel() if need else 0,
        n_seqs, n_heads, n_kv_heads, head_dim, int(window), n_splits, inv_freq.data_ptr(), pairing,
        1 if write_cache else 0, 1 if early_start else 0, _stream()),
        "attention_decode_rope" if early_start else "attention_decode_rope:late")


def attention_decode(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, kv_lens: torch.Tensor,
                     page_table: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, n_heads: int,
                     n_kv_heads: int, head_dim: int, window: int, n_splits: int,
                     scratch: torch.Tensor | None = None, early_start: bool = True, *, keep_first: int = 0,
                     slopes: torch.Tensor | None = None, sinks: torch.Tensor | None = None,
                     gate: torch.Tensor | None = None) -> None:
    """One query token per sequence (row i of q belongs to sequence i) over kv_lens[i] cached keys.
    ``scratch``: float32 workspace for the spans' partial results (allocated here when absent).
    ``early_start``: see ``attention_decode_early_start``.  ``keep_first``, ``slopes``, ``sinks``, ``gate``: as for
    ``attention_paged``."""
    _dev(q, out, kv_lens, page_table, k_pool, v_pool)
    n_seqs = out.shape[0]
    assert q.dtype == out.dtype == k_pool.dtype == torch.bfloat16 and out.is_contiguous()
    assert tuple(k_pool.shape[1:]) == (n_kv_heads, PAGE_TOKENS, head_dim)
    assert tuple(v_pool.shape[1:]) == (n_kv_heads, head_dim, PAGE_TOKENS)
    need = n_seqs * n_heads * n_splits * (head_dim + 2) if n_splits > 1 else 0
    if need and (scratch is None or scratch.numel() < need):
        scratch = torch.empty(need, dtype=torch.float32, device=q.device)
    if keep_first or slopes is not None or sinks is not None or gate is not None:
        _dev(slopes, sinks, gate)
        for t in (slopes, sinks):
            assert t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == n_heads)
        assert gate is None or (gate.dtype == torch.bfloat16 and gate.stride(1) == 1 and gate.shape[1] >= n_heads)
        ptr = lambda t: t.data_ptr() if t is not None else None
        _check(_fn("b200_attention_decode_terms")(
            q.data_ptr(), q_row_stride, out.data_ptr(), kv_lens.data_ptr(), page_table.data_ptr(), page_table.shape[1],
            k_pool.data_ptr(), v_pool.data_ptr(), scratch.data_ptr() if need else None, scratch.numel() if need else 0,
            n_seqs, n_heads, n_kv_heads, head_dim, int(window), n_splits, 1 if early_start else 0, int(keep_first),
            ptr(slopes), ptr(sinks), ptr(gate), gate.stride(0) if gate is not None else 0, _stream()),
            "attention_decode_terms" if early_start else "attention_decode_terms:late")
        return
    _check(_fn("b200_attention_decode")(
        q.data_ptr(), q_row_stride, out.data_ptr(), kv_lens.data_ptr(), page_table.data_ptr(), page_table.shape[1],
        k_pool.data_ptr(), v_pool.data_ptr(), scratch.data_ptr() if need else None, scratch.numel() if need else 0,
        n_seqs, n_heads, n_kv_heads, head_dim, int(window), n_splits, 1 if early_start else 0, _stream()),
        "attention_decode" if early_start else "attention_decode:late")


def attention_prefill(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, cu_seqlens: torch.Tensor,
                      kv_lens: torch.Tensor, page_table: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                      n_seqs: int, max_q_len: int, n_heads: int, n_kv_heads: int, head_dim: int, window: int, *,
                      keep_first: int = 0, slopes: torch.Tensor | None = None, sinks: torch.Tensor | None = None,
                      gate: torch.Tensor | None = None) -> None:
    """Causal attention of packed query tokens: sequence i owns rows cu_seqlens[i]..cu_seqlens[i+1],
    which are its last positions (kv_lens[i] - q_len .. kv_lens[i] - 1); keys come from the cache.
    ``keep_first``, ``slopes``, ``sinks``, ``gate``: as for ``attention_paged``."""
    _dev(q, out, cu_seqlens, kv_lens, page_table, k_pool, v_pool, slopes, sinks, gate)
    for t in (slopes, sinks):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == n_heads)
    assert gate is None or (gate.dtype == torch.bfloat16 and gate.stride(1) == 1 and gate.shape[1] >= n_heads)
    ptr = lambda t: t.data_ptr() if t is not None else None
    assert q.dtype == out.dtype == k_pool.dtype == torch.bfloat16 and out.is_contiguous()
    assert tuple(k_pool.shape[1:]) == (n_kv_heads, PAGE_TOKENS, head_dim)
    assert tuple(v_pool.shape[1:]) == (n_kv_heads, head_dim, PAGE_TOKENS)
    _check(_fn("b200_attention_prefill")(
        q.data_ptr(), q_row_stride, out.data_ptr(), cu_seqlens.data_ptr(), kv_lens.data_ptr(), page_table.data_ptr(),
        page_table.shape[1], k_pool.data_ptr(), v_pool.data_ptr(), n_seqs, max_q_len, n_heads, n_kv_heads, head_dim,
        int(window), int(keep_first), ptr(slopes), ptr(sinks), ptr(gate), gate.stride(0) if gate is not None else 0,
        _stream()), "attention_prefill")


def attention_prefill_tc(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, cu_seqlens: torch.Tensor,
                         kv_lens: torch.Tensor, page_table: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                         n_seqs: int, max_q_len: int, n_heads: int, n_kv_heads: int, head_dim: int, window: int) -> bool:
    """``attention_prefill`` on tcgen05 tensor cores (head_dim 64 or 128).  Returns False, having done
    nothing, for sizes it does not take."""
    if head_dim not in (64, 128) or q.dtype != torch.bfloat16 or q_row_stride % 8 or (q.data_ptr() | out.data_ptr()) & 15:
        return False
    _dev(q, out, cu_seqlens, kv_lens, page_table, k_pool, v_pool)
    assert out.dtype == k_pool.dtype == torch.bfloat16 and out.is_contiguous() and k_pool.is_contiguous()
    assert tuple(k_pool.shape[1:]) == (n_kv_heads, PAGE_TOKENS, head_dim)
    assert tuple(v_pool.shape[1:]) == (n_kv_heads, head_dim, PAGE_TOKENS)
    _check(_fn("b200_attention_prefill_tc")(
        q.data_ptr(), q_row_stride, out.shape[0], out.data_ptr(), cu_seqlens.data_ptr(), kv_lens.data_ptr(),
        page_table.data_ptr(), page_table.shape[1], k_pool.data_ptr(), v_pool.data_ptr(), k_pool.shape[0], n_seqs,
        max_q_len, n_heads, n_kv_heads, head_dim, int(window), _stream()), "attention_prefill_tc")
    return True


def attention_prefill_tc_status() -> int:
    lib = library("attention_prefill_tcgen05")
    lib.b200_attention_prefill_tc_status.restype = c_int
    return int(lib.b200_attention_prefill_tc_status())


# --------------------------------------------------------------------------- random weights
def random_fill(out: torch.Tensor, key: int, scale: float, offset: float) -> None:
    """out.flat[i] = offset + scale * (sum of sixteen 16-bit fields of the splitmix64 sequence of ``key`` at 4i..4i+3,
    centred): the numbers ``weights.random_init.random_values`` makes on the CPU, bit for bit."""
    _dev(out)
    assert out.is_contiguous()
    _check(_fn("b200_random_fill")(out.data_ptr(), dtype_code(out.dtype), out.numel(), key & ((1 << 64) - 1),
                                   float(scale), float(offset), _stream()), "random_fill")


# --------------------------------------------------------------------------- sampling
def argmax_rows(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = index of the first maximum of logits[r] (float32 [R, V]); out int32 [R]."""
    _dev(logits, out)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    _check(_fn("b200_argmax_rows")(logits.data_ptr(), logits.stride(0), out.data_ptr(), logits.shape[0],
                                   logits.shape[1], _stream()), "argmax_rows")


def sample_rows(logits: torch.Tensor, uniforms: torch.Tensor, out: torch.Tensor, temperature: float,
                top_p: float) -> None:
    """Temperature softmax and inverse-CDF draw (nucleus when 0 < top_p < 1) per row."""
    _dev(logits, uniforms, out)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    assert uniforms.dtype == torch.float32 and uniforms.numel() == logits.shape[0]
    scratch = None
    if 0.0 < top_p < 1.0:  # nucleus: the row's probabilities are kept in workspace between the passes
        scratch = torch.empty(logits.shape[0] * logits.shape[1], dtype=torch.float32, device=logits.device)
    _check(_fn("b200_sample_rows")(logits.data_ptr(), logits.stride(0), uniforms.data_ptr(), out.data_ptr(),
                                   logits.shape[0], logits.shape[1], float(temperature), float(top_p),
                                   scratch.data_ptr() if scratch is not None else None, _stream()),
           "sample_rows")


# --------------------------------------------------------------------------- several residual streams
MAX_STREAMS = 8   # streams.cu


def streams_combine(x: torch.Tensor, out: torch.Tensor, mix: torch.Tensor, write: torch.Tensor | None = None,
                    y: torch.Tensor | None = None) -> None:
    """out[t, j] = sum_a mix[a, j] x[t, a] (+ write[j] y[t]) over float32 streams x [T, S_in, width] -> out
    [T, S_out, width]; ``out`` may be ``x`` when S_in == S_out."""
    _dev(x, out, mix, write, y)
    T, s_in, width = x.shape
    s_out = out.shape[1]
    assert x.dtype == out.dtype == mix.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
    assert out.shape[0] == T and out.shape[2] == width and mix.is_contiguous() and mix.numel() == s_in * s_out
    if y is not None:
        assert write is not None and write.dtype == y.dtype == torch.float32 and write.numel() == s_out
        assert y.is_contiguous() and tuple(y.shape) == (T, width)
    _check(_fn("b200_streams_combine")(x.data_ptr(), out.data_ptr(), mix.data_ptr(),
                                       write.data_ptr() if y is not None else None, y.data_ptr() if y is not None else None,
                                       T, s_in, s_out, width, _stream()), "streams_combine")


def streams_read_norm(x: torch.Tensor, read: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
                      rows: torch.Tensor | None = None) -> None:
    """out[r] = weight * u / sqrt(mean(u^2) + eps), u = sum_a read[a] x[rows[r], a]: x float32 [T, S, width]."""
    _dev(x, read, weight, out, rows)
    T, s, width = x.shape
    assert x.dtype == read.dtype == weight.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
    assert read.numel() == s and weight.numel() == width and out.shape[1] == width
    n_rows = out.shape[0]
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.numel() == n_rows
    else:
        assert n_rows == T
    _check(_fn("b200_streams_read_norm")(x.data_ptr(), read.data_ptr(), weight.data_ptr(), out.data_ptr(),
                                         dtype_code(out.dtype), rows.data_ptr() if rows is not None else None, n_rows, s,
                                         width, float(eps), _stream()), "streams_read_norm")


def streams_step(x: torch.Tensor, mix: torch.Tensor, write: torch.Tensor, y: torch.Tensor, read: torch.Tensor | None = None,
                 weight: torch.Tensor | None = None, out: torch.Tensor | None = None, eps: float = 0.0) -> None:
    """One sublayer's write-back and the next one's read in one pass: x[t, j] <- sum_a mix[a, j] x[t, a] + write[j] y[t]
    in place, y <- 0, and with ``read``: out[t] = weight * u / sqrt(mean(u^2) + eps), u = sum_j read[j] x[t, j]."""
    _dev(x, mix, write, y, read, weight, out)
    T, s, width = x.shape
    assert x.dtype == mix.dtype == write.dtype == y.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous()
    assert mix.is_contiguous() and mix.numel() == s * s and write.numel() == s and tuple(y.shape) == (T, width)
    if read is not None:
        assert read.dtype == weight.dtype == torch.float32 and read.numel() == s and weight.numel() == width
        assert out.is_contiguous() and tuple(out.shape) == (T, width)
    _check(_fn("b200_streams_step")(x.data_ptr(), mix.data_ptr(), write.data_ptr(), y.data_ptr(),
                                    read.data_ptr() if read is not None else None,
                                    weight.data_ptr() if read is not None else None,
                                    out.data_ptr() if read is not None else None,
                                    dtype_code(out.dtype) if read is not None else 0, T, s, width, float(eps), _stream()),
           "streams_step")


# --------------------------------------------------------------------------- rows of a projection, per head
TO_ROWS, TO_CACHE_KEYS, TO_CACHE_VALUES = 0, 1, 2


ROW_WORDS = 20   # 32-bit words of one segment record (head_rows.cu: kSegmentWords)


def head_row_segment(src_off: int, n_rows: int, d: int, dst_off: int, d_pad: int | None = None, bias_off: int = -1,
                     norm: bool | int = False, weight_off: int = -1, mul: float = 1.0, target: int = TO_ROWS,
                     weight_per_row: bool = False, mix_off: int = -1, rotate: bool = False, src_stride: int = -1,
                     dst_stride: int = -1, cache_dim: int = -1, lead: int = 0) -> list[int]:
    """One segment of ``head_rows``: ``n_rows`` rows of ``d`` numbers from column ``src_off`` on, each (+ bias)
    (normalised) (* weight) * mul, written ``d_pad`` wide (zeros behind the ``d``) from column ``dst_off`` on, or with
    ``target`` TO_CACHE_KEYS / TO_CACHE_VALUES into the cache page of the token's position (``n_rows`` = the cache
    entry's kv heads, ``d_pad`` its head size).  ``norm``: True / 1 per row, 2 over all rows of the segment at once
    (the weight then usually has an entry per element: ``weight_per_row``).  ``mix_off``: the column of ``head_rows``'s
    ``other`` rows this segment is mixed with.  ``rotate``: the row's interleaved pairs (2i, 2i + 1) are turned by the
    token's position times ``head_rows``'s ``rotary`` frequencies (``mul`` then also carries a factor on cosine and sine).
    ``src_stride`` / ``dst_stride``: numbers between two rows read / written when they do not lie back to back (a source
    stride of 0: all rows read the same numbers).  ``cache_dim``: the row size of the cache, when the segment fills only
    the ``d_pad`` columns from ``dst_off`` on of every cache row.  ``lead``: how many of the ``d_pad`` numbers written are
    zeros in front of the row's ``d`` (the rest of the zeros follow it)."""
    import struct

    return [src_off, n_rows, d, dst_off, d if d_pad is None else d_pad, bias_off, int(norm), weight_off,
            struct.unpack("<i", struct.pack("<f", float(mul)))[0], target, 1 if weight_per_row else 0, mix_off,
            1 if rotate else 0, src_stride, dst_stride, cache_dim, int(lead), 0, 0, 0]


def head_rows(src: torch.Tensor, dst: torch.Tensor | None, segments, eps: float = 0.0, bias: torch.Tensor | None = None,
              weight: torch.Tensor | None = None, cache=None, mix=None, rotary=None) -> None:
    """``segments``: a ctypes array made by ``head_row_segments`` (at most six segments).  ``cache``: (positions,
    seq_ids, page_table, k_pool, v_pool) for segments that go into the paged cache; ``dst`` may be None when all do.
    ``mix``: (other [T, >= ...] of src's dtype, lambda float32 [1]) for segments with a ``mix_off``.  ``rotary``:
    (positions int32 [T], inverse frequencies float32 [>= d / 2]) for segments that rotate."""
    _dev(src, dst, bias, weight)
    assert src.stride(1) == 1
    assert dst is None or (src.dtype == dst.dtype and dst.stride(1) == 1 and src.shape[0] == dst.shape[0])
    assert bias is None or (bias.dtype == torch.float32 and bias.is_contiguous())
    assert weight is None or (weight.dtype == torch.float32 and weight.is_contiguous())
    pos = seq = table = k_pool = v_pool = None
    if cache is not None:
        pos, seq, table, k_pool, v_pool = cache
        _dev(pos, seq, table, k_pool, v_pool)
        assert pos.dtype == seq.dtype == table.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
        assert k_pool.dtype == v_pool.dtype == src.dtype and k_pool.is_contiguous() and v_pool.is_contiguous()
    other = lam = None
    if mix is not None:
        other, lam = mix
        _dev(other, lam)
        assert other.dtype == src.dtype and other.stride(1) == 1 and other.shape[0] == src.shape[0]
        assert lam.dtype == torch.float32 and lam.numel() == 1
    inv_freq = None
    if rotary is not None:
        rot_pos, inv_freq = rotary
        _dev(rot_pos, inv_freq)
        assert rot_pos.dtype == torch.int32 and inv_freq.dtype == torch.float32 and inv_freq.is_contiguous()
        assert pos is None or pos.data_ptr() == rot_pos.data_ptr()
        pos = rot_pos
    ptr = lambda t: t.data_ptr() if t is not None else None
    _check(_fn("b200_head_rows")(src.data_ptr(), src.stride(0), ptr(dst), dst.stride(0) if dst is not None else 0,
                                 dtype_code(src.dtype), ptr(bias), ptr(weight), ctypes.addressof(segments),
                                 len(segments) // ROW_WORDS, src.shape[0], float(eps), ptr(pos), ptr(seq), ptr(table),
                                 table.shape[1] if table is not None else 0, ptr(k_pool), ptr(v_pool), ptr(other),
                                 other.stride(0) if other is not None else 0, ptr(lam), ptr(inv_freq), _stream()), "head_rows")


def head_row_segments(*segments: list[int]):
    """The segments of one ``head_rows`` launch as the C function reads them (kept by the part that made them)."""
    flat = [v for s in segments for v in s]
    return (ctypes.c_int * len(flat))(*flat)


# --------------------------------------------------------------------------- small per-element kernels
def softcap_rows(logits: torch.Tensor, cap: float) -> None:
    """logits <- cap * tanh(logits / cap), in place (float32)."""
    _dev(logits)
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    _check(_fn("b200_softcap_rows")(logits.data_ptr(), logits.numel(), float(cap), _stream()), "softcap_rows")


GATE_ACTIVATIONS = {"sigmoid": 0, "silu": 1}


def gated_rmsnorm(x: torch.Tensor, weight: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, n_heads: int, d: int,
                  eps: float, activation: str = "sigmoid", gate_first: bool = False) -> None:
    """Per (token, head) row of float32 x [T, n_heads d]: x / sqrt(mean(x^2) + eps) * weight[d] * act(gate), act the
    sigmoid or SiLU.  ``gate_first``: the row is multiplied by act(gate) first and the norm runs over the gated row.
    A weight of n_heads * d numbers gives every row weights of its own (the rows are then any equal parts of x's rows)."""
    _dev(x, weight, gate, out)
    assert x.dtype == weight.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and gate.stride(1) == 1
    assert x.shape[1] == n_heads * d == out.shape[1] and gate.shape[1] >= n_heads * d and weight.numel() in (d, n_heads * d)
    assert gate.dtype == out.dtype and weight.is_contiguous()
    per_row = weight.numel() != d
    _check(_fn("b200_gated_rmsnorm")(x.data_ptr(), weight.data_ptr(), gate.data_ptr(), gate.stride(0), out.data_ptr(),
                                     dtype_code(out.dtype), x.shape[0], n_heads, d, float(eps),
                                     GATE_ACTIVATIONS[activation], 1 if gate_first else 0, 1 if per_row else 0, _stream()),
           "gated_rmsnorm")


def gate_rows(x: torch.Tensor, gate: torch.Tensor, activation: str = "sigmoid") -> None:
    """x[t, :] <- x[t, :] * act(gate[t, :x.shape[1]]) in place, act the sigmoid or SiLU, evaluated in 32 bits."""
    _dev(x, gate)
    assert x.dtype == gate.dtype and x.stride(1) == 1 and gate.stride(1) == 1
    assert gate.shape[0] == x.shape[0] and gate.shape[1] >= x.shape[1]
    _check(_fn("b200_gate_rows")(x.data_ptr(), x.stride(0), gate.data_ptr(), gate.stride(0), dtype_code(x.dtype), x.shape[0],
                                 x.shape[1], GATE_ACTIVATIONS[activation], _stream()), "gate_rows")


def scale_rows(logits: torch.Tensor, scale: float) -> None:
    """logits <- logits * scale, in place (float32)."""
    _dev(logits)
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    _check(_fn("b200_scale_rows")(logits.data_ptr(), logits.numel(), float(scale), _stream()), "scale_rows")


def differential_heads(maps: torch.Tensor, gate: torch.Tensor | None, out: torch.Tensor, n_heads: int, d: int, d_pad: int,
                       weight: float, post: float, eps: float) -> None:
    """maps [T, 2 n_heads d_pad]: heads (2h, 2h + 1) are two attention maps' results over the same values.  out[t, h] =
    post * o / sqrt(mean(o^2) + eps) * sigmoid(gate[t, h]) over the first ``d`` numbers, o = map 1 - weight * map 2."""
    _dev(maps, gate, out)
    assert maps.is_contiguous() and out.is_contiguous() and maps.dtype == out.dtype
    assert maps.shape[1] == 2 * n_heads * d_pad and out.shape[1] == n_heads * d and maps.shape[0] == out.shape[0]
    assert gate is None or (gate.dtype == out.dtype and gate.stride(1) == 1 and gate.shape[1] >= n_heads * d)
    _check(_fn("b200_differential_heads")(maps.data_ptr(), gate.data_ptr() if gate is not None else None,
                                          gate.stride(0) if gate is not None else 0, out.data_ptr(), dtype_code(out.dtype),
                                          out.shape[0], int(n_heads), int(d), int(d_pad), float(weight), float(post), float(eps),
                                          _stream()), "differential_heads")


# --------------------------------------------------------------------------- a block that gates and norms what its sublayers return
def gated_norm_step(y: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, x: torch.Tensor, eps: float, *,
                    gate: torch.Tensor | None = None, gate_bias: torch.Tensor | None = None,
                    y_bias: torch.Tensor | None = None, cast: torch.Tensor | None = None, center: bool = True,
                    levels: torch.Tensor | None = None, n: int = 0, coefficients: torch.Tensor | None = None,
                    read=None) -> None:
    """z = (y (+ y_bias)) * sigmoid(gate (+ gate_bias)); x <- x + layer_norm(z) * weight + bias (``center`` False: x <- x +
    weight * z / rms(z)); y <- 0; ``cast`` receives the new x in its own type.  x, y [T, dim], the vectors float32;
    ``gate`` [T, >= dim], float32 or bfloat16 (None: no gate).  With ``levels`` (float32 [> n, T, dim]) the new x is filed as
    level ``n`` and what stays as the stream (and in ``cast``) is sum_(j <= n) coefficients[j] levels[j], as ``depth_average``.
    ``read`` = (conv_weight float32 [dim, taps], conv_state float32 [slots, >= (taps - 1) * dim], slots int32 [T], update,
    out [T, dim]) in a step in which every sequence brings one token: ``out`` receives the stream as it is left plus a
    convolution over time on it, h + sum_j conv_weight[:, j] h_(t - taps + 1 + j), the older inputs from the state at
    ``slots[t]`` (oldest first), which moves on by this token with ``update``: what the next block's mixer reads."""
    _dev(y, weight, bias, x, gate, gate_bias, y_bias, cast)
    T, dim = x.shape
    assert x.dtype == y.dtype == weight.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous() and x.shape == y.shape
    for v in (weight, bias, gate_bias, y_bias):
        assert v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == dim)
    assert gate is None or (gate.stride(1) == 1 and gate.shape[0] == T and gate.shape[1] >= dim)
    assert cast is None or (cast.is_contiguous() and cast.shape == x.shape)
    if levels is not None:
        _dev(levels, coefficients)
        assert levels.dtype == coefficients.dtype == torch.float32 and levels.is_contiguous() and coefficients.is_contiguous()
        assert levels.shape[0] > n >= 0 and tuple(levels.shape[1:]) == (T, dim) and coefficients.numel() == n + 1
    conv = (None, None, 0, None, 0, 0, None)
    out_type = cast.dtype if cast is not None else None
    if read is not None:
        conv_w, conv_state, slots, update, out = read
        _dev(conv_w, conv_state, slots, out)
        taps = conv_w.shape[1]
        assert conv_w.dtype == conv_state.dtype == torch.float32 and conv_w.is_contiguous() and conv_w.shape[0] == dim
        assert conv_state.stride(1) == 1 and (taps < 2 or conv_state.shape[1] >= (taps - 1) * dim)
        assert slots.dtype == torch.int32 and slots.numel() == T and out.is_contiguous() and out.shape == x.shape
        assert out_type is None or out_type == out.dtype
        out_type = out.dtype
        conv = (conv_w.data_ptr(), conv_state.data_ptr(), conv_state.stride(0), slots.data_ptr(), taps, 1 if update else 0,
                out.data_ptr())
    ptr = lambda t: t.data_ptr() if t is not None else None
    _check(_fn("b200_gated_norm_step")(y.data_ptr(), ptr(y_bias), ptr(gate), gate.stride(0) if gate is not None else 0,
                                       dtype_code(gate.dtype) if gate is not None else F32, ptr(gate_bias), weight.data_ptr(),
                                       ptr(bias), x.data_ptr(), ptr(cast), dtype_code(out_type) if out_type is not None else F32,
                                       T, dim, float(eps), 1 if center else 0, ptr(levels),
                                       levels.stride(0) if levels is not None else 0, int(n), ptr(coefficients), *conv, _stream()),
           "gated_norm_step")


def depth_average(levels: torch.Tensor, n: int, coefficients: torch.Tensor, x: torch.Tensor,
                  cast: torch.Tensor | None = None) -> None:
    """levels[n] = x; x <- sum_(j <= n) coefficients[j] levels[j]; ``cast`` receives the new x in its own type.
    levels float32 [>= n + 1, T, dim], x float32 [T, dim], coefficients float32 [n + 1] on the device."""
    _dev(levels, coefficients, x, cast)
    assert levels.dtype == x.dtype == coefficients.dtype == torch.float32 and levels.is_contiguous() and x.is_contiguous()
    assert levels.shape[0] > n >= 0 and tuple(levels.shape[1:]) == tuple(x.shape) and coefficients.numel() == n + 1
    assert coefficients.is_contiguous() and (cast is None or (cast.is_contiguous() and cast.shape == x.shape))
    _check(_fn("b200_depth_average")(levels.data_ptr(), levels.stride(0), int(n), coefficients.data_ptr(), x.data_ptr(),
                                     cast.data_ptr() if cast is not None else None,
                                     dtype_code(cast.dtype) if cast is not None else F32, x.numel(), _stream()), "depth_average")


def cast_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = x (float32) in out's type."""
    _dev(x, out)
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and x.shape == out.shape
    _check(_fn("b200_cast_rows")(x.data_ptr(), out.data_ptr(), dtype_code(out.dtype), x.numel(), _stream()), "cast_rows")


UNGATED_ACTIVATIONS = {"relu_squared": 0}


def bias_act_rows(u: torch.Tensor, bias: torch.Tensor | None, activation: str = "relu_squared") -> None:
    """u <- act(u + bias) in place on a product's result [T, n]; ``relu_squared``: max(., 0)^2, evaluated in 32 bits."""
    _dev(u, bias)
    assert u.stride(1) == 1 and (bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == u.shape[1]))
    _check(_fn("b200_bias_act_rows")(u.data_ptr(), u.stride(0), dtype_code(u.dtype), bias.data_ptr() if bias is not None else None,
                                     u.shape[0], u.shape[1], UNGATED_ACTIVATIONS[activation], _stream()), "bias_act_rows")


def token_gate_rows(a: torch.Tensor, tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor, n: int) -> None:
    """out[t, j] = gelu_tanh(a[t, j]) * table[tokens[t], j] for j < n, 0 for the further columns of out."""
    _dev(a, tokens, table, out)
    assert a.dtype == out.dtype and a.stride(1) == 1 and out.stride(1) == 1 and table.stride(1) == 1
    assert tokens.dtype == torch.int32 and tokens.numel() == a.shape[0] == out.shape[0]
    assert a.shape[1] >= n and table.shape[1] >= n and out.shape[1] >= n
    _check(_fn("b200_token_gate_rows")(a.data_ptr(), a.stride(0), dtype_code(a.dtype), tokens.data_ptr(), table.data_ptr(),
                                       dtype_code(table.dtype), table.stride(0), table.shape[0], out.data_ptr(), out.stride(0),
                                       a.shape[0], int(n), out.shape[1], _stream()), "token_gate_rows")


# --------------------------------------------------------------------------- norms in groups, and a block that norms both ways
def group_rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float, groups: int,
                  rows: torch.Tensor | None = None) -> None:
    """out[r] = weight * x[rows[r]] / rms, every row cut into ``groups`` equal consecutive parts that are each divided by
    their own sqrt(mean(part^2) + eps).  x and weight float32."""
    _dev(x, weight, out, rows)
    assert x.dtype == weight.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and weight.is_contiguous()
    n_rows, dim = out.shape
    assert x.shape[1] == dim and weight.numel() == dim
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.numel() == n_rows
    _check(_fn("b200_group_rmsnorm")(x.data_ptr(), weight.data_ptr(), out.data_ptr(), dtype_code(out.dtype),
                                     rows.data_ptr() if rows is not None else None, n_rows, dim, int(groups), float(eps),
                                     _stream()), "group_rmsnorm")


def sandwich_step(y: torch.Tensor, weight: torch.Tensor, mult: float, x: torch.Tensor, eps: float, groups: int, *,
                  offset: torch.Tensor | None = None, next_weight: torch.Tensor | None = None,
                  out: torch.Tensor | None = None) -> None:
    """x <- x + mult * (weight * y / rms_groups(y)) (+ offset); y <- 0; and, with ``next_weight`` and ``out``,
    out = next_weight * x / rms_groups(x) of the updated rows.  x, y [T, dim] and the weights float32."""
    _dev(y, weight, x, offset, next_weight, out)
    assert x.dtype == y.dtype == weight.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous()
    assert x.shape == y.shape and weight.numel() == x.shape[1] and weight.is_contiguous()
    assert offset is None or (offset.dtype == torch.float32 and offset.is_contiguous() and offset.numel() == x.shape[1])
    assert (next_weight is None) == (out is None)
    if out is not None:
        assert next_weight.dtype == torch.float32 and next_weight.is_contiguous() and next_weight.numel() == x.shape[1]
        assert out.is_contiguous() and out.shape == x.shape
    ptr = lambda t: t.data_ptr() if t is not None else None
    _check(_fn("b200_sandwich_step")(y.data_ptr(), weight.data_ptr(), float(mult), x.data_ptr(), ptr(offset), ptr(next_weight),
                                     ptr(out), dtype_code(out.dtype) if out is not None else F32, x.shape[0], x.shape[1],
                                     int(groups), float(eps), _stream()), "sandwich_step")


def sandwich_step_conv_fits(dim: int, groups: int) -> bool:
    """Whether ``sandwich_step_conv`` takes rows of ``dim`` numbers normed in ``groups`` parts (whole pieces of 128
    numbers per part, at most 8192 numbers: the sizes of sandwich_step_rows_kernel in sandwich.cu)."""
    return groups >= 1 and dim % groups == 0 and (dim // groups) % 128 == 0 and dim <= 8192


def sandwich_step_conv(y: torch.Tensor, weight: torch.Tensor, mult: float, x: torch.Tensor, eps: float, groups: int,
                       next_weight: torch.Tensor, out: torch.Tensor, conv_weight: torch.Tensor, conv_state: torch.Tensor,
                       slots: torch.Tensor, *, offset: torch.Tensor | None = None, update_state: bool = True) -> None:
    """``sandwich_step`` for a step in which every sequence brings one token, with the convolution over time that the
    next reader applies to the normed rows h: out = h + sum_j conv_weight[:, j] h_(t - taps + 1 + j).  The older inputs
    are rows of ``conv_state`` [slots, >= (taps - 1) * dim] (oldest first) at ``slots[t]``; with ``update_state`` the
    state moves on by this token.  ``out`` may be of the run's type."""
    _dev(y, weight, x, offset, next_weight, out, conv_weight, conv_state, slots)
    T, dim = x.shape
    taps = conv_weight.shape[1]
    assert x.dtype == y.dtype == weight.dtype == next_weight.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous()
    assert x.shape == y.shape == out.shape and out.is_contiguous() and weight.numel() == dim and next_weight.numel() == dim
    assert weight.is_contiguous() and next_weight.is_contiguous()
    assert offset is None or (offset.dtype == torch.float32 and offset.is_contiguous() and offset.numel() == dim)
    assert conv_weight.dtype == conv_state.dtype == torch.float32 and conv_weight.is_contiguous() and conv_weight.shape[0] == dim
    assert conv_state.stride(1) == 1 and (taps < 2 or conv_state.shape[1] >= (taps - 1) * dim)
    assert slots.dtype == torch.int32 and slots.numel() == T
    _check(_fn("b200_sandwich_step_conv")(y.data_ptr(), weight.data_ptr(), float(mult), x.data_ptr(),
                                          offset.data_ptr() if offset is not None else None, next_weight.data_ptr(),
                                          out.data_ptr(), dtype_code(out.dtype), T, dim, int(groups), float(eps),
                                          conv_weight.data_ptr(), conv_state.data_ptr(), conv_state.stride(0), slots.data_ptr(),
                                          taps, int(bool(update_state)), _stream()), "sandwich_step_conv")


def add_row(x: torch.Tensor, row: torch.Tensor) -> None:
    """x[t] += row for every row t of float32 x [T, dim]."""
    _dev(x, row)
    assert x.dtype == row.dtype == torch.float32 and x.is_contiguous() and row.is_contiguous() and row.numel() == x.shape[1]
    _check(_fn("b200_add_row")(x.data_ptr(), row.data_ptr(), x.shape[0], x.shape[1], _stream()), "add_row")


# --------------------------------------------------------------------------- short convolution and the delta rule
MAX_CONV_TAPS = 16   # delta_rule.cu


def causal_conv_silu(x: torch.Tensor, weight: torch.Tensor, state: torch.Tensor, slots: torch.Tensor,
                     seq_ids: torch.Tensor, cu_seqlens: torch.Tensor, out: torch.Tensor, channels: int,
                     update_state: bool = True) -> None:
    """out[t, c] = silu(sum_j weight[c, j] x[t - (taps - 1) + j, c]) per sequence of the packed step; inputs before
    the step come from ``state`` [slots, >= (taps - 1) * channels] (float32, oldest first), which then takes the
    step's last taps - 1 inputs.  x [T, >= channels]."""
    _dev(x, weight, state, slots, seq_ids, cu_seqlens, out)
    taps = weight.shape[1]
    assert weight.dtype == state.dtype == torch.float32 and weight.is_contiguous() and weight.shape[0] == channels
    assert x.dtype == out.dtype and x.stride(1) == 1 and out.stride(1) == 1 and state.stride(1) == 1
    assert state.shape[1] >= (taps - 1) * channels
    _check(_fn("b200_causal_conv_silu")(x.data_ptr(), x.stride(0), weight.data_ptr(), state.data_ptr(), state.stride(0),
                                        slots.data_ptr(), seq_ids.data_ptr(), cu_seqlens.data_ptr(), out.data_ptr(),
                                        out.stride(0), dtype_code(x.dtype), x.shape[0], slots.numel(), channels, taps,
                                        1 if update_state else 0, _stream()), "causal_conv_silu")


CONV_ACTIVATIONS = {None: 0, "silu": 1}


def causal_conv(x: torch.Tensor, weight: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, seq_ids: torch.Tensor,
                cu_seqlens: torch.Tensor, out: torch.Tensor, channels: int, *, bias: torch.Tensor | None = None,
                activation: str | None = None, add_input: bool = False, update_state: bool = True) -> None:
    """The short causal convolution in its general form: out[t, c] = act(bias[c] + sum_j weight[c, j] x[t - (taps - 1) + j, c])
    (+ x[t, c] with ``add_input``) per sequence of the packed step; x and out may differ in type.  State as for
    ``causal_conv_silu``: float32 [slots, >= (taps - 1) * channels], the sequence's last taps - 1 inputs, oldest first."""
    _dev(x, weight, state, slots, seq_ids, cu_seqlens, out, bias)
    taps = weight.shape[1]
    assert weight.dtype == state.dtype == torch.float32 and weight.is_contiguous() and weight.shape[0] == channels
    assert x.stride(1) == 1 and out.stride(1) == 1 and state.stride(1) == 1 and x.shape[0] == out.shape[0]
    assert x.shape[1] >= channels and out.shape[1] >= channels and state.shape[1] >= (taps - 1) * channels
    assert bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == channels)
    _check(_fn("b200_causal_conv")(x.data_ptr(), x.stride(0), dtype_code(x.dtype), weight.data_ptr(),
                                   bias.data_ptr() if bias is not None else None, state.data_ptr(), state.stride(0),
                                   slots.data_ptr(), seq_ids.data_ptr(), cu_seqlens.data_ptr(), out.data_ptr(), out.stride(0),
                                   dtype_code(out.dtype), x.shape[0], slots.numel(), channels, taps,
                                   CONV_ACTIVATIONS[activation], 1 if add_input else 0, 1 if update_state else 0, _stream()),
           "causal_conv")


DECAY_SOFTPLUS_RATE, DECAY_SIGMOID_POWER = 0, 1


def linear_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, state: torch.Tensor,
                slots: torch.Tensor, cu_seqlens: torch.Tensor, out: torch.Tensor, heads: int, kv_heads: int, d_k: int,
                d_v: int, *, decay_kind: int, decay_per_head: bool = False, decay_bias: torch.Tensor | None = None,
                a_log: torch.Tensor | None = None, power: float = 1.0, q_scale: float = 1.0,
                step_scales_value: bool = False, skip: torch.Tensor | None = None, alloc=None) -> None:
    """The recurrence S <- diag(g) S + k (beta v)^T, o = S^T q + skip v per head over a packed step (no delta correction).
    q, k [T, >= kv_heads d_k] (head h reads head h // (heads // kv_heads)), v [T, >= heads d_v], decay [T, >= heads d_k]
    (or [T, >= heads] with ``decay_per_head``) before its bias and activation, all of one type; g =
    exp(-exp(a_log[h]) softplus(decay + bias)) (``DECAY_SOFTPLUS_RATE``) or sigmoid(decay + bias)^power
    (``DECAY_SIGMOID_POWER``); beta = 1, or the step size softplus(decay + bias) with ``step_scales_value``.  state float32
    [slots, >= heads d_k d_v], updated in place; out float32 [T, heads d_v]; everything but the operands' storage is 32-bit."""
    _dev(q, k, v, decay, state, slots, cu_seqlens, out, decay_bias, a_log, skip)
    assert q.dtype == k.dtype == v.dtype == decay.dtype and q.stride(1) == k.stride(1) == v.stride(1) == decay.stride(1) == 1
    assert state.dtype == out.dtype == torch.float32 and out.is_contiguous() and state.stride(1) == 1
    n_decay = heads if decay_per_head else heads * d_k
    assert q.shape[1] >= kv_heads * d_k and k.shape[1] >= kv_heads * d_k and v.shape[1] >= heads * d_v and decay.shape[1] >= n_decay
    for t, n in ((decay_bias, n_decay), (a_log, heads), (skip, heads)):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == n)
    assert decay_kind != DECAY_SOFTPLUS_RATE or a_log is not None
    assert not step_scales_value or (decay_per_head and decay_kind == DECAY_SOFTPLUS_RATE)
    assert state.shape[1] >= heads * d_k * d_v and out.shape[1] == heads * d_v and out.shape[0] == q.shape[0]
    lib = library("delta_rule")
    shape = (heads, q.shape[0], int(lib.b200_delta_rule_row(c_int(d_k), c_int(d_v))))
    scratch = alloc(shape, torch.float32) if alloc is not None else torch.empty(shape, dtype=torch.float32, device=q.device)
    ptr = lambda t: t.data_ptr() if t is not None else None
    _check(_fn("b200_linear_scan")(q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0),
                                   decay.data_ptr(), decay.stride(0), ptr(decay_bias), ptr(a_log), ptr(skip), state.data_ptr(),
                                   state.stride(0), slots.data_ptr(), cu_seqlens.data_ptr(), out.data_ptr(), scratch.data_ptr(),
                                   dtype_code(q.dtype), q.shape[0], slots.numel(), heads, kv_heads, d_k, d_v, float(q_scale),
                                   float(power), int(decay_kind), 1 if decay_per_head else 0, 1 if step_scales_value else 0,
                                   _stream()), "linear_scan")


def delta_rule_supported(d_k: int) -> bool:
    lib = library("delta_rule")
    a, b = c_int(0), c_int(0)
    return bool(lib.b200_delta_rule_plan(c_int(d_k), ctypes.byref(a), ctypes.byref(b)))


def delta_rule_scan(qkv: torch.Tensor, beta: torch.Tensor, decay: torch.Tensor, dt_bias: torch.Tensor,
                    a_log: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, cu_seqlens: torch.Tensor,
                    out: torch.Tensor, heads: int, kv_heads: int, d_k: int, d_v: int, q_scale: float,
                    unit_eps: float, alloc=None, decay_per_head: bool = False) -> None:
    """The gated delta rule over a packed step.  qkv [T, 2 kv_heads d_k + heads d_v] (after the convolution), beta
    [T, >= heads] and decay [T, >= heads d_k] as the projections leave them, state float32 [slots, >= heads d_k d_v]
    (updated in place), out float32 [T, heads d_v].  ``decay_per_head``: decay [T, >= heads] and dt_bias [heads], one
    decay for all key channels of a head.  ``alloc(shape, dtype)``: where the scan's scratch (a row of
    32-bit numbers per token and head) comes from."""
    _dev(qkv, beta, decay, dt_bias, a_log, state, slots, cu_seqlens, out)
    assert qkv.dtype == beta.dtype == decay.dtype and qkv.stride(1) == beta.stride(1) == decay.stride(1) == 1
    assert dt_bias.dtype == a_log.dtype == state.dtype == out.dtype == torch.float32 and out.is_contiguous()
    assert dt_bias.numel() == (heads if decay_per_head else heads * d_k) and a_log.numel() == heads and state.stride(1) == 1
    assert decay.shape[1] >= (heads if decay_per_head else heads * d_k)
    assert state.shape[1] >= heads * d_k * d_v and out.shape[1] == heads * d_v and out.shape[0] == qkv.shape[0]
    lib = library("delta_rule")
    shape = (heads, qkv.shape[0], int(lib.b200_delta_rule_row(c_int(d_k), c_int(d_v))))
    scratch = alloc(shape, torch.float32) if alloc is not None else torch.empty(shape, dtype=torch.float32, device=qkv.device)
    _check(_fn("b200_delta_rule_scan")(qkv.data_ptr(), qkv.stride(0), beta.data_ptr(), beta.stride(0), decay.data_ptr(),
                                       decay.stride(0), dt_bias.data_ptr(), a_log.data_ptr(), state.data_ptr(),
                                       state.stride(0), slots.data_ptr(), cu_seqlens.data_ptr(), out.data_ptr(),
                                       scratch.data_ptr(), dtype_code(qkv.dtype), qkv.shape[0], slots.numel(), heads,
                                       kv_heads, d_k, d_v, float(q_scale), float(unit_eps),
                                       1 if decay_per_head else 0, _stream()), "delta_rule_scan")


# --------------------------------------------------------------------------- routed feed-forward (mixture of experts)
MAX_EXPERTS, MAX_EXPERTS_PER_TOKEN = 1024, 32   # moe.cu


def moe_route(h: torch.Tensor, router: torch.Tensor, chosen: torch.Tensor, weights: torch.Tensor, n_groups: int,
              keep_groups: int, norm_eps: float, scores: torch.Tensor | None = None, bias: torch.Tensor | None = None) -> None:
    """Per token of h [T, width]: softmax scores over router [E, width] (float32; ``bias`` float32 [E] joins the logits), the ``top`` = chosen.shape[1] best
    experts among the ``keep_groups`` best of ``n_groups`` groups of neighbours into chosen int32 [T, top], and
    their scores over the chosen scores' sum (+ norm_eps) into weights float32 [T, top]."""
    _dev(h, router, chosen, weights, scores)
    T, width = h.shape
    E = router.shape[0]
    assert router.dtype == torch.float32 and router.is_contiguous() and router.shape[1] == width and h.stride(1) == 1
    assert chosen.dtype == torch.int32 and weights.dtype == torch.float32 and chosen.is_contiguous() and weights.is_contiguous()
    assert chosen.shape == weights.shape and chosen.shape[0] == T
    assert scores is None or (scores.dtype == torch.float32 and scores.is_contiguous() and tuple(scores.shape) == (T, E))
    _dev(bias)
    assert bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == E)
    _check(_fn("b200_moe_route")(h.data_ptr(), h.stride(0), dtype_code(h.dtype), router.data_ptr(), chosen.data_ptr(),
                                 weights.data_ptr(), scores.data_ptr() if scores is not None else None, T, width, E,
                                 int(n_groups), int(keep_groups), chosen.shape[1], float(norm_eps),
                                 bias.data_ptr() if bias is not None else None, _stream()), "moe_route")


def moe_table_route(tokens: torch.Tensor, table: torch.Tensor, chosen: torch.Tensor, weights: torch.Tensor,
                    n_experts: int) -> None:
    """Routing by token id: chosen[t] = table[tokens[t]] (int32 [vocab, top]) and every weight 1 / top."""
    _dev(tokens, table, chosen, weights)
    T, top = chosen.shape
    assert tokens.dtype == table.dtype == chosen.dtype == torch.int32 and weights.dtype == torch.float32
    assert table.is_contiguous() and chosen.is_contiguous() and weights.is_contiguous() and table.shape[1] == top
    assert tokens.numel() == T and weights.shape == chosen.shape
    _check(_fn("b200_moe_table_route")(tokens.data_ptr(), table.data_ptr(), chosen.data_ptr(), weights.data_ptr(), T, top,
                                       int(n_experts), _stream()), "moe_table_route")


def moe_rows_takes(k: int, dtype: torch.dtype) -> bool:
    """Whether ``moe_rows`` can stage its eight rows of ``k`` numbers in shared memory."""
    return 8 * (k + 8) * (4 if dtype == torch.float32 else 2) + 4096 <= 200 * 1024


def moe_rows(a: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor, out: torch.Tensor, *, order: torch.Tensor | None = None,
             top: int = 1, activation: str | None = None, gate_args=(0.0, 0.0)) -> None:
    """One weight-streaming product per expert: out[p] = a[row(p)] @ w[e].T for the places p = offsets[e] ..
    offsets[e + 1] - 1 of expert e, row(p) = order[p] // top when ``order`` is given, p otherwise.  With ``activation``
    w [E, 2 n, K] holds gate and up rows interleaved and out [P, n] (a's dtype) receives the gated values; without, w
    [E, n, K] and out [P, n] float32.  The row counts are read on the device."""
    _dev(a, w, offsets, out, order)
    E, rows, K = w.shape
    gated = activation is not None
    n_out = rows // 2 if gated else rows
    assert a.dtype == w.dtype and w.is_contiguous() and a.stride(1) == 1 and a.shape[1] == K and out.stride(1) == 1
    assert out.shape[1] == n_out and out.dtype == (a.dtype if gated else torch.float32)
    assert offsets.dtype == torch.int32 and offsets.numel() == E + 1 and (order is None or order.dtype == torch.int32)
    _check(_fn("b200_moe_rows")(a.data_ptr(), a.stride(0), dtype_code(a.dtype), order.data_ptr() if order is not None else None,
                                int(top), w.data_ptr(), offsets.data_ptr(), out.data_ptr(), out.stride(0), E, K, n_out,
                                1 if gated else 0, ACTIVATION_CODES[activation] if gated else 0, float(gate_args[0]),
                                float(gate_args[1]), _stream()), "moe_rows")


def moe_group(chosen: torch.Tensor, n_experts: int, offsets: torch.Tensor, order: torch.Tensor, place: torch.Tensor) -> None:
    """Orders the (token, choice) pairs of chosen [T, top] by expert: offsets int32 [E + 1] (expert e's run),
    order int32 [T top] (the pair at each place), place int32 [T top] (each pair's place)."""
    _dev(chosen, offsets, order, place)
    n = chosen.numel()
    assert chosen.dtype == offsets.dtype == order.dtype == place.dtype == torch.int32
    assert offsets.numel() == n_experts + 1 and order.numel() == n and place.numel() == n
    _check(_fn("b200_moe_group")(chosen.data_ptr(), n, n_experts, offsets.data_ptr(), order.data_ptr(), place.data_ptr(),
                                 _stream()), "moe_group")


def moe_gather(h: torch.Tensor, order: torch.Tensor, out: torch.Tensor, top: int) -> None:
    """out[p] = h[order[p] // top]: the inputs in the order of their experts."""
    _dev(h, order, out)
    assert h.dtype == out.dtype and out.is_contiguous() and h.stride(1) == 1 and out.shape[1] == h.shape[1]
    _check(_fn("b200_moe_gather")(h.data_ptr(), h.stride(0), dtype_code(h.dtype), order.data_ptr(), out.data_ptr(),
                                  out.shape[0], h.shape[1], top, _stream()), "moe_gather")


def moe_combine(o: torch.Tensor, place: torch.Tensor, weights: torch.Tensor, residual: torch.Tensor) -> None:
    """residual[t] += sum_k weights[t, k] o[place[t top + k]] (o float32 [T top, width])."""
    _dev(o, place, weights, residual)
    T, top = weights.shape
    assert o.dtype == residual.dtype == weights.dtype == torch.float32 and o.is_contiguous() and residual.is_contiguous()
    assert o.shape[0] == T * top and o.shape[1] == residual.shape[1] and residual.shape[0] == T
    _check(_fn("b200_moe_combine")(o.data_ptr(), place.data_ptr(), weights.data_ptr(), residual.data_ptr(), T,
                                   residual.shape[1], top, _stream()), "moe_combine")
