"""Python face of the CUDA library: one function per kernel, torch tensors in.

The library is built by ``csrc/build.py`` (at the first call if it is missing
or stale) and loaded with ctypes.  There is no fallback: when the library
cannot be built or loaded, or a tensor does not live on a CUDA device, the call
raises.  Every function launches on torch's current stream.
"""

from __future__ import annotations

import ctypes
import os
import threading

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_DTYPE_TAG = {torch.float32: F32, torch.bfloat16: BF16}
ACTIVATIONS = {"none": 0, "gelu_erf": 1, "gelu_tanh": 2, "quick_gelu": 3, "relu2": 4, "silu": 5}

_lib = None
_lock = threading.Lock()


class KernelError(RuntimeError):
    """A kernel refused its arguments or its launch failed."""


def library():
    """The loaded library; builds it first if needed."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = _build.build()
                lib = ctypes.CDLL(str(path))
                lib.ayk_last_error.restype = ctypes.c_char_p
                _lib = lib
    return _lib


def library_file() -> str:
    return str(_build.library_path())


_initialised = False


def _ready():
    global _initialised
    lib = library()
    if not _initialised:
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: this package runs its kernels on a B200 and has no CPU path")
        _check(lib.ayk_init(ctypes.c_int(torch.cuda.current_device())))
        lib.ayk_set_pdl(ctypes.c_int(0 if os.environ.get("AYAKA_B200_PDL", "1") == "0" else 1))
        _initialised = True
    return lib


def set_pdl(on: bool) -> None:
    """Launch kernels with programmatic stream serialization (the default; the
    environment variable AYAKA_B200_PDL=0 switches it off): a kernel may be
    scheduled while its predecessor still runs and waits, on the device, for
    the predecessor's results before it touches them."""
    _ready().ayk_set_pdl(ctypes.c_int(1 if on else 0))


def set_split(parts: int | None) -> None:
    """Split along K in the product for many rows (``gemm_tc_prefill``, one-SM form): when the tiles
    alone would leave most SMs idle, the 2, 4 or 8 CTAs of a cluster share a tile, each with an equal
    part of its K blocks; they exchange their sums through shared memory and each finishes a share of
    the tile's columns.  None: the
    library decides per product (the default); 0: never; 2, 4, 8: wherever the tiles allow it."""
    _ready().ayk_gemm_tc_prefill_split(ctypes.c_int(-1 if parts is None else int(parts)))


def set_staged(on: bool) -> None:
    """The staged residual epilogue of ``gemm_tc_prefill`` (float32 out over a float32 residual: both
    through shared memory by TMA, whole lines at a time) where it applies (the default), or never."""
    _ready().ayk_gemm_tc_prefill_staged(ctypes.c_int(1 if on else 0))


def prefill_plan(M: int, N: int, K: int, sms: int = 148, wide_rows: bool = False) -> tuple[int, int]:
    """(tile width, parts of K per tile) that ``gemm_tc_prefill`` picks for an [M, K] x [N, K]^T product
    on ``sms`` SMs; ``wide_rows``: the epilogue reads or writes 32-bit rows.  Host arithmetic from the
    kernel's fitted time model: works without a GPU."""
    tile, parts = ctypes.c_int(0), ctypes.c_int(0)
    library().ayk_gemm_tc_prefill_plan(ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K), ctypes.c_int(sms),
                                       ctypes.c_int(1 if wide_rows else 0), ctypes.byref(tile), ctypes.byref(parts))
    return tile.value, parts.value


def last_staged() -> int:
    """Buffers per half through which the last ``gemm_tc_prefill`` staged its residual (0: it did not)."""
    return int(_ready().ayk_gemm_tc_prefill_last_staged())


def last_split() -> int:
    """Into how many parts the last ``gemm_tc_prefill`` (one-SM form) split the K blocks of its tiles."""
    return int(_ready().ayk_gemm_tc_prefill_last_split())


def _check(code: int) -> None:
    if code != 0:
        raise KernelError(library().ayk_last_error().decode("utf-8", "replace"))


launches = 0      # kernels of this library launched so far (graph replays are counted by their owner)


def _launch(code: int) -> None:
    global launches
    launches += 1
    _check(code)


def _ptr(t: torch.Tensor | None):
    if t is None:
        return ctypes.c_void_p(0)
    if not t.is_cuda:
        raise KernelError("tensor is not on a CUDA device")
    return ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _tag(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_TAG[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} is not supported (float32 or bfloat16)") from None


def _i32(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous int32 tensor")
    return t


# ---------------------------------------------------------------- kernels --

def embed(tokens: torch.Tensor, positions: torch.Tensor, table: torch.Tensor,
          position_table: torch.Tensor | None, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = table[tokens[t]] (+ position_table[positions[t]]), float32 [T, d]."""
    lib = _ready()
    T, d = tokens.numel(), table.shape[1]
    if out is None:
        out = torch.empty((T, d), dtype=torch.float32, device=table.device)
    if position_table is not None and (position_table.dtype != table.dtype or position_table.shape[1] != d):
        raise KernelError("position table must match the token table in dtype and width")
    if not table.is_contiguous() or (position_table is not None and not position_table.is_contiguous()):
        raise KernelError("embedding tables must be contiguous")
    _launch(lib.ayk_embed(_ptr(out), _ptr(_i32(tokens, "tokens")), _ptr(_i32(positions, "positions")),
                         _ptr(table), _ptr(position_table), ctypes.c_int(T), ctypes.c_int(d),
                         ctypes.c_int(_tag(table.dtype)), _stream()))
    return out


def layernorm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor | None, eps: float,
              out_dtype: torch.dtype, rows: torch.Tensor | None = None,
              out: torch.Tensor | None = None) -> torch.Tensor:
    """LayerNorm of float32 rows (of ``x[rows]`` when rows is given), result as out_dtype."""
    lib = _ready()
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("layernorm input must be contiguous float32")
    d = x.shape[-1]
    n = x.shape[0] if rows is None else rows.numel()
    if gamma.dtype != torch.float32 or gamma.numel() != d or (beta is not None and (beta.dtype != torch.float32 or beta.numel() != d)):
        raise KernelError("layernorm weight and bias must be float32 of the row width")
    if out is None:
        out = torch.empty((n, d), dtype=out_dtype, device=x.device)
    _launch(lib.ayk_layernorm(_ptr(out), _ptr(x), _ptr(gamma), _ptr(beta),
                             _ptr(None if rows is None else _i32(rows, "rows")), ctypes.c_int(n),
                             ctypes.c_int(d), ctypes.c_float(eps), ctypes.c_int(_tag(out_dtype)), _stream()))
    return out


def gemm_simt(a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
              activation: str = "none", residual: torch.Tensor | None = None,
              out_dtype: torch.dtype | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """act(a[M,K] @ w[N,K]^T + bias) (+ residual) on the FP32 pipes."""
    lib = _ready()
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or a.dtype != w.dtype or not a.is_contiguous() or not w.is_contiguous():
        raise KernelError(f"gemm operands do not fit: a {tuple(a.shape)} {a.dtype}, w {tuple(w.shape)} {w.dtype}")
    out_dtype = out_dtype or a.dtype
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    for name, t in (("bias", bias), ("residual", residual)):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise KernelError(f"{name} must be contiguous float32")
    if residual is not None and tuple(residual.shape) != (M, N):
        raise KernelError("residual must have the output's shape")
    _launch(lib.ayk_gemm_simt(_ptr(out), _ptr(a), _ptr(w), _ptr(bias), _ptr(residual), ctypes.c_int(M),
                             ctypes.c_int(N), ctypes.c_int(K), ctypes.c_int(ACTIVATIONS[activation]),
                             ctypes.c_int(_tag(a.dtype)), ctypes.c_int(_tag(out_dtype)), _stream()))
    return out


def kv_append(kcache: torch.Tensor, vcache: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
              row_req: torch.Tensor, positions: torch.Tensor, table: torch.Tensor) -> None:
    """cache[page, pos % P] = k/v row; k and v are column slices [T, Hkv*Dh] of one matrix."""
    lib = _ready()
    T, width = k.shape
    pages, P, Hkv, Dh = kcache.shape
    if width != Hkv * Dh or v.shape != k.shape or k.stride(1) != 1 or v.stride(1) != 1 or k.stride(0) != v.stride(0):
        raise KernelError("kv_append: keys and values must be [T, kv_heads*head_dim] slices with one row stride")
    if k.dtype != kcache.dtype or not kcache.is_contiguous() or not vcache.is_contiguous():
        raise KernelError("kv_append: cache must be contiguous and of the rows' dtype")
    _launch(lib.ayk_kv_append(_ptr(kcache), _ptr(vcache), _ptr(k), _ptr(v), ctypes.c_int(k.stride(0)),
                             _ptr(_i32(row_req, "row_req")), _ptr(_i32(positions, "positions")),
                             _ptr(_i32(table, "table")), ctypes.c_int(table.stride(0)), ctypes.c_int(P),
                             ctypes.c_int(T), ctypes.c_int(width), ctypes.c_int(_tag(k.dtype)), _stream()))


def attention_simt(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, table: torch.Tensor,
                   req_q_start: torch.Tensor, req_pos0: torch.Tensor, total_rows: int, num_heads: int,
                   scale: float, window: int | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention of the step's rows over the paged cache.  q: [T, H*Dh] slice."""
    lib = _ready()
    pages, P, Hkv, Dh = kcache.shape
    T = q.shape[0]
    if q.shape[1] != num_heads * Dh or q.stride(1) != 1 or q.dtype != kcache.dtype:
        raise KernelError("attention: q must be a [T, heads*head_dim] slice of the cache's dtype")
    if total_rows != T:
        raise KernelError(f"attention: {total_rows} rows named, q has {T} (rows beyond the count would stay unwritten)")
    if out is None:
        out = torch.empty((T, num_heads * Dh), dtype=q.dtype, device=q.device)
    R = req_pos0.numel()
    _launch(lib.ayk_attention_simt(_ptr(out), _ptr(q), ctypes.c_int(q.stride(0)), _ptr(kcache), _ptr(vcache),
                                  _ptr(_i32(table, "table")), ctypes.c_int(table.stride(0)),
                                  _ptr(_i32(req_q_start, "req_q_start")), _ptr(_i32(req_pos0, "req_pos0")),
                                  ctypes.c_int(R), ctypes.c_int(total_rows), ctypes.c_int(num_heads),
                                  ctypes.c_int(Hkv), ctypes.c_int(Dh), ctypes.c_int(P), ctypes.c_float(scale),
                                  ctypes.c_int(window or 0), ctypes.c_int(_tag(q.dtype)), _stream()))
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor | None = None,
           seed: torch.Tensor | None = None, offset: torch.Tensor | None = None,
           top_k: torch.Tensor | None = None, top_p: torch.Tensor | None = None,
           min_p: torch.Tensor | None = None) -> torch.Tensor:
    """One token per row of float32 logits: greedy where temperature is 0 or
    absent; else a draw after the top_k / top_p / min_p filters (null: off)."""
    lib = _ready()
    if logits.dtype != torch.float32 or not logits.is_contiguous() or logits.dim() != 2:
        raise KernelError("sample: logits must be contiguous float32 [S, V]")
    S, V = logits.shape
    out = torch.empty((S,), dtype=torch.int32, device=logits.device)
    if temperature is not None:
        if temperature.dtype != torch.float32 or seed.dtype != torch.int64 or offset.dtype != torch.int64:
            raise KernelError("sample: temperature float32, seed and offset int64")
    for name, t, dt in (("top_k", top_k, torch.int64), ("top_p", top_p, torch.float32), ("min_p", min_p, torch.float32)):
        if t is not None and (t.dtype != dt or t.numel() != S or not t.is_contiguous()):
            raise KernelError(f"sample: {name} must be a contiguous {dt} tensor with one value per row")
    _launch(lib.ayk_sample(_ptr(out), _ptr(logits), ctypes.c_int(S), ctypes.c_int(V), _ptr(temperature),
                          _ptr(seed), _ptr(offset), _ptr(top_k), _ptr(top_p), _ptr(min_p), _stream()))
    return out


def ban_tokens(logits: torch.Tensor, rows: torch.Tensor, tokens: torch.Tensor) -> None:
    """logits[rows[i], tokens[i]] = -inf, in place (int32 index tensors on the device)."""
    lib = _ready()
    if logits.dtype != torch.float32 or not logits.is_contiguous() or logits.dim() != 2:
        raise KernelError("ban_tokens: logits must be contiguous float32 [S, V]")
    if rows.numel() != tokens.numel():
        raise KernelError("ban_tokens: one row index per token id")
    S, V = logits.shape
    _launch(lib.ayk_ban_tokens(_ptr(logits), _ptr(_i32(rows, "rows")), _ptr(_i32(tokens, "tokens")),
                               ctypes.c_int(rows.numel()), ctypes.c_int(S), ctypes.c_int(V), _stream()))


# ------------------------------------------ rms norms, convolution, recurrences --

def _f32(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dtype != torch.float32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous float32 tensor")
    return t


def embed_scaled(tokens: torch.Tensor, table: torch.Tensor, scale: float) -> torch.Tensor:
    """out[t] = table[tokens[t]] * scale, float32 [T, d]."""
    lib = _ready()
    T, d = tokens.numel(), table.shape[1]
    if not table.is_contiguous():
        raise KernelError("embedding tables must be contiguous")
    out = torch.empty((T, d), dtype=torch.float32, device=table.device)
    _launch(lib.ayk_embed_scaled(_ptr(out), _ptr(_i32(tokens, "tokens")), _ptr(table), ctypes.c_int(T), ctypes.c_int(d),
                                 ctypes.c_float(scale), ctypes.c_int(_tag(table.dtype)), _stream()))
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor | None, eps: float, out_dtype: torch.dtype,
            rows: torch.Tensor | None = None, out: torch.Tensor | None = None, groups: int = 1) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * weight over the last axis of float32 rows (of ``x[rows]`` when rows
    is given).  ``x`` may be a column slice of a wider matrix; statistics and weight in 32-bit.
    ``groups`` > 1: the row is that many equal runs, each divided by its own root mean square."""
    lib = _ready()
    if x.dtype != torch.float32 or x.dim() != 2 or x.stride(1) != 1:
        raise KernelError("rmsnorm input must be float32 rows with unit column stride")
    d = x.shape[1]
    n = x.shape[0] if rows is None else rows.numel()
    if weight is not None and (weight.dtype != torch.float32 or weight.numel() != d or not weight.is_contiguous()):
        raise KernelError("rmsnorm weight must be float32 of the row width")
    if out is None:
        out = torch.empty((n, d), dtype=out_dtype, device=x.device)
    elif out.dtype != out_dtype or out.shape != (n, d) or out.stride(1) != 1:
        raise KernelError("rmsnorm: out must be [rows, width] of the output dtype")
    if groups < 1 or d % groups:
        raise KernelError(f"rmsnorm: a row of {d} is not {groups} equal groups")
    _launch(lib.ayk_rmsnorm_grouped(_ptr(out), ctypes.c_longlong(out.stride(0)), _ptr(x), ctypes.c_longlong(x.stride(0)),
                                    _ptr(weight), _ptr(None if rows is None else _i32(rows, "rows")), ctypes.c_int(n),
                                    ctypes.c_int(d), ctypes.c_int(groups), ctypes.c_float(eps),
                                    ctypes.c_int(_tag(out_dtype)), _stream()))
    return out


def rmsnorm_conv(x: torch.Tensor, weight: torch.Tensor, taps: torch.Tensor, state: torch.Tensor, ctx, eps: float,
                 out_dtype: torch.dtype) -> torch.Tensor:
    """h + conv(h) with h = rmsnorm(x) * weight: a causal convolution over time on every channel,
    ``taps`` [n, width] float32, tap-major (tap j multiplies the input n - 1 - j steps back).  The last n - 1
    inputs h of every request live in ``state`` [slots, n - 1, width] float32 and are brought up to
    date.  Rows, requests and slots come from the step context."""
    lib = _ready()
    T, d = x.shape
    n = taps.shape[0]
    _f32(x, "x"); _f32(weight, "weight"); _f32(taps, "taps"); _f32(state, "state")
    if taps.shape[1] != d or state.shape[1:] != (n - 1, d):
        raise KernelError("rmsnorm_conv: taps [n, width] and state [slots, n - 1, width] must fit the rows")
    out = torch.empty((T, d), dtype=out_dtype, device=x.device)
    launched = ctypes.c_int(0)
    code = lib.ayk_rmsnorm_conv(_ptr(out), _ptr(x), _ptr(weight), _ptr(taps), _ptr(state), _ptr(ctx.row_req),
                                _ptr(ctx.req_q_start), _ptr(ctx.req_slot), ctypes.c_int(T), ctypes.c_int(ctx.num_requests),
                                ctypes.c_int(d), ctypes.c_int(n), ctypes.c_float(eps), ctypes.c_int(ctx.max_q_len),
                                ctypes.c_int(_tag(out_dtype)), ctypes.byref(launched), _stream())
    global launches
    launches += launched.value
    _check(code)
    return out


def rmsnorm_residual(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, mult: float,
                     groups: int = 1) -> torch.Tensor:
    """x += mult * rmsnorm(y) * weight, in place on the float32 residual stream (``groups``: as in ``rmsnorm``)."""
    lib = _ready()
    _f32(x, "x"); _f32(y, "y"); _f32(weight, "weight")
    if x.shape != y.shape or weight.numel() != x.shape[1] or groups < 1 or x.shape[1] % groups:
        raise KernelError("rmsnorm_residual: shapes do not fit")
    _launch(lib.ayk_rmsnorm_residual_grouped(_ptr(x), _ptr(y), _ptr(weight), ctypes.c_int(x.shape[0]),
                                             ctypes.c_int(x.shape[1]), ctypes.c_int(groups), ctypes.c_float(eps),
                                             ctypes.c_float(mult), _stream()))
    return x


def rmsnorm_residual_norm(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, mult: float,
                          next_weight: torch.Tensor, next_eps: float, out_dtype: torch.dtype, groups: int = 1) -> torch.Tensor:
    """x += mult * rmsnorm(y) * weight in place, and in the same kernel the next norm of the updated stream:
    returns rmsnorm(x) * next_weight in ``out_dtype`` (both norms in the same ``groups`` runs)."""
    lib = _ready()
    _f32(x, "x"); _f32(y, "y"); _f32(weight, "weight"); _f32(next_weight, "next_weight")
    if (x.shape != y.shape or weight.numel() != x.shape[1] or next_weight.numel() != x.shape[1] or groups < 1
            or x.shape[1] % groups):
        raise KernelError("rmsnorm_residual_norm: shapes do not fit")
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    _launch(lib.ayk_rmsnorm_residual_norm(_ptr(x), _ptr(out), _ptr(y), _ptr(weight), _ptr(next_weight), ctypes.c_int(x.shape[0]),
                                          ctypes.c_int(x.shape[1]), ctypes.c_int(groups), ctypes.c_float(eps),
                                          ctypes.c_float(mult), ctypes.c_float(next_eps), ctypes.c_int(_tag(out_dtype)), _stream()))
    return out


def layernorm_residual(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, eps: float,
                       following: tuple | None = None, out_dtype: torch.dtype | None = None) -> torch.Tensor | None:
    """x += layernorm(y) * weight + bias, in place on the float32 residual stream (mean, variance as the mean
    of the squared deviations, and the affine in 32-bit).  ``following`` = (weight, bias, eps): the same kernel
    also returns that layer norm of the updated stream in ``out_dtype``."""
    lib = _ready()
    _f32(x, "x"); _f32(y, "y"); _f32(weight, "weight")
    d = x.shape[1]
    if x.shape != y.shape or weight.numel() != d or (bias is not None and _f32(bias, "bias").numel() != d):
        raise KernelError("layernorm_residual: shapes do not fit")
    out, w2, b2, eps2 = None, None, None, 0.0
    if following is not None:
        w2, b2, eps2 = following
        if _f32(w2, "following weight").numel() != d or (b2 is not None and _f32(b2, "following bias").numel() != d):
            raise KernelError("layernorm_residual: the following norm does not fit the rows")
        out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    _launch(lib.ayk_layernorm_residual(_ptr(x), _ptr(out), _ptr(y), _ptr(weight), _ptr(bias), _ptr(w2), _ptr(b2),
                                       ctypes.c_int(x.shape[0]), ctypes.c_int(d), ctypes.c_float(eps), ctypes.c_float(eps2),
                                       ctypes.c_int(_tag(out_dtype) if out is not None else F32), _stream()))
    return out


def gated_act(z: torch.Tensor, n: int, activation: str, out_dtype: torch.dtype) -> torch.Tensor:
    """act(z[:, :n]) * z[:, n:2n]: the halves of a fused gate | up projection, the activation in 32-bit."""
    lib = _ready()
    if z.dim() != 2 or z.stride(1) != 1 or z.shape[1] < 2 * n:
        raise KernelError("gated_act: z must be rows of at least 2 n columns")
    out = torch.empty((z.shape[0], n), dtype=out_dtype, device=z.device)
    _launch(lib.ayk_gated_act(_ptr(out), _ptr(z), ctypes.c_longlong(z.stride(0)), ctypes.c_int(z.shape[0]), ctypes.c_int(n),
                              ctypes.c_int(ACTIVATIONS[activation]), ctypes.c_int(_tag(z.dtype)),
                              ctypes.c_int(_tag(out_dtype)), _stream()))
    return out


def add_(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """x += y, in place (contiguous float32 of one shape)."""
    lib = _ready()
    _f32(x, "x"); _f32(y, "y")
    if x.shape != y.shape:
        raise KernelError("add_: shapes differ")
    _launch(lib.ayk_add_rows(_ptr(x), _ptr(y), ctypes.c_longlong(x.numel()), _stream()))
    return x


def polynorm(z: torch.Tensor, coeff: torch.Tensor, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """a N(z) + b N(z^2) + c N(z^3) + e per row, N the division by the row's root mean square;
    ``coeff`` = (a, b, c, e) float32 on the device."""
    lib = _ready()
    if not z.is_contiguous() or z.dim() != 2:
        raise KernelError("polynorm: z must be contiguous rows")
    _f32(coeff, "coeff")
    out = torch.empty(z.shape, dtype=out_dtype, device=z.device)
    _launch(lib.ayk_polynorm(_ptr(out), _ptr(z), _ptr(coeff), ctypes.c_int(z.shape[0]), ctypes.c_int(z.shape[1]),
                             ctypes.c_float(eps), ctypes.c_int(_tag(z.dtype)), ctypes.c_int(_tag(out_dtype)), _stream()))
    return out


def rotary(x: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, gain: float, heads: int, head_stride: int,
           offset: int, dims: int, halves: bool = False) -> None:
    """Turns x[t, head * head_stride + offset + (0 .. dims)) in place: neighbouring pairs (2i, 2i+1),
    or with ``halves`` the pairs (i, i + dims/2), by the angle positions[t] * freq[i], cos and sin
    times ``gain``.  x: rows with unit column stride."""
    lib = _ready()
    if x.dim() != 2 or x.stride(1) != 1:
        raise KernelError("rotary: x must be rows with unit column stride")
    _f32(freq, "freq")
    if freq.numel() * 2 != dims or (heads - 1) * head_stride + offset + dims > x.shape[1]:
        raise KernelError("rotary: heads, offset and dims do not fit the rows")
    _launch(lib.ayk_rotary(_ptr(x), ctypes.c_longlong(x.stride(0)), _ptr(_i32(positions, "positions")), _ptr(freq),
                           ctypes.c_float(gain), ctypes.c_int(x.shape[0]), ctypes.c_int(heads), ctypes.c_int(head_stride),
                           ctypes.c_int(offset), ctypes.c_int(dims), ctypes.c_int(1 if halves else 0),
                           ctypes.c_int(_tag(x.dtype)), _stream()))


def latent_prepare(proj: torch.Tensor, latent_pages: torch.Tensor, rope_pages: torch.Tensor, norm_weight: torch.Tensor,
                   freq: torch.Tensor, gain: float, rot_dims: int, ctx, table: torch.Tensor, heads: int, dim: int,
                   rot: int, rank: int, eps: float, writes: bool) -> torch.Tensor:
    """From the float32 projection rows [q (heads x (dim + rot)) | down (rank + rot) | ...]: the normed
    latent and the rotated shared key part go into their pages (unless ``writes`` is False), the
    rotated query parts into the returned float32 query [T, heads, rank + rot] (columns rank ..);
    its first rank columns per head are left for the per-head product."""
    lib = _ready()
    _f32(proj, "proj"); _f32(norm_weight, "norm_weight"); _f32(freq, "freq")
    T = proj.shape[0]
    P = latent_pages.shape[1]
    if proj.shape[1] < heads * (dim + rot) + rank + rot or latent_pages.dtype != rope_pages.dtype:
        raise KernelError("latent_prepare: projection rows or pages do not fit")
    query = torch.empty((T, heads, rank + rot), dtype=torch.float32, device=proj.device)
    _launch(lib.ayk_latent_prepare(_ptr(latent_pages), _ptr(rope_pages), _ptr(query), _ptr(proj), ctypes.c_int(proj.stride(0)),
                                   _ptr(norm_weight), _ptr(freq), ctypes.c_float(gain), ctypes.c_int(rot_dims),
                                   _ptr(ctx.row_req), _ptr(ctx.positions), _ptr(_i32(table, "table")),
                                   ctypes.c_int(table.stride(0)), ctypes.c_int(P), ctypes.c_int(T), ctypes.c_int(heads),
                                   ctypes.c_int(dim), ctypes.c_int(rot), ctypes.c_int(rank), ctypes.c_float(eps),
                                   ctypes.c_int(1 if writes else 0), ctypes.c_int(_tag(latent_pages.dtype)), _stream()))
    return query


def head_matmul(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gate: torch.Tensor | None = None) -> torch.Tensor:
    """out[t, h, :] = w[h] @ a[t, h, :] (times sigmoid(gate[t, h]), or sigmoid(gate[t, h, :]) number by
    number): a [T, H, K] float32 view (any row and head stride, unit stride along K), w [H, N, K] contiguous,
    out [T, H, N] view, gate a [T, H] view or a [T, H * N] view."""
    lib = _ready()
    T, H, K = a.shape
    N = w.shape[1]
    if a.dtype != torch.float32 or a.stride(2) != 1 or w.shape != (H, N, K) or not w.is_contiguous():
        raise KernelError("head_matmul: a must be float32 [T, H, K], w [H, N, K]")
    if out.shape != (T, H, N) or out.stride(2) != 1:
        raise KernelError("head_matmul: out must be [T, H, N]")
    if gate is not None and (gate.dtype != torch.float32 or gate.shape not in ((T, H), (T, H * N)) or gate.stride(1) != 1):
        raise KernelError("head_matmul: gate must be float32 [T, H] or [T, H * N]")
    wide = gate is not None and gate.shape[1] != H
    common = (_ptr(out), ctypes.c_longlong(out.stride(0)), ctypes.c_int(out.stride(1)), _ptr(a),
              ctypes.c_longlong(a.stride(0)), ctypes.c_int(a.stride(1)), _ptr(w), _ptr(gate),
              ctypes.c_longlong(gate.stride(0) if gate is not None else 0), ctypes.c_int(N if wide else 1),
              ctypes.c_int(1 if wide else 0), ctypes.c_int(T), ctypes.c_int(H),
              ctypes.c_int(N), ctypes.c_int(K))
    # a handful of rows (a decode step): a warp per output column streams its weight row once
    if lib.ayk_head_matvec_takes(_ptr(a), ctypes.c_longlong(a.stride(0)), ctypes.c_int(a.stride(1)), _ptr(w), ctypes.c_int(T),
                                 ctypes.c_int(K)):
        _launch(lib.ayk_head_matvec(*common, ctypes.c_int(_tag(w.dtype)), ctypes.c_int(_tag(out.dtype)), _stream()))
    # bfloat16 weights: the tensor cores, the float32 operand in two bfloat16 parts; else the FP32 pipes
    elif w.dtype == torch.bfloat16 and lib.ayk_head_matmul_mma_takes(_ptr(a), ctypes.c_longlong(a.stride(0)),
                                                                   ctypes.c_int(a.stride(1)), ctypes.c_int(K)):
        _launch(lib.ayk_head_matmul_mma(*common, ctypes.c_int(_tag(out.dtype)), _stream()))
    else:
        _launch(lib.ayk_head_matmul(*common, ctypes.c_int(_tag(w.dtype)), ctypes.c_int(_tag(out.dtype)), _stream()))
    return out


LATENT_PARTS = 64        # at most this many partitions of the context when every request brings one row


def latent_attention(query: torch.Tensor, latent_pages: torch.Tensor, rope_pages: torch.Tensor, table: torch.Tensor,
                     ctx, scale: float, tensor_cores: bool | None = None) -> torch.Tensor:
    """Causal attention of the step's rows over cached (latent, rotated key part) pairs shared by
    all heads: query [T, H, rank + rot] float32; returns sum_j p_j latent_j as float32 [T, H, rank].
    bfloat16 pages whose rows are whole 16-byte pieces go through the tensor-core kernel (a decode
    step's context cut into partitions and merged); 32-bit pages and other sizes through the
    kernel on the FP32 pipes."""
    lib = _ready()
    T, H, Dk = query.shape
    rank, rot = latent_pages.shape[-1], rope_pages.shape[-1]
    if query.dtype != torch.float32 or not query.is_contiguous() or Dk != rank + rot:
        raise KernelError("latent_attention: query must be contiguous float32 [T, H, rank + rot]")
    out = torch.empty((T, H, rank), dtype=torch.float32, device=query.device)
    takes = latent_pages.dtype == torch.bfloat16 and bool(lib.ayk_latent_attention_mma_takes(ctypes.c_int(rank), ctypes.c_int(rot)))
    if tensor_cores is None:
        tensor_cores = takes
    elif tensor_cores and not takes:
        raise KernelError(f"latent_attention: the tensor-core kernel does not take {latent_pages.dtype} pages of {rank} + {rot}")
    if tensor_cores:
        parts, part_keys, partial = 1, 0, None
        if ctx.max_q_len == 1:
            part_keys = max(32, -(-(-(-ctx.cache.max_len // LATENT_PARTS)) // 32) * 32)
            parts = -(-ctx.cache.max_len // part_keys)
            if parts > 1:
                partial = torch.empty((T * H * parts * (rank + 2),), dtype=torch.float32, device=query.device)
        launched = ctypes.c_int(0)
        code = lib.ayk_latent_attention_mma(_ptr(out), _ptr(partial), _ptr(query), _ptr(latent_pages), _ptr(rope_pages),
                                            _ptr(_i32(table, "table")), ctypes.c_int(table.stride(0)), _ptr(ctx.req_q_start),
                                            _ptr(ctx.req_pos0), ctypes.c_int(ctx.num_requests), ctypes.c_int(T),
                                            ctypes.c_int(ctx.max_q_len), ctypes.c_int(H), ctypes.c_int(rank), ctypes.c_int(rot),
                                            ctypes.c_int(latent_pages.shape[1]), ctypes.c_float(scale), ctypes.c_int(parts),
                                            ctypes.c_int(part_keys), ctypes.byref(launched), _stream())
        global launches
        launches += launched.value
        _check(code)
        return out
    _launch(lib.ayk_latent_attention(_ptr(out), _ptr(query), _ptr(latent_pages), _ptr(rope_pages), _ptr(_i32(table, "table")),
                                     ctypes.c_int(table.stride(0)), _ptr(ctx.req_q_start), _ptr(ctx.req_pos0),
                                     ctypes.c_int(ctx.num_requests), ctypes.c_int(T), ctypes.c_int(H), ctypes.c_int(rank),
                                     ctypes.c_int(rot), ctypes.c_int(latent_pages.shape[1]), ctypes.c_float(scale),
                                     ctypes.c_int(_tag(latent_pages.dtype)), _stream()))
    return out


def hgrn2(proj: torch.Tensor, state: torch.Tensor, f_bias: torch.Tensor, lower: torch.Tensor, ctx, heads: int, dim: int,
          vdim: int, chunked: bool | None = None) -> torch.Tensor:
    """The HGRN2 recurrence over the step's rows, request by request, from and into ``state``
    [slots, heads, dim, vdim] float32.  proj: float32 rows [z_q | z_f | v]; returns o [T, heads * vdim] float32.
    ``chunked``: the kernel that takes 16 tokens at a time (default: whenever a request brings more than one row)."""
    lib = _ready()
    _f32(proj, "proj"); _f32(state, "state"); _f32(f_bias, "f_bias"); _f32(lower, "lower")
    T = proj.shape[0]
    if proj.shape[1] < heads * (2 * dim + vdim) or state.shape[1:] != (heads, dim, vdim):
        raise KernelError("hgrn2: projection rows or state do not fit")
    out = torch.empty((T, heads * vdim), dtype=torch.float32, device=proj.device)
    if chunked is None:
        chunked = ctx.max_q_len > 1
    scratch = None
    if chunked:
        lib.ayk_hgrn2_scratch_floats.restype = ctypes.c_longlong
        floats = int(lib.ayk_hgrn2_scratch_floats(ctypes.c_int(T), ctypes.c_int(ctx.num_requests), ctypes.c_int(heads), ctypes.c_int(dim)))
        scratch = torch.empty((floats,), dtype=torch.float32, device=proj.device)
    _launch(lib.ayk_hgrn2(_ptr(out), _ptr(state), _ptr(proj), ctypes.c_int(proj.stride(0)), _ptr(f_bias), _ptr(lower),
                          _ptr(ctx.req_q_start), _ptr(ctx.req_slot), ctypes.c_int(ctx.num_requests), ctypes.c_int(T),
                          ctypes.c_int(heads), ctypes.c_int(dim), ctypes.c_int(vdim), _ptr(scratch), _stream()))
    if chunked:
        global launches
        launches += 1
    return out


def mlstm_head_floats(dim: int, vdim: int) -> int:
    """Floats that one head of an mLSTM keeps per request: the matrix memory, its normalizer, the running maximum."""
    return dim * vdim + dim + 4


def mlstm(proj: torch.Tensor, state: torch.Tensor, norm_weight: torch.Tensor, ctx, heads: int, dim: int, vdim: int,
          cap: float, eps: float, out_dtype: torch.dtype, chunked: bool | None = None, slice_cols: int = 0) -> torch.Tensor:
    """The mLSTM recurrence over the step's rows, request by request, from and into ``state`` [slots, heads,
    dim * vdim + dim + 4] float32, with the head's norm, channel weight and output gate applied.  proj: float32
    rows [q | k | v | z_i (heads) | z_f (heads) | gate (heads * vdim)]; returns [T, heads * vdim] in
    ``out_dtype``.  ``chunked``: the kernel that takes 16 tokens at a time (default: whenever a request brings
    more than one row, or the values are wider than the token-by-token kernel's 256 numbers, and the head size
    fits it); ``slice_cols``: value columns per block of that kernel, 16 or 32 (0: 32, or 16 where blocks of 32
    would leave most SMs idle)."""
    lib = _ready()
    lib.ayk_mlstm_slice_cols(ctypes.c_int(slice_cols))
    _f32(proj, "proj"); _f32(state, "state"); _f32(norm_weight, "norm_weight")
    T = proj.shape[0]
    if (proj.shape[1] < 2 * heads * dim + 2 * heads * vdim + 2 * heads or state.shape[1:] != (heads, mlstm_head_floats(dim, vdim))
            or norm_weight.numel() != heads * vdim):
        raise KernelError("mlstm: projection rows, state or norm weight do not fit")
    out = torch.empty((T, heads * vdim), dtype=out_dtype, device=proj.device)
    takes = bool(lib.ayk_mlstm_chunk_takes(ctypes.c_int(dim)))
    if chunked is None:
        chunked = (ctx.max_q_len > 1 or vdim > 256) and takes
    elif chunked and not takes:
        raise KernelError(f"mlstm: the chunked kernel does not take heads of {dim} numbers")
    if not chunked and vdim > 256:
        raise KernelError(f"mlstm: heads of {dim} x {vdim} fit neither kernel (values over 256 need keys under about 750)")
    scratch = None
    if chunked:
        lib.ayk_mlstm_scratch_floats.restype = ctypes.c_longlong
        floats = int(lib.ayk_mlstm_scratch_floats(ctypes.c_int(T), ctypes.c_int(ctx.num_requests), ctypes.c_int(heads),
                                                  ctypes.c_int(dim), ctypes.c_int(vdim)))
        scratch = torch.empty((floats,), dtype=torch.float32, device=proj.device)
    _launch(lib.ayk_mlstm(_ptr(out), _ptr(state), _ptr(proj), ctypes.c_longlong(proj.stride(0)), _ptr(norm_weight),
                          _ptr(ctx.row_req), _ptr(ctx.req_q_start), _ptr(ctx.req_slot), ctypes.c_int(ctx.num_requests),
                          ctypes.c_int(T), ctypes.c_int(heads), ctypes.c_int(dim), ctypes.c_int(vdim), ctypes.c_float(cap),
                          ctypes.c_float(eps), _ptr(scratch), ctypes.c_int(_tag(out_dtype)), _stream()))
    if chunked:
        global launches
        launches += 1
    return out


# ------------------- token shift, channel recurrences, gated attention, experts --

def token_shift(x: torch.Tensor, mu: torch.Tensor | None, state: torch.Tensor | None, ctx, out_dtype: torch.dtype) -> torch.Tensor:
    """x + (previous row - x) * mu per channel; the row before a request's first row is its ``state``
    [slots, d] float32, which then takes the request's last row.  ``mu`` None: the rows of x in
    ``out_dtype`` and nothing else."""
    lib = _ready()
    _f32(x, "x")
    T, d = x.shape
    out = torch.empty((T, d), dtype=out_dtype, device=x.device)
    if mu is None:
        _launch(lib.ayk_token_shift(_ptr(out), _ptr(x), _ptr(None), _ptr(None), _ptr(None), _ptr(None), _ptr(None),
                                    ctypes.c_int(T), ctypes.c_int(d), ctypes.c_int(_tag(out_dtype)), _stream()))
        return out
    _f32(mu, "mu"); _f32(state, "state")
    if mu.numel() != d or state.shape[1:] != (d,):
        raise KernelError("token_shift: mu [d] and state [slots, d] must fit the rows")
    _launch(lib.ayk_token_shift(_ptr(out), _ptr(x), _ptr(mu), _ptr(state), _ptr(ctx.row_req), _ptr(ctx.req_q_start),
                                _ptr(ctx.req_slot), ctypes.c_int(T), ctypes.c_int(d), ctypes.c_int(_tag(out_dtype)), _stream()))
    return out


def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor | None, state: torch.Tensor, ctx) -> torch.Tensor:
    """bias + causal convolution over time on every channel of the float32 rows x [T, C] (a column
    slice of a wider matrix is fine): ``taps`` [n, C] float32, tap-major, the last one multiplies the
    current row.  ``state`` [slots, n, C] float32: rows 1 .. n - 1 of a slot hold the request's last
    n - 1 inputs, oldest first (row 0 belongs to the caller), and are brought up to date."""
    lib = _ready()
    T, C = x.shape
    n = taps.shape[0]
    _f32(taps, "taps"); _f32(state, "state")
    if x.dtype != torch.float32 or x.stride(1) != 1 or taps.shape[1] != C or state.shape[1:] != (n, C):
        raise KernelError("causal_conv: x float32 [T, C], taps [n, C] and state [slots, n, C] must fit")
    if bias is not None:
        _f32(bias, "bias")
    out = torch.empty((T, C), dtype=torch.float32, device=x.device)
    inputs = state[:, 1:] if n > 1 else state                  # the pointer only: rows lie C apart, slots n * C
    _launch(lib.ayk_causal_conv(_ptr(out), _ptr(x), ctypes.c_longlong(x.stride(0)), _ptr(taps), _ptr(bias),
                                ctypes.c_void_p(inputs.data_ptr()), ctypes.c_longlong(state.stride(0)), _ptr(ctx.row_req),
                                _ptr(ctx.req_q_start), _ptr(ctx.req_slot), ctypes.c_int(T), ctypes.c_int(ctx.num_requests),
                                ctypes.c_int(C), ctypes.c_int(n), _stream()))
    if n > 1:
        global launches
        launches += 1
    return out


def mingru_scan(proj: torch.Tensor, state: torch.Tensor, ctx, width: int, out_dtype: torch.dtype) -> torch.Tensor:
    """minGRU over the step's rows, request by request, from and into ``state`` [slots, width] float32.
    proj: float32 rows [z | u | g] before their sigmoid, candidate and SiLU.  Returns S * silu(g) [T, width]."""
    lib = _ready()
    _f32(proj, "proj"); _f32(state, "state")
    T = proj.shape[0]
    if proj.shape[1] < 3 * width or state.shape[1:] != (width,):
        raise KernelError("mingru_scan: projection rows or state do not fit")
    out = torch.empty((T, width), dtype=out_dtype, device=proj.device)
    _launch(lib.ayk_mingru_scan(_ptr(out), _ptr(state), ctypes.c_longlong(state.stride(0)), _ptr(proj),
                                ctypes.c_longlong(proj.stride(0)), _ptr(ctx.req_q_start), _ptr(ctx.req_slot),
                                ctypes.c_int(ctx.num_requests), ctypes.c_int(T), ctypes.c_int(width),
                                ctypes.c_int(ctx.max_q_len), ctypes.c_int(_tag(out_dtype)), _stream()))
    return out


def rglru_scan(proj: torch.Tensor, u: torch.Tensor, gates: torch.Tensor, gate_bias: torch.Tensor, lam: torch.Tensor,
               state: torch.Tensor, ctx, width: int, blocks: int, decay: float, out_dtype: torch.dtype) -> torch.Tensor:
    """The real-gated linear recurrent unit over the step's rows: a = exp(-decay sigmoid(r) softplus(lam)),
    S = a S + sqrt(1 - a^2) sigmoid(i) u, from and into row 0 of ``state`` [slots, n, width] float32.
    proj: float32 rows whose first ``width`` columns are the other branch before its GELU; u [T, width];
    gates [T, blocks, r | i] before their biases ``gate_bias`` [blocks, r | i].  Returns S * gelu(y)."""
    lib = _ready()
    _f32(proj, "proj"); _f32(u, "u"); _f32(gates, "gates"); _f32(gate_bias, "gate_bias"); _f32(lam, "lam"); _f32(state, "state")
    T = proj.shape[0]
    if (proj.shape[1] < width or u.shape != (T, width) or gates.numel() != T * 2 * width or gate_bias.numel() != 2 * width
            or lam.numel() != width or state.shape[2] != width):
        raise KernelError("rglru_scan: rows, gates or state do not fit")
    out = torch.empty((T, width), dtype=out_dtype, device=proj.device)
    _launch(lib.ayk_rglru_scan(_ptr(out), _ptr(state), ctypes.c_longlong(state.stride(0)), _ptr(proj),
                               ctypes.c_longlong(proj.stride(0)), _ptr(u), _ptr(gates), _ptr(gate_bias), _ptr(lam),
                               ctypes.c_float(decay), _ptr(ctx.req_q_start), _ptr(ctx.req_slot), ctypes.c_int(ctx.num_requests),
                               ctypes.c_int(T), ctypes.c_int(width), ctypes.c_int(blocks), ctypes.c_int(ctx.max_q_len),
                               ctypes.c_int(_tag(out_dtype)), _stream()))
    return out


def scale_(x: torch.Tensor, factor: float) -> torch.Tensor:
    """x *= factor, in place (contiguous float32)."""
    lib = _ready()
    _f32(x, "x")
    _launch(lib.ayk_scale(_ptr(x), ctypes.c_longlong(x.numel()), ctypes.c_float(factor), _stream()))
    return x


def qk_norm_rotary(proj: torch.Tensor, kpages: torch.Tensor, vpages: torch.Tensor, q_norm: torch.Tensor, k_norm: torch.Tensor,
                   freq: torch.Tensor, rot_dims: int, ctx, table: torch.Tensor, heads: int, eps: float, writes: bool,
                   out_dtype: torch.dtype) -> torch.Tensor:
    """From float32 projection rows [q | k | v]: the whole query row and the whole key row RMS-normed
    with one weight per element, the first ``rot_dims`` dimensions of every head rotated by the position
    (dimension i with i + rot_dims/2); keys and values go into their pages (unless ``writes`` is False),
    the queries are returned [T, heads * dim] in ``out_dtype``."""
    lib = _ready()
    _f32(proj, "proj"); _f32(q_norm, "q_norm"); _f32(k_norm, "k_norm"); _f32(freq, "freq")
    T = proj.shape[0]
    pages, P, G, D = kpages.shape
    Dv = vpages.shape[3]
    if (proj.shape[1] < heads * D + G * D + G * Dv or q_norm.numel() != heads * D or k_norm.numel() != G * D
            or kpages.dtype != out_dtype or vpages.dtype != out_dtype or not kpages.is_contiguous() or not vpages.is_contiguous()):
        raise KernelError("qk_norm_rotary: projection rows, weights or pages do not fit")
    q = torch.empty((T, heads * D), dtype=out_dtype, device=proj.device)
    _launch(lib.ayk_qk_norm_rotary(_ptr(q), _ptr(kpages), _ptr(vpages), _ptr(proj), ctypes.c_longlong(proj.stride(0)),
                                   _ptr(q_norm), _ptr(k_norm), _ptr(freq), ctypes.c_int(rot_dims), _ptr(ctx.row_req),
                                   _ptr(ctx.positions), _ptr(_i32(table, "table")), ctypes.c_int(table.stride(0)),
                                   ctypes.c_int(P), ctypes.c_int(T), ctypes.c_int(heads), ctypes.c_int(G), ctypes.c_int(D),
                                   ctypes.c_int(Dv), ctypes.c_float(eps), ctypes.c_int(1 if writes else 0),
                                   ctypes.c_int(_tag(out_dtype)), _stream()))
    return q


GATED_PART = 256          # keys per partition of the context when every request brings one row


def sigmoid_attention(q: torch.Tensor, kpages: torch.Tensor, vpages: torch.Tensor, table: torch.Tensor, ctx, heads: int,
                      scale: float, softcap: float, head_bias: torch.Tensor | None, tensor_cores: bool = True) -> torch.Tensor:
    """Causal attention without a softmax over the paged cache: the weight of a visible key is
    sigmoid(cap tanh(q . k scale / cap) + head_bias[head]) (cap 0: no cap), the output the weighted sum of
    the values.  q [T, heads * dim] of the pages' dtype; returns [T, heads * vdim].  When every request
    brings one row the context is cut into partitions whose partial sums are added by a second kernel.
    bfloat16 pages with head sizes of 16, 32, 64 or 128 go through the tensor-core kernel (``tensor_cores``
    False: through the kernel on the FP32 pipes like everything else)."""
    lib = _ready()
    lib.ayk_gated_attention_tensor_cores(ctypes.c_int(1 if tensor_cores else 0))
    pages, P, G, D = kpages.shape
    Dv = vpages.shape[3]
    T = q.shape[0]
    if q.shape[1] != heads * D or not q.is_contiguous() or q.dtype != kpages.dtype or vpages.dtype != kpages.dtype:
        raise KernelError("sigmoid_attention: q must be a contiguous [T, heads * dim] matrix of the pages' dtype")
    if head_bias is not None:
        _f32(head_bias, "head_bias")
    out = torch.empty((T, heads * Dv), dtype=q.dtype, device=q.device)
    parts, partial = 1, None
    if ctx.max_q_len == 1:
        parts = max(1, -(-ctx.cache.max_len // GATED_PART))
        if parts > 1:
            partial = _decode_buffer(q.device, parts * T * heads * Dv)
    launched = ctypes.c_int(0)
    code = lib.ayk_gated_attention(_ptr(out), _ptr(partial), _ptr(q), _ptr(kpages), _ptr(vpages), _ptr(_i32(table, "table")),
                                   ctypes.c_int(table.stride(0)), _ptr(ctx.req_q_start), _ptr(ctx.req_pos0), _ptr(ctx.row_req),
                                   _ptr(ctx.positions), ctypes.c_int(ctx.num_requests), ctypes.c_int(T), ctypes.c_int(heads),
                                   ctypes.c_int(G), ctypes.c_int(D), ctypes.c_int(Dv), ctypes.c_int(P), ctypes.c_float(scale),
                                   ctypes.c_float(softcap), _ptr(head_bias), ctypes.c_int(parts), ctypes.c_int(GATED_PART),
                                   ctypes.c_int(_tag(q.dtype)), ctypes.byref(launched), _stream())
    global launches
    launches += launched.value
    _check(code)
    return out


def grouped_part(max_len: int) -> int:
    """Keys per partition of the context when every request brings one row: 64, or the power of two that
    leaves at most 64 partitions of the longest context the cache holds."""
    part = 64
    while part * 64 < max_len:
        part *= 2
    return part


def head_norm_prepare(proj: torch.Tensor, kpages: torch.Tensor, vpages: torch.Tensor, q_norm: torch.Tensor, k_norm: torch.Tensor,
                      ctx, table: torch.Tensor, heads: int, kv_heads: int, dim: int, maps: int, v_col0: int, eps: float,
                      writes: bool, out_dtype: torch.dtype, mix: torch.Tensor | None = None) -> torch.Tensor:
    """From float32 projection rows [q | k | ...]: every query head (``heads * maps`` of them, a head's maps
    side by side) and every key head (``kv_heads * maps``) RMS-normed over its ``dim`` numbers with one weight
    shared by all heads; the normed keys go into ``kpages``, columns ``v_col0 ...`` of the row (as wide as a
    token's values) into ``vpages`` (unless ``writes`` is False).  Returns the queries [T, heads * maps * dim],
    the heads that share a key head side by side ([key head][map][head of the group]).  ``mix`` [heads, heads]
    float32 (one map only): the queries are returned mixed, [T, heads, kv_heads * dim] with
    q~[h, c] = sum over the heads g of key head c of mix[h, g] q[g], so that q~[h] times a token's key heads
    side by side is the mix of the heads' scores."""
    lib = _ready()
    _f32(proj, "proj"); _f32(q_norm, "q_norm"); _f32(k_norm, "k_norm")
    T = proj.shape[0]
    v_width = vpages.shape[2] * vpages.shape[3]
    if (kpages.shape[2] * kpages.shape[3] != kv_heads * maps * dim or q_norm.numel() != dim or k_norm.numel() != dim
            or proj.shape[1] < max((heads + kv_heads) * maps * dim, v_col0 + v_width) or kpages.dtype != out_dtype
            or vpages.dtype != out_dtype or not kpages.is_contiguous() or not vpages.is_contiguous()):
        raise KernelError("head_norm_prepare: projection rows, weights or pages do not fit")
    if mix is not None:
        _f32(mix, "mix")
        if maps != 1 or mix.shape != (heads, heads):
            raise KernelError("head_norm_prepare: the mix is [heads, heads] and takes one map")
    width = heads * kv_heads * dim if mix is not None else heads * maps * dim
    q = torch.empty((T, width), dtype=out_dtype, device=proj.device)
    _launch(lib.ayk_head_norm_prepare(_ptr(q), _ptr(kpages), _ptr(vpages), _ptr(proj), ctypes.c_longlong(proj.stride(0)),
                                      _ptr(q_norm), _ptr(k_norm), _ptr(mix), _ptr(ctx.row_req), _ptr(ctx.positions),
                                      _ptr(_i32(table, "table")), ctypes.c_int(table.stride(0)), ctypes.c_int(kpages.shape[1]),
                                      ctypes.c_int(T), ctypes.c_int(heads), ctypes.c_int(kv_heads), ctypes.c_int(dim),
                                      ctypes.c_int(maps), ctypes.c_int(v_col0), ctypes.c_int(v_width), ctypes.c_float(eps),
                                      ctypes.c_int(1 if writes else 0), ctypes.c_int(_tag(out_dtype)), _stream()))
    return q


def grouped_attention(q: torch.Tensor, kpages: torch.Tensor, vpages: torch.Tensor, table: torch.Tensor, ctx, heads: int,
                      key_heads: int, key_dim: int, scale: float, slopes: torch.Tensor | None = None,
                      window: int | None = None, keep_first: int = 0, gate: torch.Tensor | None = None,
                      maps: int = 1, lam: float = 0.0, post_scale: float = 1.0, eps: float = 0.0,
                      tensor_cores: bool = True, chunk: int | None = None) -> torch.Tensor:
    """Softmax attention of the step's rows over the paged cache with keys and values grouped separately:
    ``heads`` query heads of ``key_dim`` read ``key_heads`` key heads (the pages' rows taken as
    [key_heads, key_dim]) and the value heads of ``vpages``; score (q . k) scale - slopes[h] (i - j); key j
    visible to query i when j <= i and (i - j < window or j < keep_first) and, with ``chunk``, only when
    floor(i / chunk) = floor(j / chunk).  ``gate`` (float32 rows): the output is multiplied by
    sigmoid(gate).  ``maps`` == 2: the query heads are [group][map][head of the group] and the result is per
    head o1 - lam o2, divided by its root mean square (``eps`` under the root), times ``post_scale``; a
    gate then has one number per output head.  When every request brings one row the context is cut into parts that a
    second kernel merges.  Returns [T, heads / maps * vdim] of the pages' dtype."""
    lib = _ready()
    lib.ayk_grouped_attention_tensor_cores(ctypes.c_int(1 if tensor_cores else 0))
    pages, P, VH, DV = vpages.shape
    T = q.shape[0]
    if (q.shape[1] != heads * key_dim or not q.is_contiguous() or q.dtype != kpages.dtype or vpages.dtype != kpages.dtype
            or kpages.shape[2] * kpages.shape[3] != key_heads * key_dim or heads % maps):
        raise KernelError("grouped_attention: q must be a contiguous [T, heads * key_dim] matrix of the pages' dtype")
    if slopes is not None and (_f32(slopes, "slopes").numel() != heads):
        raise KernelError("grouped_attention: one slope per query head")
    out_heads = heads // maps
    hpg = heads // max(key_heads, VH)
    if gate is not None and (gate.dtype != torch.float32 or gate.stride(1) != 1 or
                             gate.shape[1] < (heads * DV if maps == 1 else out_heads)):
        raise KernelError("grouped_attention: the gate is float32 rows as wide as the output (one number per head with two maps)")
    out = torch.empty((T, out_heads * DV), dtype=q.dtype, device=q.device)
    part_keys = grouped_part(ctx.cache.max_len)
    parts = max(1, -(-ctx.cache.max_len // part_keys)) if ctx.max_q_len == 1 else 1
    two_steps = parts > 1 or maps > 1
    po = pml = None
    if two_steps:
        buf = _decode_buffer(q.device, parts * T * heads * (DV + 2))
        po, pml = buf[:parts * T * heads * DV], buf[parts * T * heads * DV:]
    gate_stride = gate.stride(0) if gate is not None else 0
    _launch(lib.ayk_grouped_attention(_ptr(None if two_steps else out), _ptr(po), _ptr(pml), _ptr(q), _ptr(kpages), _ptr(vpages),
                                      _ptr(_i32(table, "table")), ctypes.c_int(table.stride(0)), _ptr(ctx.req_q_start),
                                      _ptr(ctx.req_pos0), ctypes.c_int(ctx.num_requests), ctypes.c_int(T), ctypes.c_int(heads),
                                      ctypes.c_int(key_heads), ctypes.c_int(VH), ctypes.c_int(key_dim), ctypes.c_int(DV),
                                      ctypes.c_int(P), ctypes.c_float(scale), _ptr(slopes), ctypes.c_int(window or 0),
                                      ctypes.c_int(keep_first), ctypes.c_int(chunk or 0), _ptr(None if two_steps else gate),
                                      ctypes.c_longlong(gate_stride),
                                      ctypes.c_int(parts), ctypes.c_int(part_keys), ctypes.c_int(_tag(q.dtype)), _stream()))
    if two_steps:
        _launch(lib.ayk_grouped_finish(_ptr(out), _ptr(po), _ptr(pml), _ptr(ctx.positions), ctypes.c_int(T), ctypes.c_int(heads),
                                       ctypes.c_int(DV), ctypes.c_int(parts), ctypes.c_int(part_keys), ctypes.c_int(maps),
                                       ctypes.c_int(hpg if maps > 1 else 1), _ptr(gate), ctypes.c_longlong(gate_stride),
                                       ctypes.c_float(lam), ctypes.c_float(post_scale), ctypes.c_float(eps),
                                       ctypes.c_int(_tag(q.dtype)), _stream()))
    return out


class MoeRoute:
    """A step's routing on the device: ``ids`` and ``weights`` [T, top]; ``sorted`` [T * top], the
    (token, choice) pairs laid out expert by expert; ``tiles``: the number of row tiles and for each its
    expert, first sorted row and rows."""

    def __init__(self, ids, weights, sorted_pairs, tiles, max_tiles, top):
        self.ids, self.weights, self.sorted, self.tiles, self.max_tiles, self.top = ids, weights, sorted_pairs, tiles, max_tiles, top


def moe_route(logits: torch.Tensor, experts: int, top: int, scored: dict | None = None) -> MoeRoute:
    """The ``top`` largest of each row's first ``experts`` float32 logits, weighted by the softmax over
    the chosen ones, and the plan of the grouped products.  ``scored`` = {correction, groups, keep, factor}:
    routing by sigmoid scores s instead; experts are ranked by s + correction (float32 [experts] or None) among
    the experts of the ``keep`` best of ``groups`` equal runs of consecutive experts (a run's score: the sum of its two
    largest ranking scores), the weights are the chosen s over their sum, times ``factor``."""
    lib = _ready()
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or logits.shape[1] < experts:
        raise KernelError("moe_route: logits must be float32 rows of at least ``experts`` columns")
    T = logits.shape[0]
    rows = int(lib.ayk_moe_tile_rows())
    max_tiles = (T * top) // rows + experts
    ids = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    weights = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    sorted_pairs = torch.empty((T * top,), dtype=torch.int32, device=logits.device)
    tiles = torch.empty((1 + 3 * max_tiles,), dtype=torch.int32, device=logits.device)
    if scored is not None:
        correction = scored.get("correction")
        if correction is not None and _f32(correction, "correction").numel() != experts:
            raise KernelError("moe_route: one correction per expert")
        _launch(lib.ayk_moe_route_scored(_ptr(ids), _ptr(weights), _ptr(sorted_pairs), _ptr(tiles), _ptr(logits),
                                         ctypes.c_longlong(logits.stride(0)), _ptr(correction), ctypes.c_int(T),
                                         ctypes.c_int(experts), ctypes.c_int(top), ctypes.c_int(int(scored.get("groups", 1))),
                                         ctypes.c_int(int(scored.get("keep", 1))), ctypes.c_float(float(scored.get("factor", 1.0))),
                                         _stream()))
    else:
        _launch(lib.ayk_moe_route(_ptr(ids), _ptr(weights), _ptr(sorted_pairs), _ptr(tiles), _ptr(logits),
                                  ctypes.c_longlong(logits.stride(0)), ctypes.c_int(T), ctypes.c_int(experts), ctypes.c_int(top), _stream()))
    global launches
    launches += 1
    return MoeRoute(ids, weights, sorted_pairs, tiles, max_tiles, top)


def _glu(glu: tuple | None) -> tuple[float, float, float]:
    """(limit, slope, plus) of an experts' activation min(g, limit) sigmoid(slope g) (clamp(u) + plus); two
    numbers mean plus = 1."""
    if glu is None:
        return 0.0, 0.0, 0.0
    return (float(glu[0]), float(glu[1]), float(glu[2]) if len(glu) > 2 else 1.0)


def moe_gemm(a: torch.Tensor, w: torch.Tensor, route: MoeRoute, glu: tuple | None, out_dtype: torch.dtype) -> torch.Tensor:
    """Grouped product over the sorted pairs.  ``glu`` = (limit, slope): a holds the tokens' rows
    [T, K], w [experts, 2 N, K] gate over up, and the result is the experts' activation
    min(g, limit) sigmoid(slope g) (clamp(u) + 1) per sorted pair, [T * top, N] in ``out_dtype``.  ``glu`` None:
    a holds rows per sorted pair, w [experts, N, K], and the float32 result [T * top, N] lies pair by pair
    (token-major).  bfloat16 operands run on the tensor cores, float32 on the FP32 pipes."""
    lib = _ready()
    E, n_w, K = w.shape
    if a.dtype != w.dtype or a.shape[1] != K or a.stride(1) != 1 or not w.is_contiguous():
        raise KernelError("moe_gemm: operands do not fit")
    pairs = route.sorted.numel()
    N = n_w // 2 if glu is not None else n_w
    out = torch.empty((pairs, N), dtype=out_dtype, device=a.device)
    limit, slope, plus = _glu(glu)
    _launch(lib.ayk_moe_gemm(_ptr(out), _ptr(a), ctypes.c_longlong(a.stride(0)), _ptr(w), _ptr(route.sorted), _ptr(route.tiles),
                             ctypes.c_int(route.max_tiles), ctypes.c_int(route.top), ctypes.c_int(1 if glu is not None else 0),
                             ctypes.c_int(0 if glu is not None else 1), ctypes.c_int(N), ctypes.c_int(n_w), ctypes.c_int(K),
                             ctypes.c_int(1 if glu is not None else 0), ctypes.c_float(limit), ctypes.c_float(slope),
                             ctypes.c_float(plus), ctypes.c_int(_tag(a.dtype)), ctypes.c_int(_tag(out_dtype)), _stream()))
    return out


def moe_gemv_takes(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the pair-by-pair product takes these operands (bfloat16, rows in whole 16-byte pieces)."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and bool(_ready().ayk_moe_gemv_takes(ctypes.c_int(w.shape[2]), ctypes.c_longlong(a.stride(0)))))


def moe_gemv(a: torch.Tensor, w: torch.Tensor, route: MoeRoute, glu: tuple | None) -> torch.Tensor:
    """The experts' product for a handful of pairs, each pair streaming its expert's matrix on its own: no
    sorting, rows lie pair by pair (token-major).  ``glu`` = (limit, slope): a [T, K] tokens' rows, w
    [experts, 2 N, K], bfloat16 activations [T * top, N]; None: a [T * top, K], w [experts, N, K], float32 out."""
    lib = _ready()
    E, n_w, K = w.shape
    pairs = route.ids.numel()
    N = n_w // 2 if glu is not None else n_w
    if a.shape[1] != K or a.stride(1) != 1 or not w.is_contiguous() or not moe_gemv_takes(a, w):
        raise KernelError("moe_gemv: operands do not fit")
    out = torch.empty((pairs, N), dtype=torch.bfloat16 if glu is not None else torch.float32, device=a.device)
    limit, slope, plus = _glu(glu)
    _launch(lib.ayk_moe_gemv(_ptr(out), _ptr(a), ctypes.c_longlong(a.stride(0)), _ptr(w), _ptr(route.ids), ctypes.c_int(pairs),
                             ctypes.c_int(route.top), ctypes.c_int(N), ctypes.c_int(n_w), ctypes.c_int(K),
                             ctypes.c_int(1 if glu is not None else 0), ctypes.c_float(limit), ctypes.c_float(slope), ctypes.c_float(plus), _stream()))
    return out


def glu_limited(x: torch.Tensor, n: int, limit: float, slope: float, out_dtype: torch.dtype, plus: float = 1.0) -> torch.Tensor:
    """min(g, limit) sigmoid(slope g) (clamp(u, -limit, limit) + plus) with g = x[:, :n] and u = x[:, n:2n]
    of float32 or bfloat16 rows; the arithmetic is 32-bit.  An infinite limit clamps nothing."""
    lib = _ready()
    if x.stride(1) != 1 or x.shape[1] < 2 * n:
        raise KernelError("glu_limited: rows of at least 2 n columns")
    out = torch.empty((x.shape[0], n), dtype=out_dtype, device=x.device)
    _launch(lib.ayk_glu_limited(_ptr(out), _ptr(x), ctypes.c_longlong(x.stride(0)), ctypes.c_int(x.shape[0]), ctypes.c_int(n),
                                ctypes.c_float(limit), ctypes.c_float(slope), ctypes.c_float(plus), ctypes.c_int(_tag(x.dtype)),
                                ctypes.c_int(_tag(out_dtype)), _stream()))
    return out


MOE_TENSOR_PAIRS = 64         # (token, choice) pairs from which the experts' products run on tcgen05


def moe_experts_tc(h: torch.Tensor, in_weight: torch.Tensor, down_weight: torch.Tensor, route: MoeRoute, limit: float,
                   slope: float, plus: float = 1.0) -> tuple[torch.Tensor, torch.Tensor]:
    """The experts of a step on tcgen05 (bfloat16): the pairs' rows are gathered expert by expert, every expert's
    starting at a multiple of 128 rows, and the two products run as grouped forms of the many-row kernel, each
    128-row tile against the matrix of its expert.  in_weight [experts, 2 inner, width] gate over up,
    down_weight [experts, width, inner].  Returns (float32 rows [padded, width], row of every pair)."""
    lib = _ready()
    E, n1, d = in_weight.shape
    inner = n1 // 2
    T = h.shape[0]
    pairs = T * route.top
    pad = int(lib.ayk_moe_pad_rows())
    max_tiles = pairs // pad + E
    dev_ = h.device
    row_of_pair = torch.empty((pairs,), dtype=torch.int32, device=dev_)
    w_rows = torch.empty((2, max_tiles), dtype=torch.int32, device=dev_)
    gathered = torch.empty((max_tiles * pad, d), dtype=torch.bfloat16, device=dev_)
    _launch(lib.ayk_moe_plan_padded(_ptr(row_of_pair), _ptr(w_rows[0]), _ptr(w_rows[1]), _ptr(gathered), _ptr(route.ids), _ptr(h),
                                    ctypes.c_longlong(h.stride(0)), ctypes.c_int(T), ctypes.c_int(E), ctypes.c_int(route.top),
                                    ctypes.c_int(d), ctypes.c_int(n1), ctypes.c_int(d), ctypes.c_int(max_tiles), _stream()))
    global launches
    launches += 1
    both = torch.empty((max_tiles * pad, n1), dtype=torch.bfloat16, device=dev_)
    _launch(lib.ayk_gemm_tc_prefill_grouped(_ptr(both), _ptr(gathered), _ptr(in_weight), _ptr(w_rows[0]), ctypes.c_int(max_tiles * pad),
                                            ctypes.c_int(n1), ctypes.c_int(d), ctypes.c_int(E * n1), ctypes.c_int(BF16),
                                            ctypes.c_int(sm_count()), _stream()))
    hidden = glu_limited(both, inner, limit, slope, torch.bfloat16, plus)
    picked = torch.empty((max_tiles * pad, d), dtype=torch.float32, device=dev_)
    _launch(lib.ayk_gemm_tc_prefill_grouped(_ptr(picked), _ptr(hidden), _ptr(down_weight), _ptr(w_rows[1]), ctypes.c_int(max_tiles * pad),
                                            ctypes.c_int(d), ctypes.c_int(inner), ctypes.c_int(E * d), ctypes.c_int(F32),
                                            ctypes.c_int(sm_count()), _stream()))
    return picked, row_of_pair


def moe_combine(picked: torch.Tensor, route: MoeRoute, shared: torch.Tensor, mix: torch.Tensor | None,
                row_of_pair: torch.Tensor | None = None) -> torch.Tensor:
    """shared[t] = sum_k weights[t, k] picked[row of pair t * top + k] + sigmoid(mix[t]) shared[t], in place;
    float32.  ``row_of_pair`` None: pair p lies at row p."""
    lib = _ready()
    _f32(picked, "picked"); _f32(shared, "shared")
    T, d = shared.shape
    if picked.shape[1] != d or (row_of_pair is None and picked.shape[0] != T * route.top) or \
            (mix is not None and (mix.dtype != torch.float32 or mix.numel() != T)):
        raise KernelError("moe_combine: rows do not fit")
    _launch(lib.ayk_moe_combine(_ptr(shared), _ptr(picked), _ptr(None if row_of_pair is None else _i32(row_of_pair, "row_of_pair")),
                                _ptr(route.weights), _ptr(mix),
                                ctypes.c_longlong(mix.stride(0) if mix is not None else 0), ctypes.c_int(T),
                                ctypes.c_int(route.top), ctypes.c_int(d), _stream()))
    return shared


# ------------------------------------------------------------- dispatchers --

_tc_scratch: dict = {}
_tc_retired: list = []          # a captured CUDA graph may still write to an outgrown buffer
_sm_count = 0


def sm_count() -> int:
    """Streaming multiprocessors of the current device, asked of the driver once (148 on a B200)."""
    global _sm_count
    if _sm_count == 0:
        _sm_count = int(_ready().ayk_device_sm_count())
    return _sm_count


def _tc_workspace(device, floats: int):
    ws = _tc_scratch.get(device)
    if ws is None or ws[0].numel() < floats:
        if ws is not None:
            _tc_retired.append(ws[0])
        partials = torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=device)
        counters = ws[1] if ws is not None else torch.zeros(8192, dtype=torch.int32, device=device)
        ws = (partials, counters)
        _tc_scratch[device] = ws
    return ws


CLUSTER_ROWS = 64        # up to this many rows the splits of a tile exchange their sums inside a cluster


def tc_splits(M: int, N: int, K: int) -> int:
    """Split-K factor of the tensor-core product: skinny products (few output
    tiles) are cut along K so that about one CTA per SM streams the weight.
    Up to 64 rows the factor is 1, 2, 4, 8 or 16: those splits form a cluster.  16 (beyond the
    portable cluster size) only where each split still has four K blocks: a product of 13
    tiles and K = 6400 streamed at 3.6 TB/s from 104 CTAs, which do not keep enough
    bytes in flight, and at the copy rate from 200.  (The rule itself lives in the library,
    where the native step program uses it too.)"""
    return int(_ready().ayk_tc_splits(ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K)))


def gemm_tc(a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
            activation: str = "none", residual: torch.Tensor | None = None,
            out_dtype: torch.dtype | None = None, out: torch.Tensor | None = None,
            splits: int | None = None, static_weight: bool = True, cluster: bool | None = None) -> torch.Tensor:
    """act(a[M,K] @ w[N,K]^T + bias) (+ residual), bfloat16 operands, on tcgen05.
    ``splits``: CTAs along K per output tile (default: chosen by shape).  ``cluster``:
    the splits exchange their sums through shared memory of a thread-block cluster
    instead of scratch in global memory (default where it applies: up to 64 rows,
    2, 4, 8 or 16 splits)."""
    lib = _ready()
    M, K = a.shape
    N = w.shape[0]
    if (w.shape[1] != K or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16
            or not a.is_contiguous() or not w.is_contiguous()):
        raise KernelError(f"gemm_tc operands do not fit: a {tuple(a.shape)} {a.dtype}, w {tuple(w.shape)} {w.dtype}")
    out_dtype = out_dtype or a.dtype
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    for name, t in (("bias", bias), ("residual", residual)):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise KernelError(f"{name} must be contiguous float32")
    if residual is not None and tuple(residual.shape) != (M, N):
        raise KernelError("residual must have the output's shape")
    if splits is None:
        splits = tc_splits(M, N, K)
    can_cluster = M <= CLUSTER_ROWS and splits in (2, 4, 8, 16) and -(-K // 64) >= splits
    if cluster is None:
        cluster = can_cluster
    elif cluster and not can_cluster:
        raise KernelError(f"gemm_tc: the cluster form takes up to {CLUSTER_ROWS} rows and 2, 4, 8 or 16 splits (rows {M}, splits {splits})")
    partials = counters = None
    if splits > 1 and not cluster:
        tiles = -(-N // 128) * -(-M // 16)
        partials, counters = _tc_workspace(a.device, splits * M * N)
        if tiles > counters.numel():
            raise KernelError("gemm_tc: too many output tiles for split-K")
    _launch(lib.ayk_gemm_tc(_ptr(out), _ptr(a), _ptr(w), _ptr(bias), _ptr(residual), ctypes.c_int(M),
                           ctypes.c_int(N), ctypes.c_int(K), ctypes.c_int(ACTIVATIONS[activation]),
                           ctypes.c_int(_tag(out_dtype)), ctypes.c_int(splits), _ptr(partials), _ptr(counters),
                           ctypes.c_int(1 if static_weight else 0), ctypes.c_int(1 if cluster else 0), _stream()))
    return out


PREFILL_ROWS = 16        # more rows than this: the kernel with 128-row tiles and no split along K


class KVAppend:
    """Where the key and value columns of a fused q | k | v projection belong in the paged
    cache: ``linear`` hands this to the product that can file them itself (the many-row
    tensor-core kernel, in its epilogue) and sets ``done``; the caller appends them with
    ``kv_append`` otherwise."""

    def __init__(self, kcache: torch.Tensor, vcache: torch.Tensor, row_req: torch.Tensor, positions: torch.Tensor,
                 table: torch.Tensor, col0: int, width: int):
        self.kcache, self.vcache, self.row_req, self.positions, self.table = kcache, vcache, row_req, positions, table
        self.col0, self.width = col0, width
        self.done = False

    def fits(self, n_out: int, out_dtype) -> bool:
        pages, P, Hkv, Dh = self.kcache.shape
        return (out_dtype == torch.bfloat16 and self.kcache.dtype == torch.bfloat16 and self.width == Hkv * Dh
                and self.col0 % 8 == 0 and self.width % 8 == 0 and n_out == self.col0 + 2 * self.width
                and self.kcache.is_contiguous() and self.vcache.is_contiguous())


def gemm_tc_prefill(a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
                    activation: str = "none", residual: torch.Tensor | None = None,
                    out_dtype: torch.dtype | None = None, out: torch.Tensor | None = None,
                    tile_n: int = 0, pair: bool | None = None, kv: KVAppend | None = None) -> torch.Tensor:
    """act(a[M,K] @ w[N,K]^T + bias) (+ residual) for many rows: persistent tcgen05
    kernel, epilogue of a tile under the main loop of the next.  ``pair``: two SMs
    on a 256-row tile (tcgen05 cta_group::2) or one SM on a 128-row tile (the default;
    AYAKA_B200_GEMM_PAIR=1 makes pairs the default from 129 rows on).  ``kv``: the product is a
    q | k | v projection whose key and value columns also go into the paged cache."""
    lib = _ready()
    M, K = a.shape
    N = w.shape[0]
    if (w.shape[1] != K or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16
            or not a.is_contiguous() or not w.is_contiguous()):
        raise KernelError(f"gemm_tc_prefill operands do not fit: a {tuple(a.shape)} {a.dtype}, w {tuple(w.shape)} {w.dtype}")
    out_dtype = out_dtype or a.dtype
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    for name, t in (("bias", bias), ("residual", residual)):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise KernelError(f"{name} must be contiguous float32")
    if residual is not None and tuple(residual.shape) != (M, N):
        raise KernelError("residual must have the output's shape")
    if kv is not None:
        if activation != "none" or residual is not None or not kv.fits(N, out_dtype):
            raise KernelError("gemm_tc_prefill: keys and values are filed only by a plain bfloat16 q | k | v projection")
        P = kv.kcache.shape[1]
        _launch(lib.ayk_gemm_tc_prefill_kv(_ptr(out), _ptr(a), _ptr(w), _ptr(bias), ctypes.c_int(M), ctypes.c_int(N),
                                           ctypes.c_int(K), ctypes.c_int(tile_n), ctypes.c_int(sm_count()),
                                           ctypes.c_int(-1 if pair is None else int(pair)), _ptr(kv.kcache), _ptr(kv.vcache),
                                           _ptr(_i32(kv.row_req, "row_req")), _ptr(_i32(kv.positions, "positions")),
                                           _ptr(_i32(kv.table, "table")), ctypes.c_int(kv.table.stride(0)), ctypes.c_int(P),
                                           ctypes.c_int(kv.col0), ctypes.c_int(kv.width), _stream()))
        kv.done = True
        return out
    _launch(lib.ayk_gemm_tc_prefill(_ptr(out), _ptr(a), _ptr(w), _ptr(bias), _ptr(residual), ctypes.c_int(M),
                                    ctypes.c_int(N), ctypes.c_int(K), ctypes.c_int(ACTIVATIONS[activation]),
                                    ctypes.c_int(_tag(out_dtype)), ctypes.c_int(tile_n), ctypes.c_int(sm_count()),
                                    ctypes.c_int(-1 if pair is None else int(pair)), _stream()))
    return out


class _KvTarget(ctypes.Structure):
    _fields_ = [("kcache", ctypes.c_void_p), ("vcache", ctypes.c_void_p), ("row_req", ctypes.c_void_p),
                ("positions", ctypes.c_void_p), ("table", ctypes.c_void_p), ("table_stride", ctypes.c_int32),
                ("page_size", ctypes.c_int32), ("col0", ctypes.c_int32), ("width", ctypes.c_int32),
                ("dtype", ctypes.c_int32)]


def linear(a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
           activation: str = "none", residual: torch.Tensor | None = None,
           out_dtype: torch.dtype | None = None, out: torch.Tensor | None = None,
           kv: KVAppend | None = None) -> torch.Tensor:
    """act(a @ w^T + bias) (+ residual).  float32 operands run on the FP32
    pipes (true 32-bit); bfloat16 operands on the tensor cores (tcgen05) when
    K is a multiple of 8, else on the FP32 pipes with 32-bit accumulation: up to 16 rows,
    and up to 64 rows with few output tiles, the kernel whose CTAs split K inside a cluster;
    above, the persistent kernel with 128-row tiles.  The choice is made in the library
    (``ayk_linear``), by the same code that the native step program runs.
    ``kv``: see KVAppend; ``kv.done`` tells whether the product filed the rows."""
    lib = _ready()
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or a.dtype != w.dtype or not a.is_contiguous() or not w.is_contiguous():
        raise KernelError(f"linear: operands do not fit: a {tuple(a.shape)} {a.dtype}, w {tuple(w.shape)} {w.dtype}")
    out_dtype = out_dtype or a.dtype
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    elif tuple(out.shape) != (M, N) or out.dtype != out_dtype or not out.is_contiguous():
        raise KernelError("linear: out must be a contiguous [M, N] tensor of the output dtype")
    for name, t in (("bias", bias), ("residual", residual)):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise KernelError(f"{name} must be contiguous float32")
    if residual is not None and tuple(residual.shape) != (M, N):
        raise KernelError("residual must have the output's shape")
    target, filed = None, ctypes.c_int(0)
    if kv is not None and kv.fits(N, out_dtype):
        target = _KvTarget(kv.kcache.data_ptr(), kv.vcache.data_ptr(), _i32(kv.row_req, "row_req").data_ptr(),
                           _i32(kv.positions, "positions").data_ptr(), _i32(kv.table, "table").data_ptr(),
                           kv.table.stride(0), kv.kcache.shape[1], kv.col0, kv.width, _tag(kv.kcache.dtype))
    _launch(lib.ayk_linear(_ptr(out), _ptr(a), _ptr(w), _ptr(bias), _ptr(residual), ctypes.c_int(M), ctypes.c_int(N),
                           ctypes.c_int(K), ctypes.c_int(ACTIVATIONS[activation]), ctypes.c_int(_tag(a.dtype)),
                           ctypes.c_int(_tag(out_dtype)), ctypes.byref(target) if target is not None else None,
                           ctypes.byref(filed), _stream()))
    if kv is not None and filed.value:
        kv.done = True
    return out


DECODE_PART = 128
_decode_scratch: dict = {}      # device -> partials; outgrown buffers stay alive below
_decode_retired: list = []      # a captured CUDA graph may still write to an outgrown buffer


def _decode_buffer(device, floats: int) -> torch.Tensor:
    have = _decode_scratch.get(device)
    if have is None or have.numel() < floats:
        if have is not None:
            _decode_retired.append(have)
        have = torch.empty(max(floats, 1 << 21), dtype=torch.float32, device=device)
        _decode_scratch[device] = have
    return have


def attention_decode(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, table: torch.Tensor,
                     req_pos0: torch.Tensor, num_heads: int, scale: float, window: int | None,
                     max_context: int, out: torch.Tensor | None = None,
                     append: tuple | None = None, settled: bool = False) -> torch.Tensor:
    """One query row per request over its pages, split along the context and
    merged.  ``max_context``: the longest context the engine allows (fixes the grid).
    ``append`` = (k, v, row_req): this step's key and value rows, not yet in the
    cache; they are stored at each request's position on the way (inside the
    attention kernel where it can, else by the append kernel first).  ``settled``:
    the cache rows before the requests' positions were written by work that is
    complete (an earlier step); the kernel may then read them while the kernels
    launched just before it still run."""
    lib = _ready()
    pages, P, Hkv, Dh = kcache.shape
    R = q.shape[0]
    if q.shape[1] != num_heads * Dh or q.stride(1) != 1 or q.dtype != kcache.dtype:
        raise KernelError("attention_decode: q must be a [R, heads*head_dim] slice of the cache's dtype")
    if req_pos0.numel() != R:
        raise KernelError("attention_decode: one row per request")
    parts = -(-max_context // DECODE_PART)
    scratch = _decode_buffer(q.device, R * num_heads * parts * (Dh + 2))
    if out is None:
        out = torch.empty((R, num_heads * Dh), dtype=q.dtype, device=q.device)
    k_new = v_new = row_req = None
    new_stride = 0
    if append is not None:
        k_new, v_new, row_req = append
        if (k_new.shape != (R, Hkv * Dh) or v_new.shape != k_new.shape or k_new.stride(1) != 1 or v_new.stride(1) != 1
                or k_new.stride(0) != v_new.stride(0) or k_new.dtype != kcache.dtype or v_new.dtype != kcache.dtype):
            raise KernelError("attention_decode: new keys and values must be [R, kv_heads*head_dim] slices of one matrix")
        new_stride = k_new.stride(0)
    _launch(lib.ayk_attention_decode(_ptr(out), _ptr(q), ctypes.c_int(q.stride(0)), _ptr(kcache), _ptr(vcache),
                                     _ptr(_i32(table, "table")), ctypes.c_int(table.stride(0)),
                                     _ptr(_i32(req_pos0, "req_pos0")), ctypes.c_int(R), ctypes.c_int(num_heads),
                                     ctypes.c_int(Hkv), ctypes.c_int(Dh), ctypes.c_int(P), ctypes.c_float(scale),
                                     ctypes.c_int(window or 0), ctypes.c_int(parts), _ptr(scratch),
                                     _ptr(k_new), _ptr(v_new), ctypes.c_int(new_stride),
                                     _ptr(_i32(row_req, "row_req") if row_req is not None else None),
                                     ctypes.c_longlong(pages), ctypes.c_int(1 if settled else 0),
                                     ctypes.c_int(_tag(q.dtype)), _stream()))
    global launches
    launches += 1            # the call launches two kernels (partitions, merge)
    return out


def attention_tc_takes(q: torch.Tensor, kcache: torch.Tensor) -> bool:
    """Whether the tensor-core attention kernel takes this geometry: bfloat16,
    head size 64, pages of 8 to 128 tokens, 16-byte aligned query rows."""
    pages, P, Hkv, Dh = kcache.shape
    return (q.dtype == torch.bfloat16 and Dh == 64 and 8 <= P <= 128 and P & (P - 1) == 0
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0)


def attention_tc(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, table: torch.Tensor,
                 req_q_start: torch.Tensor, req_pos0: torch.Tensor, total_rows: int, num_heads: int,
                 scale: float, window: int | None = None, out: torch.Tensor | None = None,
                 first_row: int = 0) -> torch.Tensor:
    """Causal attention of prompt portions over the paged cache on tcgen05 (bfloat16, head size 64).
    ``first_row``: the requests named here cover rows first_row .. T of ``q`` and ``out`` (their
    ``req_q_start`` holds absolute row numbers); earlier rows are left to another kernel."""
    lib = _ready()
    pages, P, Hkv, Dh = kcache.shape
    T = q.shape[0]
    if q.shape[1] != num_heads * Dh or q.stride(1) != 1 or q.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16:
        raise KernelError("attention_tc: q must be a bfloat16 [T, heads*head_dim] slice, the cache bfloat16")
    if total_rows + first_row != T:
        raise KernelError(f"attention_tc: rows {first_row} .. {first_row + total_rows} named, q has {T} "
                          f"(rows beyond the count would stay unwritten)")
    if not kcache.is_contiguous() or not vcache.is_contiguous():
        raise KernelError("attention_tc: the cache must be contiguous")
    if out is None:
        out = torch.empty((T, num_heads * Dh), dtype=q.dtype, device=q.device)
    R = req_pos0.numel()
    _launch(lib.ayk_attention_tc(_ptr(out), _ptr(q), ctypes.c_int(q.stride(0)), ctypes.c_int(T), ctypes.c_int(total_rows),
                                 _ptr(kcache), _ptr(vcache), ctypes.c_int(pages), _ptr(_i32(table, "table")),
                                 ctypes.c_int(table.stride(0)), _ptr(_i32(req_q_start, "req_q_start")),
                                 _ptr(_i32(req_pos0, "req_pos0")), ctypes.c_int(R), ctypes.c_int(num_heads),
                                 ctypes.c_int(Hkv), ctypes.c_int(Dh), ctypes.c_int(P), ctypes.c_float(scale),
                                 ctypes.c_int(window or 0), _stream()))
    return out


MIXED_DECODE_MIN = 1     # single-token requests in a mixed step from which they take the decode kernels


def tc_error() -> int:
    """0, or the code of the bounded wait that ran out in a tensor-core kernel
    (1-4: matrix product, 11-17: attention)."""
    lib = library()
    return (int(lib.ayk_gemm_tc_error()) or int(lib.ayk_attention_tc_error())
            or int(lib.ayk_gemm_tc_prefill_error()))


def attention(q, kcache, vcache, table, ctx, num_heads: int, scale: float,
              window: int | None = None, append: tuple | None = None) -> torch.Tensor:
    """Attention of the step's rows (``ctx`` gives the rows of each request): the
    split-context decode kernels when every request brings one row (head sizes in
    steps of 16); the tensor-core kernel for prompt portions in bfloat16 with head
    size 64, beside the decode kernels for the single rows of a mixed step; else
    the general kernel, which takes every head size up to 256.  ``append`` = (k, v): the rows' keys and values, which
    go into the cache first (in a decode step, inside the attention kernel)."""
    # Head sizes that are no multiple of 16 are taken by the general kernel alone (the decode kernels
    # read keys in 16-byte pieces and refuse them).
    if ctx.max_q_len == 1 and kcache.shape[3] % 16 == 0:
        return attention_decode(q, kcache, vcache, table, ctx.req_pos0, num_heads, scale, window,
                                ctx.cache.max_len,
                                append=(append[0], append[1], ctx.row_req) if append is not None else None,
                                settled=getattr(ctx, "earlier_rows_settled", False))
    if append is not None:
        kv_append(kcache, vcache, append[0], append[1], ctx.row_req, ctx.positions, table)
    if attention_tc_takes(q, kcache):
        # A mixed step: its single-token requests are its first rows (the step runner packs them
        # first).  They go through the split-context decode kernels, one row per request, and the
        # prompt portions through the tiled kernel: two launches on disjoint row ranges over one
        # block table.  (As rows of the tiled kernel each would be a 128-row tile with one live row.)
        D = getattr(ctx, "num_single", 0)
        if D >= MIXED_DECODE_MIN and D < ctx.num_requests:
            out = torch.empty((ctx.num_rows, q.shape[1]), dtype=q.dtype, device=q.device)
            attention_decode(q[:D], kcache, vcache, table[:D], ctx.req_pos0[:D], num_heads, scale, window,
                             ctx.cache.max_len, out=out[:D], settled=getattr(ctx, "earlier_rows_settled", False))
            return attention_tc(q, kcache, vcache, table[D:], ctx.req_q_start[D:], ctx.req_pos0[D:],
                                ctx.num_rows - D, num_heads, scale, window, out=out, first_row=D)
        return attention_tc(q, kcache, vcache, table, ctx.req_q_start, ctx.req_pos0, ctx.num_rows,
                            num_heads, scale, window)
    return attention_simt(q, kcache, vcache, table, ctx.req_q_start, ctx.req_pos0, ctx.num_rows,
                          num_heads, scale, window)
