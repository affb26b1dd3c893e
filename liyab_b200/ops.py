"""Python faces of the CUDA kernels.

Each function checks what the kernel cannot check for itself (device, types,
contiguity, sizes it refuses), passes raw device pointers and the current CUDA
stream to the library's C interface, and turns a non-zero status into a
`LiyabError`.  Nothing here computes: there is no CPU path and no library
fallback; a tensor that is not on a CUDA device is an error.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc.build import load_library
from .status import ErrorCode, LiyabError, invalid_argument

F32, BF16 = 0, 1
ACTIVATIONS = {"none": 0, "gelu_tanh": 1, "gelu_erf": 2, "xielu": 3, "relu2": 4}      # xielu: the bias holds N + 2 values, the last two the learned pair
_DT = {torch.float32: F32, torch.bfloat16: BF16}

_c = ctypes
_p, _i, _l, _f = _c.c_void_p, _c.c_int, _c.c_int64, _c.c_float

_SIGNATURES = {
    "lb_embed_positions": [_i, _p, _p, _p, _p, _p, _i, _i, _f, _p],
    "lb_gather_tokens": [_p, _p, _p, _i, _p],
    "lb_layernorm": [_i, _p, _p, _p, _p, _p, _i, _i, _f, _p],
    "lb_kv_append": [_i, _p, _p, _l, _p, _p, _i, _i, _i, _i, _p],
    "lb_gemm_ffma": [_i, _i, _p, _l, _p, _l, _p, _p, _l, _p, _l, _i, _i, _i, _i, _p],
    "lb_gemm_tcgen05": [_i, _p, _l, _p, _l, _p, _p, _l, _p, _l, _i, _i, _i, _i, _i, _p, _p, _i, _p],
    "lb_gemm_tcgen05_status": [_p],
    "lb_gemm_rows_supports": [_p, _l, _p, _l, _i, _i, _i],
    "lb_gemm_rows_normed_supports": [_p, _l, _p, _l, _i, _i, _i],
    "lb_gemm_rows_normed": [_i, _p, _l, _p, _p, _f, _p, _l, _p, _p, _l, _p, _l, _i, _i, _i, _i, _p, _p, _i, _i, _i, _i, _p],
    "lb_gemm_rows": [_i, _p, _l, _p, _l, _p, _p, _l, _p, _l, _i, _i, _i, _i, _p, _p, _i, _i, _i, _i, _p],
    "lb_gemm_persistent_tile": [_i, _p, _l, _p, _l, _p, _l, _p, _l, _i, _i, _i],
    "lb_gemm_persistent_timing": [_p],
    "lb_gemm_persistent": [_i, _p, _l, _p, _l, _p, _p, _l, _p, _l, _i, _i, _i, _i, _i, _p, _p, _i, _i, _i, _i, _p],
    "lb_gemm_persistent_kv_supports": [_i, _i, _i, _i, _i, _i, _i, _i],
    "lb_paged_attention_generic": [_i, _p, _l, _p, _p, _p, _p, _i, _p, _l, _i, _i, _i, _i, _i, _f, _i, _p],
    "lb_decode_attention": [_p, _l, _p, _p, _p, _i, _p, _l, _p, _p, _i, _i, _i, _i, _i, _f, _i, _i, _p],
    "lb_decode_attention_supports": [_i, _i, _i, _i],
    "lb_decode_attention_mma": [_p, _l, _p, _i, _p, _p, _i, _p, _l, _p, _p, _i, _i, _i, _i, _i, _f, _i, _i, _p],
    "lb_decode_attention_mma_supports": [_i, _i, _i, _i],
    "lb_prefill_attention": [_p, _l, _p, _p, _p, _p, _i, _p, _l, _i, _i, _i, _i, _i, _i, _f, _i, _p],
    "lb_prefill_attention_supports": [_i, _i, _i, _i],
    "lb_prefill_attention_tc": [_p, _l, _i, _p, _i, _p, _p, _p, _i, _p, _l, _i, _i, _i, _i, _i, _i, _f, _i, _p],
    "lb_prefill_attention_tc_supports": [_i, _i, _i, _i],
    "lb_sample": [_p, _l, _i, _i, _p, _p, _p, _p, _p, _p, _p],
    "lb_paged_attention_generic_biased": [_i, _p, _l, _p, _p, _p, _p, _i, _p, _l, _i, _i, _i, _i, _i, _f, _i, _p, _p],
    "lb_decode_attention_biased": [_p, _l, _p, _p, _p, _i, _p, _l, _p, _p, _i, _i, _i, _i, _i, _f, _i, _i, _p, _p],
    "lb_decode_attention_mma_biased": [_p, _l, _p, _i, _p, _p, _i, _p, _l, _p, _p, _i, _i, _i, _i, _i, _f, _i, _i, _p, _p],
    "lb_prefill_attention_biased": [_p, _l, _p, _p, _p, _p, _i, _p, _l, _i, _i, _i, _i, _i, _i, _f, _i, _p, _p],
    "lb_prefill_attention_tc_biased": [_p, _l, _i, _p, _i, _p, _p, _p, _i, _p, _l, _i, _i, _i, _i, _i, _i, _f, _i, _p, _p],
    "lb_paged_attention_generic_sink": [_i, _p, _l, _p, _p, _p, _p, _i, _p, _l, _i, _i, _i, _i, _i, _f, _i, _p, _p, _p],
    "lb_decode_attention_sink": [_p, _l, _p, _p, _p, _i, _p, _l, _p, _p, _i, _i, _i, _i, _i, _f, _i, _i, _p, _p, _p],
    "lb_decode_attention_mma_sink": [_p, _l, _p, _i, _p, _p, _i, _p, _l, _p, _p, _i, _i, _i, _i, _i, _f, _i, _i, _p, _p, _p],
    "lb_prefill_attention_sink": [_p, _l, _p, _p, _p, _p, _i, _p, _l, _i, _i, _i, _i, _i, _i, _f, _i, _p, _p, _p],
    "lb_prefill_attention_tc_sink": [_p, _l, _i, _p, _i, _p, _p, _p, _i, _p, _l, _i, _i, _i, _i, _i, _i, _f, _i, _p, _p, _p],
    "lb_qkv_rotary_store": [_i, _p, _l, _i, _i, _i, _p, _p, _p, _l, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _f, _p, _p, _i, _p, _p, _l, _p, _p],
    "lb_row_norm_gate": [_i, _p, _l, _p, _l, _p, _p, _l, _i, _i, _i, _f, _p],
    "lb_activate_columns": [_p, _l, _i, _i, _i, _p],
    "lb_router_table": [_p, _p, _p, _p, _i, _i, _i, _i, _p],
}

_lib = None
LAUNCHES = 0        # kernel launches issued through this module (a captured graph replays its own count)


def lib():
    """The kernel library with argument types declared (built at first use)."""
    global _lib
    if _lib is None:
        l = load_library()
        l.lb_last_error.restype = _c.c_char_p
        for name, args in _SIGNATURES.items():
            fn = getattr(l, name)
            fn.argtypes = args
            fn.restype = _i
        _lib = l
    return _lib


def declare(name: str, argtypes) -> None:
    """Registers the signature of a further exported function."""
    _SIGNATURES[name] = argtypes
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.argtypes = argtypes
        fn.restype = _i


def check(status: int, what: str) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if status != 0:
        msg = lib().lb_last_error().decode("utf-8", "replace")
        try:
            code = ErrorCode(status)
        except ValueError:
            code = ErrorCode.INTERNAL
        raise LiyabError(code, f"{what}: {msg}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr() -> int:
    """The current CUDA stream of the current device as a raw pointer (asked once per launch, so by the short way
    where torch offers it)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _dev(t: torch.Tensor, name: str, dtype: Optional[torch.dtype] = None) -> int:
    if not t.is_cuda:
        raise invalid_argument(f"{name} is on {t.device}; the engine's kernels run on a CUDA device only")
    if dtype is not None and t.dtype != dtype:
        raise invalid_argument(f"{name} has dtype {t.dtype}, expected {dtype}")
    return t.data_ptr()


def _opt(t: Optional[torch.Tensor], name: str, dtype: Optional[torch.dtype] = None) -> Optional[int]:
    return None if t is None else _dev(t, name, dtype)


def _code(dtype: torch.dtype, name: str) -> int:
    if dtype not in _DT:
        raise invalid_argument(f"{name} has dtype {dtype}; the kernels take float32 and bfloat16")
    return _DT[dtype]


# ------------------------------------------------------------------ elementwise

def embed_positions(tokens: torch.Tensor, positions: torch.Tensor, table: torch.Tensor,
                    pos_table: Optional[torch.Tensor], out: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """out[t] = table[tokens[t]] * scale + pos_table[positions[t]], 32-bit."""
    n, width = tokens.numel(), table.shape[1]
    if pos_table is not None and (pos_table.dtype != table.dtype or pos_table.shape[1] != width):
        raise invalid_argument("embed: the position table does not match the embedding table")
    if out.shape[0] < n or out.shape[1] != width or not out.is_contiguous():
        raise invalid_argument("embed: output buffer has the wrong shape")
    check(lib().lb_embed_positions(_code(table.dtype, "table"), _dev(tokens, "tokens", torch.int32),
                                   _dev(positions, "positions", torch.int32), _dev(table, "table"),
                                   _opt(pos_table, "pos_table"), _dev(out, "out", torch.float32), n, width,
                                   float(scale), stream_ptr()), "embed_positions")
    return out


def gather_tokens(dst: torch.Tensor, src: torch.Tensor, token_map: torch.Tensor, n: int) -> None:
    """dst[i] = src[token_map[i]] where token_map[i] >= 0 (tokens that never left the device)."""
    check(lib().lb_gather_tokens(_dev(dst, "dst", torch.int32), _dev(src, "src", torch.int32),
                                 _dev(token_map, "token_map", torch.int32), n, stream_ptr()), "gather_tokens")


def layernorm(x: torch.Tensor, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor], eps: float,
              out: torch.Tensor, n_rows: int, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = LayerNorm(x[rows[r]] or x[r]); statistics in 32-bit."""
    width = x.shape[1]
    if not x.is_contiguous() or not out.is_contiguous() or out.shape[1] != width or out.shape[0] < n_rows:
        raise invalid_argument("layernorm: buffers must be contiguous [rows, width]")
    check(lib().lb_layernorm(_code(out.dtype, "out"), _dev(x, "x", torch.float32), _opt(rows, "rows", torch.int32),
                             _opt(weight, "weight", torch.float32), _opt(bias, "bias", torch.float32), _dev(out, "out"),
                             n_rows, width, float(eps), stream_ptr()), "layernorm")
    return out


def kv_append(k: torch.Tensor, v: torch.Tensor, slot_mapping: torch.Tensor, cache: torch.Tensor, n_tokens: int,
              n_kv_head: int, head_dim: int, page_size: int) -> None:
    """Copies the step's key and value rows (views with a common row stride) into the layer's pages."""
    if k.stride(0) != v.stride(0) or k.stride(1) != 1 or v.stride(1) != 1 or k.dtype != cache.dtype:
        raise invalid_argument("kv_append: k and v must share a row stride, be dense in a row and match the cache type")
    check(lib().lb_kv_append(_code(cache.dtype, "cache"), _dev(k, "k"), _dev(v, "v"), k.stride(0),
                             _dev(slot_mapping, "slot_mapping", torch.int32), _dev(cache, "cache"), n_tokens,
                             n_kv_head, head_dim, page_size, stream_ptr()), "kv_append")


# ------------------------------------------------------------------ matrix products

def gemm_ffma(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, m: int,
              activation: str = "none", residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[:m] = act(a[:m] @ w.T + bias) + residual, on the 32-bit units."""
    n, k = w.shape
    if a.shape[1] != k or a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1 or out.shape[1] != n:
        raise invalid_argument(f"gemm: shapes do not fit: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if a.dtype != w.dtype:
        raise invalid_argument(f"gemm: a is {a.dtype} but w is {w.dtype}")
    if residual is not None and (residual.shape[1] != n or residual.stride(1) != 1):
        raise invalid_argument("gemm: residual has the wrong shape")
    check(lib().lb_gemm_ffma(_code(a.dtype, "a"), _code(out.dtype, "out"), _dev(a, "a"), a.stride(0), _dev(w, "w"),
                             w.stride(0), _opt(bias, "bias", torch.float32), _opt(residual, "residual", torch.float32),
                             residual.stride(0) if residual is not None else 0, _dev(out, "out"), out.stride(0), m, n,
                             k, ACTIVATIONS[activation], stream_ptr()), "gemm_ffma")
    return out


def tcgen05_accepts(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tensor-core product takes these operands: bfloat16, and TMA's 16-byte rules."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0 and a.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and a.stride(1) == 1 and w.stride(1) == 1)


def gemm_splits(m: int, n: int, k: int) -> int:
    """How many ways K is split for a product of few tokens: enough blocks for most of the GPU's SMs."""
    if m > 64 or m <= 0:
        return 1
    tiles, k_blocks = -(-n // 128), -(-k // 64)
    return max(1, min(k_blocks, 16, -(-96 // tiles)))


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, m: int,
                 activation: str = "none", residual: Optional[torch.Tensor] = None, token_tile: int = 0,
                 partial: Optional[torch.Tensor] = None, counters: Optional[torch.Tensor] = None, n_splits: int = 1
                 ) -> torch.Tensor:
    """out[:m] = act(a[:m] @ w.T + bias) + residual on the tcgen05 tensor cores (bfloat16 operands).
    n_splits > 1 (m <= 64) splits K over blocks; `partial` holds n_splits * m * n floats and `counters`
    one zeroed int per 128 features."""
    n, k = w.shape
    if a.shape[1] != k or out.stride(1) != 1 or out.shape[1] != n:
        raise invalid_argument(f"gemm: shapes do not fit: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if not tcgen05_accepts(a, w):
        raise invalid_argument("gemm_tcgen05: operands must be bfloat16 with K and row strides multiples of 8")
    if residual is not None and (residual.shape[1] != n or residual.stride(1) != 1):
        raise invalid_argument("gemm: residual has the wrong shape")
    check(lib().lb_gemm_tcgen05(_code(out.dtype, "out"), _dev(a, "a"), a.stride(0), _dev(w, "w"), w.stride(0),
                                _opt(bias, "bias", torch.float32), _opt(residual, "residual", torch.float32),
                                residual.stride(0) if residual is not None else 0, _dev(out, "out"), out.stride(0), m, n,
                                k, ACTIVATIONS[activation], token_tile, _opt(partial, "partial", torch.float32),
                                _opt(counters, "counters", torch.int32), n_splits, stream_ptr()), "gemm_tcgen05")
    return out


def _kv_args(kv: Optional[tuple]) -> tuple:
    if kv is None:
        return None, None, 0, 0, 0, 0
    cache, slot_mapping, q_dim, n_kv_head, head_dim, page_size = kv
    if cache.dtype != torch.bfloat16:
        raise invalid_argument("gemm: the cache destination must be bfloat16")
    return _dev(cache, "cache"), _dev(slot_mapping, "slot_mapping", torch.int32), q_dim, n_kv_head, head_dim, page_size


def gemm_rows_supports(a: torch.Tensor, w: torch.Tensor, m: int) -> bool:
    """Whether the one-launch product for 1 to 64 tokens takes these operands."""
    if not tcgen05_accepts(a, w):
        return False
    return bool(lib().lb_gemm_rows_supports(_dev(a, "a"), a.stride(0), _dev(w, "w"), w.stride(0), m, w.shape[0], w.shape[1]))


def gemm_rows(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, m: int,
              activation: str = "none", residual: Optional[torch.Tensor] = None, kv: Optional[tuple] = None) -> torch.Tensor:
    """out[:m] = act(a[:m] @ w.T + bias) + residual for 1 to 64 tokens: one launch, weights streamed once.
    `kv` = (cache, slot_mapping, q_dim, n_kv_head, head_dim, page_size): the features from q_dim on are keys and
    values of a fused projection and also go to the tokens' cache slots."""
    n, k = w.shape
    if a.shape[1] != k or out.stride(1) != 1 or out.shape[1] != n:
        raise invalid_argument(f"gemm: shapes do not fit: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if residual is not None and (residual.shape[1] != n or residual.stride(1) != 1):
        raise invalid_argument("gemm: residual has the wrong shape")
    check(lib().lb_gemm_rows(_code(out.dtype, "out"), _dev(a, "a"), a.stride(0), _dev(w, "w"), w.stride(0),
                             _opt(bias, "bias", torch.float32), _opt(residual, "residual", torch.float32),
                             residual.stride(0) if residual is not None else 0, _dev(out, "out"), out.stride(0), m, n, k,
                             ACTIVATIONS[activation], *_kv_args(kv), stream_ptr()), "gemm_rows")
    return out


def gemm_rows_normed(x: torch.Tensor, gain: Optional[torch.Tensor], offset: Optional[torch.Tensor], eps: float, w: torch.Tensor,
                     bias: Optional[torch.Tensor], out: torch.Tensor, m: int, activation: str = "none",
                     residual: Optional[torch.Tensor] = None, kv: Optional[tuple] = None) -> torch.Tensor:
    """out[:m] = act(LayerNorm(x[:m]) @ w.T + bias) + residual for up to 16 tokens and K up to 1024: the rows are
    normalised inside the product's kernel.  `kv` as for gemm_rows."""
    n, k = w.shape
    cache, slots, q_dim, n_kv_head, head_dim, page_size = _kv_args(kv)
    check(lib().lb_gemm_rows_normed(_code(out.dtype, "out"), _dev(x, "x", torch.float32), x.stride(0), _opt(gain, "gain", torch.float32),
                                    _opt(offset, "offset", torch.float32), float(eps), _dev(w, "w", torch.bfloat16), w.stride(0),
                                    _opt(bias, "bias", torch.float32), _opt(residual, "residual", torch.float32),
                                    residual.stride(0) if residual is not None else 0, _dev(out, "out"), out.stride(0), m, n, k,
                                    ACTIVATIONS[activation], cache, slots, q_dim, n_kv_head, head_dim, page_size, stream_ptr()),
          "gemm_rows_normed")
    return out


def gemm_persistent_tile(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, m: int,
                         residual: Optional[torch.Tensor] = None) -> int:
    """The feature tile the persistent tensor-core product would use for these operands, 0 where it does not take them."""
    if not tcgen05_accepts(a, w) or out.stride(1) != 1 or (residual is not None and residual.stride(1) != 1):
        return 0
    n, k = w.shape
    return int(lib().lb_gemm_persistent_tile(
        _code(out.dtype, "out"), _dev(a, "a"), a.stride(0), _dev(w, "w"), w.stride(0),
        _opt(residual, "residual", torch.float32), residual.stride(0) if residual is not None else 0, _dev(out, "out"),
        out.stride(0), m, n, k))


def gemm_persistent_kv_supports(w: torch.Tensor, out: torch.Tensor, q_dim: int, n_kv_head: int, head_dim: int,
                                page_size: int) -> bool:
    """Whether gemm_persistent can put the keys and values of a fused projection with these sizes into the cache."""
    return bool(lib().lb_gemm_persistent_kv_supports(_code(out.dtype, "out"), w.shape[0], ACTIVATIONS["none"], 0, q_dim,
                                                     n_kv_head, head_dim, page_size))


def gemm_persistent(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, m: int,
                    activation: str = "none", residual: Optional[torch.Tensor] = None, feature_tile: int = 0,
                    kv: Optional[tuple] = None) -> torch.Tensor:
    """out[:m] = act(a[:m] @ w.T + bias) + residual for more than 64 tokens: persistent tcgen05 kernel, every
    operand, the residual and the result moved by TMA.  `kv` = (cache, slot_mapping, q_dim, n_kv_head, head_dim,
    page_size): the product is a fused query/key/value projection; the features from q_dim on go into the cache's
    pages (row i at slot_mapping[i]) and not into `out`."""
    n, k = w.shape
    if a.shape[1] != k or out.stride(1) != 1 or out.shape[1] != n:
        raise invalid_argument(f"gemm: shapes do not fit: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if residual is not None and (residual.shape[1] != n or residual.stride(1) != 1):
        raise invalid_argument("gemm: residual has the wrong shape")
    check(lib().lb_gemm_persistent(_code(out.dtype, "out"), _dev(a, "a"), a.stride(0), _dev(w, "w"), w.stride(0),
                                   _opt(bias, "bias", torch.float32), _opt(residual, "residual", torch.float32),
                                   residual.stride(0) if residual is not None else 0, _dev(out, "out"), out.stride(0), m, n,
                                   k, ACTIVATIONS[activation], feature_tile, *_kv_args(kv), stream_ptr()), "gemm_persistent")
    return out


def device_status() -> int:
    """0 unless a bounded wait inside a kernel ran out since the last call (then where it gave up).
    Synchronises the device."""
    status = ctypes.c_int(0)
    check(lib().lb_gemm_tcgen05_status(ctypes.byref(status)), "device_status")
    return status.value


def linear(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, m: int,
           activation: str = "none", residual: Optional[torch.Tensor] = None, workspace=None) -> torch.Tensor:
    """out[:m] = act(a[:m] @ w.T + bias) + residual: the kernel is chosen by type and size.  With a workspace
    (scratch buffers) a product of few tokens splits K over blocks."""
    if tcgen05_accepts(a, w):
        if m > 64 and gemm_persistent_tile(a, w, out, m, residual) > 0:
            return gemm_persistent(a, w, bias, out, m, activation, residual)
        # Up to 64 tokens: one launch on mma.sync where every block can afford to fetch all activations (measured on
        # B200, 64 tokens: 6-7 us against 8-9 us for K = 768; for K = 3072 the 393 KB of activations per block cost
        # more than the split of K saves: 13 us against 8 us; 8 tokens with K = 1600 or 3072 lose to the split too).
        if m <= 64 and w.shape[1] <= 1024 and gemm_rows_supports(a, w, m):
            return gemm_rows(a, w, bias, out, m, activation, residual)
        splits = gemm_splits(m, w.shape[0], w.shape[1]) if workspace is not None else 1
        if splits > 1:
            partial = workspace.flat("gemm.partial", splits * m * w.shape[0], torch.float32)
            counters = workspace.flat("gemm.counters", -(-w.shape[0] // 128), torch.int32, zero=True)
            return gemm_tcgen05(a, w, bias, out, m, activation, residual, 0, partial, counters, splits)
        return gemm_tcgen05(a, w, bias, out, m, activation, residual)
    return gemm_ffma(a, w, bias, out, m, activation, residual)


# ------------------------------------------------------------------ attention

def paged_attention_generic(q: torch.Tensor, cache: torch.Tensor, tok_seq: torch.Tensor, positions: torch.Tensor,
                            block_table: torch.Tensor, out: torch.Tensor, n_tokens: int, n_head: int, n_kv_head: int,
                            head_dim: int, page_size: int, scale: float, window: int = 0, distance: Optional[torch.Tensor] = None,
                            sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of the step's tokens over their requests' pages, 32-bit arithmetic.  `distance` (float32, r1 [n_head] then
    r2 [n_head]): the score of the key d positions back loses r1 ln(1 + r2 d).  `sink` (float32 [n_head]): exp(sink[h]) joins the divisor
    of head h's softmax, with no key and no value."""
    if q.dtype != cache.dtype or out.dtype != cache.dtype:
        raise invalid_argument("attention: q, cache and out must have one element type")
    if q.stride(1) != 1 or out.stride(1) != 1:
        raise invalid_argument("attention: q and out must be dense within a row")
    check(lib().lb_paged_attention_generic_sink(
        _code(cache.dtype, "cache"), _dev(q, "q"), q.stride(0), _dev(cache, "cache"),
        _dev(tok_seq, "tok_seq", torch.int32), _dev(positions, "positions", torch.int32),
        _dev(block_table, "block_table", torch.int32), block_table.stride(0), _dev(out, "out"), out.stride(0),
        n_tokens, n_head, n_kv_head, head_dim, page_size, float(scale), int(window), _distance(distance, n_head), _sink(sink, n_head), stream_ptr()),
        "paged_attention_generic")
    return out


def _distance(distance: Optional[torch.Tensor], n_head: int) -> Optional[int]:
    if distance is not None and (distance.numel() != 2 * n_head or not distance.is_contiguous()):
        raise invalid_argument("attention: the penalty by distance is r1 [n_head] then r2 [n_head]")
    return _opt(distance, "distance", torch.float32)


def _sink(sink: Optional[torch.Tensor], n_head: int) -> Optional[int]:
    if sink is not None and (sink.numel() != n_head or not sink.is_contiguous()):
        raise invalid_argument("attention: the sinks are one float a head")
    return _opt(sink, "sink", torch.float32)


def decode_attention_kernels(n_head: int, n_kv_head: int, head_dim: int, page_size: int) -> tuple:
    """(scalar kernel takes the shape, tensor-core kernel takes it)."""
    return (bool(lib().lb_decode_attention_supports(n_head, n_kv_head, head_dim, page_size)),
            bool(lib().lb_decode_attention_mma_supports(n_head, n_kv_head, head_dim, page_size)))


def decode_attention_supports(n_head: int, n_kv_head: int, head_dim: int, page_size: int) -> bool:
    return any(decode_attention_kernels(n_head, n_kv_head, head_dim, page_size))


def decode_splits(n_seq: int, n_kv_head: int, max_context: int = 0, tensor_cores: bool = False) -> int:
    """How many ways each request's keys are split.  Scalar kernel: enough blocks for about four full waves of
    the GPU, but no ranges shorter than 128 keys at the longest context.  Tensor-core kernel: a block gets through
    its keys far faster, so fewer and longer ranges (about 450 blocks, 96 keys or more each; up to eight ranges merge
    inside a cluster); from 32 requests of 12 heads on, none.  A function of the batch's shape only, so a captured step and an eager one split alike."""
    work = max(1, n_seq * n_kv_head)
    if tensor_cores:
        cap = max(1, max_context // 96) if max_context else 32
        n = max(1, min(32, cap, 444 // work))
        return 8 if 8 < n < 16 else n          # eight ranges that merge inside a cluster beat a few more that cannot
    cap = max(1, max_context // 128) if max_context else 32
    return max(1, min(32, cap, -(-2960 // work)))


def decode_attention(q: torch.Tensor, cache: torch.Tensor, positions: torch.Tensor, block_table: torch.Tensor,
                     out: torch.Tensor, partial: Optional[torch.Tensor], counters: Optional[torch.Tensor], n_seq: int,
                     n_head: int, n_kv_head: int, head_dim: int, page_size: int, scale: float, window: int,
                     n_splits: int, tensor_cores: Optional[bool] = None, distance: Optional[torch.Tensor] = None,
                     sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of one new token per request over its pages (bfloat16), keys split `n_splits` ways.
    `tensor_cores`: None picks the tensor-core kernel where it takes the shape, else the scalar one.  `distance`: as for
    paged_attention_generic."""
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise invalid_argument("decode attention takes bfloat16 only")
    if q.stride(1) != 1 or out.stride(1) != 1 or q.stride(0) % 8 != 0 or q.data_ptr() % 16 != 0:
        raise invalid_argument("decode attention: q rows must be dense, 16-byte aligned and a multiple of 8 elements apart")
    if n_splits > 1:
        need = n_seq * n_head * n_splits * (head_dim + 2)
        if partial is None or counters is None or partial.numel() < need or counters.numel() < n_seq * n_kv_head:
            raise invalid_argument("decode attention: scratch buffers are missing or too small")
    if tensor_cores is None:
        tensor_cores = decode_attention_kernels(n_head, n_kv_head, head_dim, page_size)[1]
    cache_args = (_dev(cache, "cache"), cache.shape[0]) if tensor_cores else (_dev(cache, "cache"),)
    fn = lib().lb_decode_attention_mma_sink if tensor_cores else lib().lb_decode_attention_sink
    check(fn(
        _dev(q, "q"), q.stride(0), *cache_args, _dev(positions, "positions", torch.int32),
        _dev(block_table, "block_table", torch.int32), block_table.stride(0), _dev(out, "out"), out.stride(0),
        _opt(partial, "partial", torch.float32), _opt(counters, "counters", torch.int32), n_seq, n_head, n_kv_head,
        head_dim, page_size, float(scale), int(window), int(n_splits), _distance(distance, n_head), _sink(sink, n_head), stream_ptr()), "decode_attention")
    return out


def prefill_attention_supports(n_head: int, n_kv_head: int, head_dim: int, page_size: int) -> bool:
    return bool(lib().lb_prefill_attention_supports(n_head, n_kv_head, head_dim, page_size))


_SM_COUNT = {}


def _sm_count(device) -> int:
    key = torch.device(device).index or 0
    if key not in _SM_COUNT:
        _SM_COUNT[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _SM_COUNT[key]


def prefill_attention_tc_supports(n_head: int, n_kv_head: int, head_dim: int, page_size: int) -> bool:
    return bool(lib().lb_prefill_attention_tc_supports(n_head, n_kv_head, head_dim, page_size))


def prefill_attention(q: torch.Tensor, cache: torch.Tensor, q_start: torch.Tensor, n_past: torch.Tensor,
                      block_table: torch.Tensor, out: torch.Tensor, n_seq: int, max_q_len: int, n_head: int,
                      n_kv_head: int, head_dim: int, page_size: int, scale: float, window: int = 0,
                      tcgen05: Optional[bool] = None, distance: Optional[torch.Tensor] = None, sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of the step's prompt portions over their pages (bfloat16, tensor cores).  `tcgen05`: None picks
    the tcgen05 kernel where it takes the shape and the rows are 16-byte aligned, else the mma.sync one.  `distance`: as for
    paged_attention_generic."""
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise invalid_argument("prefill attention takes bfloat16 only")
    if q.stride(1) != 1 or out.stride(1) != 1:
        raise invalid_argument("prefill attention: q and out must be dense within a row")
    if tcgen05 is None:
        # Measured on B200: the tcgen05 kernel walks a long tile's keys about 1.4x faster, but runs one block per SM,
        # so it wins while the launch is bound by its longest blocks (up to four blocks per SM) and loses to the
        # mma.sync kernel's several blocks per SM beyond that.
        blocks = n_seq * n_head * -(-max_q_len // 128)
        tcgen05 = (prefill_attention_tc_supports(n_head, n_kv_head, head_dim, page_size) and q.stride(0) % 8 == 0
                   and out.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0
                   and blocks <= 4 * _sm_count(q.device))
    if tcgen05:
        check(lib().lb_prefill_attention_tc_sink(
            _dev(q, "q"), q.stride(0), q.shape[0], _dev(cache, "cache"), cache.shape[0],
            _dev(q_start, "q_start", torch.int32), _dev(n_past, "n_past", torch.int32),
            _dev(block_table, "block_table", torch.int32), block_table.stride(0), _dev(out, "out"), out.stride(0), n_seq,
            max_q_len, n_head, n_kv_head, head_dim, page_size, float(scale), int(window), _distance(distance, n_head), _sink(sink, n_head), stream_ptr()),
            "prefill_attention_tc")
        return out
    check(lib().lb_prefill_attention_sink(
        _dev(q, "q"), q.stride(0), _dev(cache, "cache"), _dev(q_start, "q_start", torch.int32),
        _dev(n_past, "n_past", torch.int32), _dev(block_table, "block_table", torch.int32), block_table.stride(0),
        _dev(out, "out"), out.stride(0), n_seq, max_q_len, n_head, n_kv_head, head_dim, page_size, float(scale),
        int(window), _distance(distance, n_head), _sink(sink, n_head), stream_ptr()), "prefill_attention")
    return out


# ------------------------------------------------------------------ sampling

def sample(logits: torch.Tensor, n_rows: int, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           uniform: torch.Tensor, out_ids: torch.Tensor, out_probs: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token id per row; see csrc/sampling.cu for the distribution."""
    vocab = logits.shape[1]
    if logits.stride(1) != 1:
        raise invalid_argument("sample: logits must be dense within a row")
    if out_probs is not None and (not out_probs.is_contiguous() or out_probs.shape[1] != vocab):
        raise invalid_argument("sample: out_probs must be contiguous [rows, vocab]")
    check(lib().lb_sample(_dev(logits, "logits", torch.float32), logits.stride(0), n_rows, vocab,
                          _dev(temperature, "temperature", torch.float32), _dev(top_k, "top_k", torch.int32),
                          _dev(top_p, "top_p", torch.float32), _dev(uniform, "uniform", torch.float64),
                          _dev(out_ids, "out_ids", torch.int32), _opt(out_probs, "out_probs", torch.float32),
                          stream_ptr()), "sample")
    return out_ids


# ------------------------------------------------------------------ parallel blocks: norm in groups, token shift, xIELU, side input

for _name, _args in {
    "lb_rms_groups": [_i, _p, _l, _p, _p, _p, _l, _i, _i, _i, _f, _p],
    "lb_token_shift": [_i, _p, _l, _p, _p, _l, _p, _p, _p, _p, _i, _i, _i, _i, _p],
    "lb_rms_shift": [_i, _p, _l, _p, _p, _p, _l, _p, _l, _p, _p, _p, _p, _i, _i, _i, _i, _i, _f, _p],
    "lb_xielu": [_i, _p, _l, _i, _i, _p, _p],
    "lb_token_side": [_i, _p, _l, _p, _p, _p, _p, _p, _p, _i, _i, _i, _f, _p],
    "lb_latent_store": [_i, _p, _l, _p, _p, _p, _p, _p, _i, _i, _i, _i, _f, _p],
    "lb_rope_heads": [_i, _i, _p, _l, _p, _p, _p, _l, _i, _i, _i, _i, _i, _i, _p],
    "lb_head_matmul": [_i, _i, _i, _p, _l, _l, _p, _l, _l, _l, _p, _l, _l, _i, _i, _i, _i, _p],
    "lb_head_matmul_mma_supports": [_l, _l, _l, _l, _l, _l, _l, _i, _i],
    "lb_head_matmul_mma": [_i, _p, _l, _l, _p, _l, _l, _l, _p, _l, _l, _i, _i, _i, _i, _p],
    "lb_latent_attention": [_i, _p, _l, _p, _p, _p, _p, _i, _p, _l, _i, _i, _i, _i, _i, _f, _i, _p],
    "lb_latent_attention_mma_supports": [_i, _i, _i, _i],
    "lb_latent_attention_mma": [_p, _l, _p, _p, _p, _p, _i, _p, _l, _p, _p, _i, _i, _i, _i, _i, _i, _i, _f, _i, _i, _i, _p],
}.items():
    _SIGNATURES[_name] = _args


def rms_groups(x: torch.Tensor, weight: Optional[torch.Tensor], groups: int, eps: float, out: torch.Tensor,
               rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = x[rows[r]] (or x[r]) cut into `groups` equal parts, each over its own root mean square, times weight."""
    n = out.shape[0]
    check(lib().lb_rms_groups(_code(out.dtype, "out"), _dev(x, "x", torch.float32), x.stride(0), _opt(rows, "rows", torch.int32),
                              _opt(weight, "weight", torch.float32), _dev(out, "out"), out.stride(0), n, x.shape[1], groups, float(eps),
                              stream_ptr()), "rms_groups")
    return out


def token_shift(h: torch.Tensor, mix: torch.Tensor, out: torch.Tensor, state: torch.Tensor, tok_seq: torch.Tensor, q_start: torch.Tensor,
                slots: torch.Tensor, x: Optional[torch.Tensor] = None, weight: Optional[torch.Tensor] = None, groups: int = 1,
                eps: float = 0.0) -> torch.Tensor:
    """out[t] = h[t] + (h[t - 1] - h[t]) * mix with the row before a request's first row from `state` [slot, width] and its last
    row left there.  With `x` (float32 rows) and `weight`, h is made here as rms_groups(x) in the same launch."""
    T, S, width = h.shape[0], q_start.numel() - 1, h.shape[1]
    decode = 1 if T == S else 0
    layout = (_dev(tok_seq, "tok_seq", torch.int32), _dev(q_start, "q_start", torch.int32), _dev(slots, "slots", torch.int32))
    if x is None:
        check(lib().lb_token_shift(_code(h.dtype, "h"), _dev(h, "h"), h.stride(0), _dev(mix, "mix", torch.float32), _dev(out, "out", h.dtype),
                                   out.stride(0), _dev(state, "state", h.dtype), *layout, T, S, decode, width, stream_ptr()), "token_shift")
    else:
        check(lib().lb_rms_shift(_code(h.dtype, "h"), _dev(x, "x", torch.float32), x.stride(0), _dev(weight, "weight", torch.float32),
                                 _dev(mix, "mix", torch.float32), _dev(h, "h"), h.stride(0), _dev(out, "out", h.dtype), out.stride(0),
                                 _dev(state, "state", h.dtype), *layout, T, S, decode, width, groups, float(eps), stream_ptr()), "rms_shift")
    return out


def xielu(z: torch.Tensor, pq: torch.Tensor) -> torch.Tensor:
    """In place over the rows of z: z > 0 -> softplus(p) z^2 + z/2, else (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2."""
    check(lib().lb_xielu(_code(z.dtype, "z"), _dev(z, "z"), z.stride(0), z.shape[0], z.shape[1], _dev(pq, "pq", torch.float32), stream_ptr()), "xielu")
    return z


def token_side(x: torch.Tensor, tokens: torch.Tensor, table: torch.Tensor, gate: torch.Tensor, proj: torch.Tensor, weight: torch.Tensor,
               eps: float) -> torch.Tensor:
    """x[t] += rms(proj (gelu_tanh(gate x[t]) * table[tokens[t]])) * weight, in place (the kernels for steps of few tokens)."""
    T, width, dim = x.shape[0], x.shape[1], gate.shape[0]
    scratch = torch.empty(T * dim, dtype=torch.float32, device=x.device)
    check(lib().lb_token_side(_code(gate.dtype, "gate"), _dev(x, "x", torch.float32), x.stride(0), _dev(tokens, "tokens", torch.int32),
                              _dev(table, "table", gate.dtype), _dev(gate, "gate"), _dev(proj, "proj", gate.dtype), _dev(weight, "weight", torch.float32),
                              _dev(scratch, "scratch"), T, width, dim, float(eps), stream_ptr()), "token_side")
    return x


def latent_store(d: torch.Tensor, gain: torch.Tensor, freq: torch.Tensor, positions: torch.Tensor, slot_mapping: torch.Tensor, cache: torch.Tensor,
                 rank: int, rot: int, rot_dims: int, eps: float) -> None:
    """Row t of d (float32 [rank | rot]) -> the RMS-normed latent and the rotated key part, into the cache rows [slot, rank + rot]."""
    check(lib().lb_latent_store(_code(cache.dtype, "cache"), _dev(d, "d", torch.float32), d.stride(0), _dev(gain, "gain", torch.float32),
                                _dev(freq, "freq", torch.float32), _dev(positions, "positions", torch.int32),
                                _dev(slot_mapping, "slot_mapping", torch.int32), _dev(cache, "cache"), d.shape[0], rank, rot, rot_dims, float(eps),
                                stream_ptr()), "latent_store")


def rope_heads(q: torch.Tensor, freq: torch.Tensor, positions: torch.Tensor, wide: torch.Tensor, n_head: int, dim: int, rot: int, rot_dims: int,
               rank: int) -> torch.Tensor:
    """The rotated parts of the queries [T, H * (dim + rot)] (float32) into the wide queries [T, H * (rank + rot)]."""
    check(lib().lb_rope_heads(_code(q.dtype, "q"), _code(wide.dtype, "wide"), _dev(q, "q"), q.stride(0), _dev(freq, "freq", torch.float32),
                              _dev(positions, "positions", torch.int32), _dev(wide, "wide"), wide.stride(0), q.shape[0], n_head, dim, rot, rot_dims, rank,
                              stream_ptr()), "rope_heads")
    return wide


def head_matmul(a: torch.Tensor, a_head: int, b: torch.Tensor, b_head: int, b_k: int, b_n: int, c: torch.Tensor, c_head: int, n: int, k: int,
                n_head: int, tensor_cores: bool = False) -> torch.Tensor:
    """c[t, h * c_head + j] = sum_i a[t, h * a_head + i] * b.flat[h * b_head + i * b_k + j * b_n] for j < n, i < k, every head h."""
    m = a.shape[0]
    if tensor_cores:
        if not lib().lb_head_matmul_mma_supports(a.stride(0), a_head, b_head, b_k, b_n, c.stride(0), c_head, n, k):
            raise invalid_argument("head_matmul: the tensor-core kernel does not take these strides")
        check(lib().lb_head_matmul_mma(_code(a.dtype, "a"), _dev(a, "a"), a.stride(0), a_head, _dev(b, "b", torch.bfloat16), b_head, b_k, b_n,
                                       _dev(c, "c", torch.bfloat16), c.stride(0), c_head, m, n, k, n_head, stream_ptr()), "head_matmul_mma")
    else:
        check(lib().lb_head_matmul(_code(a.dtype, "a"), _code(b.dtype, "b"), _code(c.dtype, "c"), _dev(a, "a"), a.stride(0), a_head, _dev(b, "b"),
                                   b_head, b_k, b_n, _dev(c, "c"), c.stride(0), c_head, m, n, k, n_head, stream_ptr()), "head_matmul")
    return c


def latent_attention(wide: torch.Tensor, cache: torch.Tensor, tok_seq: torch.Tensor, positions: torch.Tensor, q_start: torch.Tensor,
                     n_past: torch.Tensor, block_table: torch.Tensor, out: torch.Tensor, n_head: int, rank: int, rot: int, page_size: int,
                     scale: float, window: int, tensor_cores: bool = False, n_splits: int = 1) -> torch.Tensor:
    """out[t, h, :rank] = softmax attention of the wide queries over the latent cache rows [slot, rank + rot] of the token's request.
    `tensor_cores`: the bfloat16 kernel (wide queries and cache bfloat16), optionally with every request's keys cut into n_splits parts."""
    T, S = wide.shape[0], q_start.numel() - 1
    if tensor_cores:
        if not lib().lb_latent_attention_mma_supports(n_head, rank, rot, page_size):
            raise invalid_argument("latent_attention: the tensor-core kernel does not take this shape")
        max_q = int((q_start[1:] - q_start[:-1]).max().item())
        part_o = torch.empty(max(1, n_splits * T * n_head * rank), dtype=torch.float32, device=wide.device)
        part_ml = torch.empty(max(1, n_splits * T * n_head * 2), dtype=torch.float32, device=wide.device)
        check(lib().lb_latent_attention_mma(_dev(wide, "wide", torch.bfloat16), wide.stride(0), _dev(cache, "cache", torch.bfloat16),
                                            _dev(q_start, "q_start", torch.int32), _dev(n_past, "n_past", torch.int32),
                                            _dev(block_table, "block_table", torch.int32), block_table.stride(0), _dev(out, "out", torch.float32),
                                            out.stride(0), _dev(part_o, "part_o"), _dev(part_ml, "part_ml"), T, S, max_q, n_head, rank, rot, page_size,
                                            float(scale), window, n_splits, 1, stream_ptr()), "latent_attention_mma")
    else:
        check(lib().lb_latent_attention(_code(cache.dtype, "cache"), _dev(wide, "wide", torch.float32), wide.stride(0), _dev(cache, "cache"),
                                        _dev(tok_seq, "tok_seq", torch.int32), _dev(positions, "positions", torch.int32),
                                        _dev(block_table, "block_table", torch.int32), block_table.stride(0), _dev(out, "out", torch.float32),
                                        out.stride(0), T, n_head, rank, rot, page_size, float(scale), window, stream_ptr()), "latent_attention")
    return out


# ---- gated mixers, matrix memories, routed experts -----------------------------------------------------------------
for _name, _args in {
    "lb_rms_groups_offset": [_i, _p, _l, _p, _p, _f, _p, _l, _i, _i, _i, _f, _p],
    "lb_add_row": [_p, _l, _p, _i, _i, _p],
    "lb_rms_sum_add": [_p, _l, _i, _p, _p, _p, _i, _i, _f, _f, _p],
    "lb_rms_sum_add_rounded": [_p, _l, _i, _p, _p, _p, _i, _i, _f, _f, _p, _l, _p],
    "lb_qk_norm_store": [_i, _p, _l, _i, _i, _i, _p, _p, _p, _l, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _f, _p],
    "lb_head_gate": [_i, _i, _p, _l, _i, _p, _l, _p, _p, _l, _i, _i, _i, _i, _i, _f, _p],
    "lb_gated_act": [_i, _p, _l, _p, _l, _i, _i, _i, _p],
    "lb_matrix_memory": [_p, _p, _p, _p, _p, _l, _p, _p, _i, _p, _p, _p, _p, _l, _p, _l, _i, _i, _i, _i, _i, _f, _f, _f, _i, _p],
    "lb_matrix_memory_pieces": [_p, _p, _p, _p, _p, _l, _p, _p, _i, _p, _p, _p, _p, _l, _p, _l, _i, _i, _i, _i, _i, _i, _f, _f, _f, _p, _p],
    "lb_matrix_memory_shared": [_p, _p, _p, _p, _p, _l, _p, _p, _i, _p, _p, _p, _p, _l, _p, _l, _i, _i, _i, _i, _i, _f, _f, _f, _i, _i, _p],
    "lb_matrix_memory_pieces_shared": [_p, _p, _p, _p, _p, _l, _p, _p, _i, _p, _p, _p, _p, _l, _p, _l, _i, _i, _i, _i, _i, _i, _f, _f, _f, _p, _i, _p],
    "lb_matrix_memory_activated": [_p, _p, _p, _p, _p, _l, _p, _p, _i, _p, _p, _p, _p, _l, _p, _l, _i, _i, _i, _i, _i, _f, _f, _f, _i, _i, _i, _p],
    "lb_matrix_memory_pieces_activated": [_p, _p, _p, _p, _p, _l, _p, _p, _i, _p, _p, _p, _p, _l, _p, _l, _i, _i, _i, _i, _i, _i, _f, _f, _f, _p, _i, _i, _p],
    "lb_router_topk": [_i, _p, _l, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p],
    "lb_expert_plan": [_p, _i, _i, _p, _p, _p, _p],
    "lb_expert_product": [_i, _i, _p, _l, _p, _l, _p, _p, _p, _p, _l, _i, _i, _i, _i, _i, _i, _p],
    "lb_expert_product_set_plain": [_i],
    "lb_expert_combine": [_p, _l, _p, _l, _p, _i, _i, _i, _p],
}.items():
    _SIGNATURES[_name] = _args

GATES = {"sigmoid": 0, "silu": 1, "gelu_tanh": 2}


def rms_offset(x: torch.Tensor, weight: torch.Tensor, gain_offset: float, eps: float, out: torch.Tensor) -> torch.Tensor:
    """out[r] = x[r] / sqrt(mean(x[r]^2) + eps) * (gain_offset + weight)."""
    check(lib().lb_rms_groups_offset(_code(out.dtype, "out"), _dev(x, "x", torch.float32), x.stride(0), None, _dev(weight, "weight", torch.float32),
                                     float(gain_offset), _dev(out, "out"), out.stride(0), out.shape[0], x.shape[1], 1, float(eps), stream_ptr()), "rms_groups_offset")
    return out


def add_row(x: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    check(lib().lb_add_row(_dev(x, "x", torch.float32), x.stride(0), _dev(v, "v", torch.float32), x.shape[0], x.shape[1], stream_ptr()), "add_row")
    return x


def rms_sum_add(x: torch.Tensor, branches, weights, scale: float, eps: float, rounded: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x[r] += scale * sum_i rms(branches[i][r]) * weights[i] (float32 rows; a weight may be None); with `rounded` (bfloat16 rows) the new rows of
    x are left there as well."""
    n = len(branches)
    ys = (_c.c_void_p * n)(*[_dev(y, "branch", torch.float32) for y in branches])
    ld = (_c.c_int64 * n)(*[y.stride(0) for y in branches])
    ws = (_c.c_void_p * n)(*[_opt(w, "weight", torch.float32) for w in weights])
    check(lib().lb_rms_sum_add_rounded(_dev(x, "x", torch.float32), x.stride(0), n, ys, ld, ws, x.shape[0], x.shape[1], float(scale), float(eps),
                                       _opt(rounded, "rounded", torch.bfloat16), rounded.stride(0) if rounded is not None else 0, stream_ptr()), "rms_sum_add")
    return x


def qk_norm_store(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                  q_out: torch.Tensor, cache: Optional[torch.Tensor], slot_mapping: torch.Tensor, n_head: int, n_kv_head: int, dim: int, vdim: int,
                  padded: int, page_size: int, norm: bool, eps: float) -> torch.Tensor:
    """Queries, keys and values of the float rows `proj` (see csrc/api.h): normalised per head, padded to `padded` values, keys and values
    into the cache pages [page, K|V, kv_head, slot, padded]."""
    check(lib().lb_qk_norm_store(_code(q_out.dtype, "q_out"), _dev(proj, "proj", torch.float32), proj.stride(0), q_off, k_off, v_off,
                                 _opt(q_weight, "q_weight", torch.float32), _opt(k_weight, "k_weight", torch.float32), _dev(q_out, "q_out"), q_out.stride(0),
                                 _opt(cache, "cache", q_out.dtype), _dev(slot_mapping, "slot_mapping", torch.int32), proj.shape[0], n_head, n_kv_head, dim, vdim,
                                 padded, page_size, int(norm), float(eps), stream_ptr()), "qk_norm_store")
    return q_out


def head_gate(o: torch.Tensor, o_head: int, g: Optional[torch.Tensor], gain: Optional[torch.Tensor], out: torch.Tensor, n_head: int, vdim: int, norm: bool,
              gate: str, eps: float) -> torch.Tensor:
    """out[t, h, :] = (o[t, h, :vdim] over its root mean square when `norm`) * gain * gate(g[t, h, :])."""
    check(lib().lb_head_gate(_code(o.dtype, "o"), _code(out.dtype, "out"), _dev(o, "o"), o.stride(0), o_head, _opt(g, "g", torch.float32),
                             g.stride(0) if g is not None else 0, _opt(gain, "gain", torch.float32), _dev(out, "out"), out.stride(0), o.shape[0], n_head, vdim,
                             int(norm), GATES[gate], float(eps), stream_ptr()), "head_gate")
    return out


def gated_act(gu: torch.Tensor, out: torch.Tensor, gate: str) -> torch.Tensor:
    check(lib().lb_gated_act(_code(out.dtype, "out"), _dev(gu, "gu", torch.float32), gu.stride(0), _dev(out, "out"), out.stride(0), gu.shape[0], out.shape[1],
                             GATES[gate], stream_ptr()), "gated_act")
    return out


_QKV_ACT = {None: -1, "sigmoid": 0, "silu": 1, "gelu_tanh": 2, "relu": 3}


def memory_slot_floats(n_head: int, dim: int, vdim: int, value_tile: int) -> int:
    return n_head * ((vdim + value_tile - 1) // value_tile) * (dim * value_tile + dim + 1)


def matrix_memory(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, zi_off: Optional[int], zf_off: Optional[int], decay: Optional[torch.Tensor],
                  freq: Optional[torch.Tensor], rot_dims: int, positions: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor, state: torch.Tensor,
                  out: torch.Tensor, n_head: int, dim: int, vdim: int, value_tile: int, q_scale: float, k_scale: float, cap: float, chunked: bool,
                  qk_share: int = 1, qkv_act: Optional[str] = None) -> torch.Tensor:
    """The matrix memories of csrc/matrix_memory.cu over the float rows `proj` whose columns hold q, k, v (and the gates' pre-activations) at the
    given offsets; state [slots, memory_slot_floats(..)] float32.  Without `decay` and without `zi_off` the column `zf_off` holds the log of the
    factor a token and head; `qk_share` heads in a row read one query and key; `qkv_act` (sigmoid, silu, gelu_tanh, relu) acts on q, k and v as they are read."""
    base = _dev(proj, "proj", torch.float32)
    at = lambda off: None if off is None else base + 4 * off
    check(lib().lb_matrix_memory_activated(at(q_off), at(k_off), at(v_off), at(zi_off), at(zf_off), proj.stride(0), _opt(decay, "decay", torch.float32),
                                 _opt(freq, "freq", torch.float32), rot_dims, _dev(positions, "positions", torch.int32), _dev(q_start, "q_start", torch.int32),
                                 _dev(slots, "slots", torch.int32), _dev(state, "state", torch.float32), state.stride(0), _dev(out, "out", torch.float32),
                                 out.stride(0), q_start.numel() - 1, n_head, dim, vdim, value_tile, float(q_scale), float(k_scale), float(cap), int(chunked),
                                 int(qk_share), _QKV_ACT[qkv_act], stream_ptr()), "matrix_memory")
    return out


def matrix_memory_pieces(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, zi_off: Optional[int], zf_off: Optional[int], decay: Optional[torch.Tensor],
                         freq: Optional[torch.Tensor], rot_dims: int, positions: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor, state: torch.Tensor,
                         out: torch.Tensor, n_head: int, dim: int, vdim: int, value_tile: int, q_scale: float, k_scale: float, cap: float,
                         qk_share: int = 1, qkv_act: Optional[str] = None) -> torch.Tensor:
    """matrix_memory in its form for long portions: every piece of 32 rows a block of its own (three launches)."""
    base = _dev(proj, "proj", torch.float32)
    at = lambda off: None if off is None else base + 4 * off
    T, S = proj.shape[0], q_start.numel() - 1
    fn = lib().lb_matrix_memory_pieces_floats
    fn.argtypes, fn.restype = [_i] * 6, _c.c_int64
    scratch = torch.empty(int(fn(T, S, n_head, dim, vdim, value_tile)), dtype=torch.float32, device=proj.device)
    check(lib().lb_matrix_memory_pieces_activated(at(q_off), at(k_off), at(v_off), at(zi_off), at(zf_off), proj.stride(0), _opt(decay, "decay", torch.float32),
                                        _opt(freq, "freq", torch.float32), rot_dims, _dev(positions, "positions", torch.int32),
                                        _dev(q_start, "q_start", torch.int32), _dev(slots, "slots", torch.int32), _dev(state, "state", torch.float32),
                                        state.stride(0), _dev(out, "out", torch.float32), out.stride(0), T, S, n_head, dim, vdim, value_tile, float(q_scale),
                                        float(k_scale), float(cap), _dev(scratch, "scratch"), int(qk_share), _QKV_ACT[qkv_act], stream_ptr()), "matrix_memory_pieces")
    return out


def routed_experts(h: torch.Tensor, router: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, x: torch.Tensor, top: int, gate: str = "silu",
                   softmax: bool = False, renormalise: bool = False, plain: bool = False):
    """x[t] += sum over row t's `top` experts e of down_e (gate(W_gate_e a) * (W_up_e a)), a = score * h[t]: the router, the plan, the experts' two
    products and the sum, as the feed-forward part launches them.  gate_up [E, 2 inner, width], down [E, width, inner].  `plain`: bfloat16 products
    on the 32-bit units.  Returns (ids, weights) [T, top]."""
    T, width = h.shape
    E, inner = gate_up.shape[0], gate_up.shape[1] // 2
    dev = h.device
    ids = torch.empty(T, top, dtype=torch.int32, device=dev)
    weights = torch.empty(T, top, dtype=torch.float32, device=dev)
    place = torch.empty(T * top, dtype=torch.int32, device=dev)
    pair_at = torch.empty(T * top, dtype=torch.int32, device=dev)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
    mid = torch.empty(T * top, inner, dtype=h.dtype, device=dev)
    y = torch.empty(T * top, width, dtype=torch.float32, device=dev)
    s = stream_ptr()
    check(lib().lb_router_topk(_code(h.dtype, "h"), _dev(h, "h"), h.stride(0), _dev(router, "router", h.dtype), _dev(ids, "ids"), _dev(weights, "weights"), T, E,
                               width, top, int(softmax), int(renormalise), s), "router_topk")
    check(lib().lb_expert_plan(_dev(ids, "ids"), T * top, E, _dev(offsets, "offsets"), _dev(place, "place"), _dev(pair_at, "pair_at"), s), "expert_plan")
    lib().lb_expert_product_set_plain(int(plain))
    try:
        check(lib().lb_expert_product(_code(h.dtype, "h"), 1, _dev(h, "h"), h.stride(0), _dev(gate_up, "gate_up", h.dtype), 2 * inner * width, _dev(offsets, "offsets"),
                                      _dev(pair_at, "pair_at"), _dev(weights, "weights"), _dev(mid, "mid"), mid.stride(0), T * top, E, inner, width, top, GATES[gate], s),
              "expert_product")
        check(lib().lb_expert_product(_code(h.dtype, "h"), 0, _dev(mid, "mid"), mid.stride(0), _dev(down, "down", h.dtype), width * inner, _dev(offsets, "offsets"),
                                      _dev(pair_at, "pair_at"), _dev(weights, "weights"), _dev(y, "y"), y.stride(0), T * top, E, width, inner, top, GATES[gate], s),
              "expert_product")
    finally:
        lib().lb_expert_product_set_plain(0)
    check(lib().lb_expert_combine(_dev(x, "x", torch.float32), x.stride(0), _dev(y, "y"), y.stride(0), _dev(place, "place"), T, width, top, s), "expert_combine")
    return ids, weights


# ---- a sinusoid of the position, a gated norm in groups, gates with a cap, a router with a bias ---------------------------------------
for _name, _args in {
    "lb_embed_sinusoid": [_i, _p, _p, _p, _p, _p, _p, _i, _i, _f, _f, _p],
    "lb_gated_group_norm": [_i, _p, _l, _p, _l, _p, _i, _p, _l, _p, _p, _l, _i, _i, _i, _f, _p],
    "lb_gated_act_kind": [_i, _p, _l, _p, _l, _i, _i, _i, _f, _f, _p],
    "lb_router_topk_biased": [_i, _p, _l, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p],
    "lb_ssm_prepare": [_p, _l, _i, _i, _p, _p, _p, _p, _p, _l, _p, _p, _p, _p, _l, _i, _i, _i, _i, _i, _i, _i, _p],
}.items():
    _SIGNATURES[_name] = _args

GATE_KINDS = {"sigmoid": 0, "silu": 1, "gelu_tanh": 2, "relu": 3, "capped": 4}


def embed_sinusoid(tokens: torch.Tensor, positions: torch.Tensor, table: torch.Tensor, base: float, gain: Optional[torch.Tensor], x: torch.Tensor,
                   scale: float = 1.0, eps: float = 1e-6) -> torch.Tensor:
    """x[t] = table[tokens[t]] * scale + e(positions[t]), e[2i] = sin(p w_i), e[2i+1] = cos(p w_i), w_i = base^(-2i / width); with `gain` the row
    is then divided by its root mean square and multiplied by it.  The frequencies are made in double precision and passed as two floats each."""
    width = table.shape[1]
    w = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * torch.arange((width + 1) // 2, dtype=torch.float64) / width)
    hi = w.to(torch.float32)
    freq2 = torch.stack([hi, (w - hi.to(torch.float64)).to(torch.float32)], dim=1).contiguous().to(x.device)
    check(lib().lb_embed_sinusoid(_code(table.dtype, "table"), _dev(tokens, "tokens", torch.int32), _dev(positions, "positions", torch.int32),
                                  _dev(table, "table"), _dev(freq2, "freq2"), _opt(gain, "gain", torch.float32), _dev(x, "x", torch.float32), tokens.numel(),
                                  width, float(scale), float(eps), stream_ptr()), "embed_sinusoid")
    return x


def gated_group_norm(o: torch.Tensor, skip: Optional[torch.Tensor], skip_gain: Optional[torch.Tensor], head: int, z: Optional[torch.Tensor],
                     weight: Optional[torch.Tensor], out: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """out = (o + skip_gain[column / head] * skip) * silu(z), cut into `groups` equal parts each over its own root mean square, times weight."""
    check(lib().lb_gated_group_norm(_code(out.dtype, "out"), _dev(o, "o", torch.float32), o.stride(0), _opt(skip, "skip", torch.float32),
                                    skip.stride(0) if skip is not None else 0, _opt(skip_gain, "skip_gain", torch.float32), head,
                                    _opt(z, "z", torch.float32), z.stride(0) if z is not None else 0, _opt(weight, "weight", torch.float32), _dev(out, "out"),
                                    out.stride(0), o.shape[0], o.shape[1], groups, float(eps), stream_ptr()), "gated_group_norm")
    return out


def gated_act_kind(gu: torch.Tensor, out: torch.Tensor, gate: str, alpha: float = 0.0, limit: float = 0.0) -> torch.Tensor:
    """out = gate(gu[:, :inner]) * gu[:, inner:]; "capped": g' = min(g, limit), u' = clamp(u, -limit, limit), g' sigmoid(alpha g') (u' + 1)."""
    inner = gu.shape[1] // 2
    check(lib().lb_gated_act_kind(_code(out.dtype, "out"), _dev(gu, "gu", torch.float32), gu.stride(0), _dev(out, "out"), out.stride(0), gu.shape[0], inner,
                                  GATE_KINDS[gate], float(alpha), float(limit), stream_ptr()), "gated_act")
    return out


def router_topk(h: torch.Tensor, router: torch.Tensor, bias: Optional[torch.Tensor], top: int, softmax: bool, renormalise: bool):
    """The `top` largest of router h + bias per row (32-bit sums, ties to the lower expert) and their weights.  Returns (ids, weights) [T, top]."""
    T, width = h.shape
    ids = torch.empty(T, top, dtype=torch.int32, device=h.device)
    weights = torch.empty(T, top, dtype=torch.float32, device=h.device)
    check(lib().lb_router_topk_biased(_code(h.dtype, "h"), _dev(h, "h"), h.stride(0), _dev(router, "router", h.dtype), _opt(bias, "bias", torch.float32),
                                      _dev(ids, "ids"), _dev(weights, "weights"), T, router.shape[0], width, top, int(softmax), int(renormalise), stream_ptr()),
          "router_topk")
    return ids, weights


def ssm_prepare(proj: torch.Tensor, xbc_off: int, dt_off: int, taps: torch.Tensor, tap_bias: Optional[torch.Tensor], dt_bias: Optional[torch.Tensor],
                a_log: torch.Tensor, state: torch.Tensor, tok_seq: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor, out: torch.Tensor,
                n_head: int, vdim: int, group_values: int, decode_only: bool) -> torch.Tensor:
    """The rows a state space's recurrence reads (csrc/state_space.cu) from the float rows `proj`: the channels at `xbc_off` through their causal
    convolution (`taps` [channels, K], the last K - 1 inputs of every request in `state` [slots, (K - 1) x channels]) and SiLU, the steps at `dt_off`
    through softplus; out [T, 2 x n_head x vdim + group_values + n_head].  `decode_only`: every request brings one row."""
    check(lib().lb_ssm_prepare(_dev(proj, "proj", torch.float32), proj.stride(0), xbc_off, dt_off, _dev(taps, "taps", torch.float32),
                               _opt(tap_bias, "tap_bias", torch.float32), _opt(dt_bias, "dt_bias", torch.float32), _dev(a_log, "a_log", torch.float32),
                               _dev(state, "state", torch.float32), state.stride(0), _dev(tok_seq, "tok_seq", torch.int32),
                               _dev(q_start, "q_start", torch.int32), _dev(slots, "slots", torch.int32), _dev(out, "out", torch.float32), out.stride(0),
                               proj.shape[0], q_start.numel() - 1, n_head, vdim, group_values, taps.shape[1], int(decode_only), stream_ptr()), "ssm_prepare")
    return out


# ------------------------------------------------------------------ rows around rotated attention, norms over all heads, experts by table

def qkv_rotary_store(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                     q_out: torch.Tensor, cache: Optional[torch.Tensor], slot_mapping: torch.Tensor, n_head: int, n_kv_head: int, dim: int, vdim: int,
                     padded: int, page_size: int, norm_mode: int, eps: float, positions: torch.Tensor, freq: Optional[torch.Tensor], rot_dims: int,
                     v_first_in: Optional[torch.Tensor] = None, v_first_out: Optional[torch.Tensor] = None, blend: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Queries, keys and values of a float projection on their way to attention: norm_mode 0 none, 1 a head, 2 the whole projection; the first
    rot_dims values of every head rotated by positions[t] * freq[i]; values blended with v_first_in by blend[0], or left in v_first_out."""
    shared = v_first_in if v_first_in is not None else v_first_out
    check(lib().lb_qkv_rotary_store(_code(q_out.dtype, "q_out"), _dev(proj, "proj", torch.float32), proj.stride(0), q_off, k_off, v_off,
                                    _opt(q_weight, "q_weight", torch.float32), _opt(k_weight, "k_weight", torch.float32), _dev(q_out, "q_out"), q_out.stride(0),
                                    _opt(cache, "cache", q_out.dtype), _dev(slot_mapping, "slot_mapping", torch.int32), proj.shape[0], n_head, n_kv_head, dim, vdim,
                                    padded, page_size, norm_mode, float(eps), _dev(positions, "positions", torch.int32), _opt(freq, "freq", torch.float32), rot_dims,
                                    _opt(v_first_in, "v_first_in", torch.float32), _opt(v_first_out, "v_first_out", torch.float32),
                                    shared.stride(0) if shared is not None else 0, _opt(blend, "blend", torch.float32), stream_ptr()), "qkv_rotary_store")
    return q_out


def row_norm_gate(o: torch.Tensor, g: Optional[torch.Tensor], gain: Optional[torch.Tensor], out: torch.Tensor, gate: str, eps: float) -> torch.Tensor:
    """out = o over the root mean square of the whole row, times gain, times gate(g) (sigmoid or silu)."""
    check(lib().lb_row_norm_gate(_code(out.dtype, "out"), _dev(o, "o", torch.float32), o.stride(0), _opt(g, "g", torch.float32), g.stride(0) if g is not None else 0,
                                 _opt(gain, "gain", torch.float32), _dev(out, "out"), out.stride(0), o.shape[0], o.shape[1], {"sigmoid": 0, "silu": 1}[gate],
                                 float(eps), stream_ptr()), "row_norm_gate")
    return out


def activate_columns(x: torch.Tensor, cols: int, gate: str) -> torch.Tensor:
    """In place over the first `cols` columns of the float rows x: sigmoid, silu, gelu_tanh or relu."""
    check(lib().lb_activate_columns(_dev(x, "x", torch.float32), x.stride(0), x.shape[0], cols, {"sigmoid": 0, "silu": 1, "gelu_tanh": 2, "relu": 3}[gate],
                                    stream_ptr()), "activate_columns")
    return x


def router_table(tokens: torch.Tensor, table: torch.Tensor, n_experts: int):
    """(ids [T, top] int32, weights [T, top] float32): the experts of every row from the table's row of its token id, each weighing 1 / top."""
    T, top = tokens.shape[0], table.shape[1]
    ids = torch.empty(T, top, dtype=torch.int32, device=tokens.device)
    weights = torch.empty(T, top, dtype=torch.float32, device=tokens.device)
    check(lib().lb_router_table(_dev(tokens, "tokens", torch.int32), _dev(table, "table", torch.int32), _dev(ids, "ids"), _dev(weights, "weights"), T, top,
                                n_experts, table.shape[0], stream_ptr()), "router_table")
    return ids, weights
