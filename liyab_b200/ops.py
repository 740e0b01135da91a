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
ACTIVATIONS = {"none": 0, "gelu_tanh": 1, "gelu_erf": 2}
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
                            head_dim: int, page_size: int, scale: float, window: int = 0) -> torch.Tensor:
    """Causal attention of the step's tokens over their requests' pages, 32-bit arithmetic."""
    if q.dtype != cache.dtype or out.dtype != cache.dtype:
        raise invalid_argument("attention: q, cache and out must have one element type")
    if q.stride(1) != 1 or out.stride(1) != 1:
        raise invalid_argument("attention: q and out must be dense within a row")
    check(lib().lb_paged_attention_generic(
        _code(cache.dtype, "cache"), _dev(q, "q"), q.stride(0), _dev(cache, "cache"),
        _dev(tok_seq, "tok_seq", torch.int32), _dev(positions, "positions", torch.int32),
        _dev(block_table, "block_table", torch.int32), block_table.stride(0), _dev(out, "out"), out.stride(0),
        n_tokens, n_head, n_kv_head, head_dim, page_size, float(scale), int(window), stream_ptr()),
        "paged_attention_generic")
    return out


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
                     n_splits: int, tensor_cores: Optional[bool] = None) -> torch.Tensor:
    """Attention of one new token per request over its pages (bfloat16), keys split `n_splits` ways.
    `tensor_cores`: None picks the tensor-core kernel where it takes the shape, else the scalar one."""
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
    fn = lib().lb_decode_attention_mma if tensor_cores else lib().lb_decode_attention
    check(fn(
        _dev(q, "q"), q.stride(0), *cache_args, _dev(positions, "positions", torch.int32),
        _dev(block_table, "block_table", torch.int32), block_table.stride(0), _dev(out, "out"), out.stride(0),
        _opt(partial, "partial", torch.float32), _opt(counters, "counters", torch.int32), n_seq, n_head, n_kv_head,
        head_dim, page_size, float(scale), int(window), int(n_splits), stream_ptr()), "decode_attention")
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
                      tcgen05: Optional[bool] = None) -> torch.Tensor:
    """Attention of the step's prompt portions over their pages (bfloat16, tensor cores).  `tcgen05`: None picks
    the tcgen05 kernel where it takes the shape and the rows are 16-byte aligned, else the mma.sync one."""
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
        check(lib().lb_prefill_attention_tc(
            _dev(q, "q"), q.stride(0), q.shape[0], _dev(cache, "cache"), cache.shape[0],
            _dev(q_start, "q_start", torch.int32), _dev(n_past, "n_past", torch.int32),
            _dev(block_table, "block_table", torch.int32), block_table.stride(0), _dev(out, "out"), out.stride(0), n_seq,
            max_q_len, n_head, n_kv_head, head_dim, page_size, float(scale), int(window), stream_ptr()), "prefill_attention_tc")
        return out
    check(lib().lb_prefill_attention(
        _dev(q, "q"), q.stride(0), _dev(cache, "cache"), _dev(q_start, "q_start", torch.int32),
        _dev(n_past, "n_past", torch.int32), _dev(block_table, "block_table", torch.int32), block_table.stride(0),
        _dev(out, "out"), out.stride(0), n_seq, max_q_len, n_head, n_kv_head, head_dim, page_size, float(scale),
        int(window), stream_ptr()), "prefill_attention")
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
