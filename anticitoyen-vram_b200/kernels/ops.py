"""Python faces of the CUDA kernels (ctypes over the C entry points of ``csrc/``).

Each function takes torch CUDA tensors, checks what the kernel assumes (device,
dtype, contiguity) and launches on the current stream.  There is no other
implementation behind these names: without the compiled library, or without a
CUDA device, the first call raises.
"""

from __future__ import annotations

import ctypes
import functools
from ctypes import c_float, c_int, c_void_p

import torch

from .build import BuildError, library_path

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

_ERRORS = {
    -2: "unsupported element type",
    -3: "a size is outside what this kernel takes",
    -4: "a pointer or stride is not aligned as this kernel needs",
    -5: "scratch memory is too small",
}


class KernelError(RuntimeError):
    pass


_lib = None
_cudart_err = None


def library() -> ctypes.CDLL:
    """Load (building on first use) the kernel library; raise if it cannot be had."""
    global _lib
    if _lib is None:
        try:
            path = library_path()
        except BuildError as exc:
            raise KernelError(f"the CUDA kernels of acvram_b200 could not be built: {exc}") from exc
        lib = ctypes.CDLL(path)
        _declare(lib)
        _lib = lib
    return _lib


def set_programmatic_launch(classes: int | bool) -> None:
    """Which kernel classes are launched so that they may begin while their predecessor finishes
    (bit set: 1 matrix product, 2 norm, 4 rope/append, 8 decode attention, 16 SwiGLU, 32 the rest;
    True = the default set, False = none)."""
    if classes is True:
        classes = 0x3f
    library().acv_set_pdl(int(classes))


def loaded_library_path() -> str | None:
    return None if _lib is None else _lib._name


def _declare(lib: ctypes.CDLL) -> None:
    P, I, F, LL = c_void_p, c_int, c_float, ctypes.c_longlong
    sig = {
        "acv_embed": [P, P, P, I, I, I, I, P],
        "acv_add_rmsnorm": [P, P, P, P, P, I, I, F, I, P],
        "acv_swiglu": [P, P, I, I, I, P],
        "acv_add_bias": [P, I, P, I, I, I, P],
        "acv_qk_norm_rope_append": [P, I, I, I, I, I, P, P, F, P, I, I, P, P, P, I, P, P, P, I, I, I, P],
        "acv_attention_generic": [P, I, P, I, P, P, P, P, P, I, P, I, I, I, I, I, I, F, I, I, P],
        "acv_gemm_simt": [P, I, P, I, P, I, I, I, I, I, I, P],
        "acv_gemm_tc_qkv": [P, I, P, I, P, I, I, I, I, I, I, I, P, LL, P, LL, P, I, I, I, I, I, I, P, P, F, P, I, P, P, P, I, P, P, P, I, I, P],
        "acv_gemm_tc": [P, I, P, I, P, I, I, I, I, I, I, I, I, I, P, LL, P, LL, P, I, I, I, P],
        "acv_attention_decode": [P, I, P, I, P, P, P, P, I, P, P, I, P, I, I, I, I, I, F, I, I, P, P, P, LL, LL, LL, I, I, P],
        "acv_attention_tc": [P, I, I, P, I, P, P, P, P, I, P, P, P, I, P, I, I, I, I, I, F, I, P, P],
        "acv_attention_chunk": [P, I, P, I, P, P, P, P, I, P, P, P, I, P, I, I, I, I, I, F, I, I, P],
        "acv_table_update": [P, I, I, P, I, P],
        "acv_argmax": [P, I, I, I, P, P],
        "acv_apply_penalties": [P, I, I, P, P, P, I, P, P, P, P],
        "acv_sample": [P, I, I, I, P, P, P, P, P, P, P, P, P],
        "acv_top_logprobs": [P, I, I, I, I, P, P, P],
    }
    for name, args in sig.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = c_int
    lib.acv_set_pdl.argtypes = [c_int]
    lib.acv_set_pdl.restype = None
    lib.acv_decode_layer.argtypes = [ctypes.POINTER(DecodeLayerArgs), P]
    lib.acv_decode_layer.restype = c_int
    lib.acv_decode_layer_takes.argtypes = [I] * 8
    lib.acv_decode_layer_takes.restype = c_int
    lib.acv_attention_decode_resident.argtypes = [I] * 9
    lib.acv_attention_decode_resident.restype = c_int
    lib.acv_random_normal.argtypes = [P, LL, ctypes.c_ulonglong, F, F, P, P, I, P]
    lib.acv_random_normal.restype = c_int
    lib.acv_random_int.argtypes = [P, LL, ctypes.c_ulonglong, ctypes.c_uint, P]
    lib.acv_random_int.restype = c_int
    lib.acv_gemm_tc_test_fault.argtypes = [c_int, c_int]
    lib.acv_gemm_tc_test_fault.restype = None


class DecodeLayerArgs(ctypes.Structure):
    """The arguments of ``acv_decode_layer`` (csrc/decode_layer.cu, ``DlLayerArgs``), field for field."""
    _P, _I, _F, _LL = c_void_p, c_int, c_float, ctypes.c_longlong
    _fields_ = [
        ("T", _I), ("H", _I), ("I", _I), ("NH", _I), ("NKV", _I), ("D", _I),
        ("eps", _F), ("qk_eps", _F), ("scale", _F),
        ("x", _P), ("delta_in", _P), ("w_norm1", _P), ("w_norm2", _P),
        ("w_qkv", _P), ("w_o", _P), ("w_gu", _P), ("w_down", _P),
        ("q_norm", _P), ("k_norm", _P), ("cos_sin", _P), ("table_rows", _I),
        ("positions", _P), ("seq_of_token", _P), ("kv_len", _P),
        ("block_table", _P), ("bt_stride", _I), ("bt_rows", _P),
        ("k_pages", _P), ("v_pages", _P), ("page_size", _I), ("num_pages", _I),
        ("h", _P), ("qkv", _P), ("attn_out", _P), ("a_out", _P), ("act", _P), ("delta_out", _P),
        ("workspace", _P), ("workspace_floats", _LL), ("counters", _P), ("n_counters", _LL),
        ("part", _P), ("part_floats", _LL), ("att_counters", _P), ("n_att_counters", _LL),
        ("bars", _P), ("status", _P),
        ("sm_count", _I), ("max_kv", _I), ("trace", _P),
    ]


LAUNCHES = 0   # kernels of this package launched so far (library matrix products are not counted)


def _check(code: int, name: str) -> None:
    global LAUNCHES
    if code == 0:
        LAUNCHES += 1
        return
    if code < 0:
        raise KernelError(f"{name}: {_ERRORS.get(code, f'refused with code {code}')}")
    raise KernelError(f"{name}: CUDA error {code} ({_cuda_error_text(code)})")


def _cuda_error_text(code: int) -> str:
    """The runtime's own words for a cudaError_t, asked of the library that the kernels are linked against."""
    try:
        fn = ctypes.CDLL("libcudart.so.12").cudaGetErrorString
        fn.restype = ctypes.c_char_p
        fn.argtypes = [ctypes.c_int]
        return fn(code).decode()
    except Exception:       # no such library name on this system: the number has to do
        return "see cudaError_t"


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DT[dtype]
    except KeyError:
        raise KernelError(f"element type {dtype} is not built (float32 and bfloat16 are)") from None


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("acvram_b200 kernels run on a CUDA device only; got a CPU tensor")


# ----------------------------------------------------------------------------- elementwise
def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] = table[tokens[t]].  table [V, H]; tokens int32 [T]; out [T, H]."""
    _need_cuda(table, tokens, out)
    T, H = out.shape
    _check(library().acv_embed(_p(table), _p(tokens), _p(out), T, H, table.shape[0], dtype_code(table.dtype),
                               _stream()), "embed")
    return out


def add_rmsnorm(x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float, out: torch.Tensor,
                rows: torch.Tensor | None = None) -> torch.Tensor:
    """x += delta (in place, when delta is given); out = rmsnorm(x) * weight.

    With ``rows`` (int32 [R]) only those rows are normed, into out[0..R), and x is
    left as it is.  weight is float32 [H]."""
    _need_cuda(x, out, weight)
    n = out.shape[0] if rows is not None else x.shape[0]
    _check(library().acv_add_rmsnorm(_p(x), _p(delta), _p(weight), _p(out), _p(rows), n, x.shape[-1], eps,
                                     dtype_code(x.dtype), _stream()), "add_rmsnorm")
    return out


def add_bias(out: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """out[t, n] += bias[n] in place (bias float32 [N]; the sum in float, rounded once to out's type)."""
    _need_cuda(out, bias)
    if bias.dtype != torch.float32 or bias.numel() != out.shape[1] or out.stride(1) != 1:
        raise KernelError("add_bias: a float32 bias of the output's width is wanted")
    _check(library().acv_add_bias(_p(out), out.stride(0), _p(bias), out.shape[0], out.shape[1], dtype_code(out.dtype),
                                  _stream()), "add_bias")
    return out


def table_update(table: torch.Tensor, triples: torch.Tensor, n: int) -> None:
    """table[row, column] = page for the first ``n`` (row, column, page) triples of ``triples`` (int32, on the device)."""
    _need_cuda(table, triples)
    if table.dtype != torch.int32 or triples.dtype != torch.int32 or not table.is_contiguous() or triples.numel() < 3 * n:
        raise KernelError("table_update: a contiguous int32 table and 3 n int32 values are wanted")
    _check(library().acv_table_update(_p(table), table.shape[0], table.shape[1], _p(triples), n, _stream()), "table_update")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out = silu(gate_up[:, :I]) * gate_up[:, I:].  gate_up [T, 2I] contiguous."""
    _need_cuda(gate_up, out)
    T, I = out.shape
    _check(library().acv_swiglu(_p(gate_up), _p(out), T, I, dtype_code(out.dtype), _stream()), "swiglu")
    return out


def random_normal(out: torch.Tensor, key: int, mean: float, std: float, t1: torch.Tensor, t2: torch.Tensor) -> torch.Tensor:
    """out (float32 or bfloat16, contiguous) = mean + std * z, z the normal deviates of the Philox stream keyed by
    ``key``; t1, t2: the quantile tables (weights/random_init.py).  Bit-equal to the host's arithmetic."""
    _need_cuda(out, t1, t2)
    if not out.is_contiguous() or t1.numel() != 1024 or t2.numel() != 1025:
        raise KernelError("random_normal: a contiguous output and tables of 1024 and 1025 floats are wanted")
    with torch.cuda.device(out.device):
        _check(library().acv_random_normal(_p(out), out.numel(), key, mean, std, _p(t1), _p(t2), dtype_code(out.dtype),
                                           _stream()), "random_normal")
    return out


def random_int(out: torch.Tensor, key: int, mask: int) -> torch.Tensor:
    """out (int32, contiguous) = words of the Philox stream keyed by ``key``, and-ed with ``mask``."""
    _need_cuda(out)
    with torch.cuda.device(out.device):
        _check(library().acv_random_int(_p(out), out.numel(), key, mask, _stream()), "random_int")
    return out


# ----------------------------------------------------------------------------- attention
def qk_norm_rope_append(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                        q_weight: torch.Tensor | None, k_weight: torch.Tensor | None, eps: float,
                        cos_sin: torch.Tensor | None, positions: torch.Tensor, seq_of_token: torch.Tensor,
                        block_table: torch.Tensor | None, k_pages: torch.Tensor | None,
                        v_pages: torch.Tensor | None, table_rows: torch.Tensor | None = None) -> None:
    """Per-head norm, rotation and cache append over the stacked projection qkv [T, (NH+2NKV)*D], in place.

    cos_sin float32 [positions, R] (cos of R/2 angles, then sin); pages [NP, NKV, page, D].  ``table_rows``
    (int32 [requests], optional): the row of ``block_table`` of each request of the batch (default: its index)."""
    _need_cuda(qkv)
    T = qkv.shape[0]
    rot = cos_sin.shape[1] if cos_sin is not None else 0
    rows = cos_sin.shape[0] if cos_sin is not None else 0
    page = k_pages.shape[2] if k_pages is not None else 1
    n_pages = k_pages.shape[0] if k_pages is not None else 0
    bts = block_table.stride(0) if block_table is not None else 0
    _check(library().acv_qk_norm_rope_append(
        _p(qkv), qkv.stride(0), T, num_heads, num_kv_heads, head_dim, _p(q_weight), _p(k_weight), eps, _p(cos_sin),
        rot, rows, _p(positions), _p(seq_of_token), _p(block_table), bts, _p(table_rows), _p(k_pages), _p(v_pages), page, n_pages,
        dtype_code(qkv.dtype), _stream()), "qk_norm_rope_append")


def attention_generic(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                      positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                      num_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: int = 0,
                      table_rows: torch.Tensor | None = None) -> torch.Tensor:
    """Paged causal attention for every token of the step.  q: rows of num_heads*head_dim (row stride free)."""
    _need_cuda(q, out, k_pages)
    T = q.shape[0]
    _check(library().acv_attention_generic(
        _p(q), q.stride(0), _p(out), out.stride(0), _p(k_pages), _p(v_pages), _p(positions), _p(seq_of_token),
        _p(block_table), block_table.stride(0), _p(table_rows), T, num_heads, num_kv_heads, head_dim, k_pages.shape[2],
        k_pages.shape[0], scale, window, dtype_code(q.dtype), _stream()), "attention_generic")
    return out


# ----------------------------------------------------------------------------- matrix products
def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M,N] = a[M,K] @ w[N,K]^T with 32-bit accumulation on the CUDA cores."""
    _need_cuda(a, w, out)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N or a.dtype != w.dtype:
        raise KernelError(f"gemm_simt: shapes {tuple(a.shape)} x {tuple(w.shape)} -> {tuple(out.shape)} do not fit")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm_simt: innermost strides must be 1")
    _check(library().acv_gemm_simt(_p(a), a.stride(0), _p(w), w.stride(0), _p(out), out.stride(0), M, N, K,
                                   dtype_code(a.dtype), dtype_code(out.dtype), _stream()), "gemm_simt")
    return out


# ----------------------------------------------------------------------------- tensor-core matrix product (bfloat16)
_gemm_scratch: dict = {}


def _gemm_buffers(device, ws_floats: int, n_counters: int):
    key = str(device)
    have = _gemm_scratch.get(key)
    if have is None or have[0].numel() < ws_floats or have[1].numel() < n_counters:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("gemm_tc: workspace would grow during a graph capture; run the shape once first")
        old = have or (torch.empty(0), torch.empty(0), None)
        ws = torch.empty(max(ws_floats, 2 * old[0].numel(), 1 << 20), device=device, dtype=torch.float32)
        cnt = torch.zeros(max(n_counters, 2 * old[1].numel(), 4096), device=device, dtype=torch.int32)
        status = old[2] if old[2] is not None else torch.zeros(1, device=device, dtype=torch.int32)
        if key in _gemm_scratch:
            _retired.append(_gemm_scratch[key])
        have = (ws, cnt, status)
        _gemm_scratch[key] = have
    return have


_sm_counts: dict = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device (asked once per device; 148, a B200's, where there is no device)."""
    if not torch.cuda.is_available():
        return 148
    index = torch.cuda.current_device() if device is None or torch.device(device).index is None else torch.device(device).index
    if index not in _sm_counts:
        _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _sm_counts[index]


# Split and pipeline depth of the products with few tokens (weight rows on the tensor core's M side), as measured
# on a B200 with layer sizes from 0.6B to 32B models: the first row that fits decides.  Splits of K are the CTAs
# of one cluster (summed through its shared memory).  Columns: tiles per SM from (inclusive) to (exclusive),
# k-blocks of 64 from to, tokens per tile (bn) from to (inclusive), then what to do: splits, stages.
#   many tiles: no split, several CTAs share an SM; few tiles: 2..4 splits fill the SMs
INF = float("inf")
GEMM_FEW_TOKENS_RULES = (
    (2.0,    INF,    0,   INF, 16, 128, 1, 8),
    (1.0,    2.0,    0,   INF, 16, 16,  2, 3),
    (1.0,    2.0,    0,   INF, 32, 128, 1, 4),
    (0.0,    1.0,    0,   16,  16, 128, 1, 8),
    (0.0,    1.0,    128, INF, 16, 32,  4, 8),
    (0.0,    1.0,    128, INF, 64, 128, 4, 6),
    (0.2501, 1.0,    16,  128, 16, 16,  4, 4),
    (0.0,    0.2501, 16,  128, 16, 16,  4, 6),
    (0.0,    0.2196, 16,  128, 32, 32,  4, 6),
    (0.2196, 1.0,    16,  128, 32, 32,  2, 6),
    (0.0,    1.0,    16,  128, 64, 128, 3, 6),
)


# Widths of a tile of the tokens-on-rows form, and what a tile costs beside its width, in columns' worth of time.
# Measured on a B200 (2048 x 4096 x 4096: 61 us in tiles of 256 columns, two rounds of the SMs of which the second is
# three quarters empty; 72 us in tiles of 160, three full rounds): a k-block of a tile costs about as much for the 128
# token rows it loads as for 120 of its columns, so a narrower tile pays only where it saves a whole round (1056 x 5120:
# 69 us at 256, 63 us at 160).  The width is chosen so that rounds x (width + overhead) comes out least.
GEMM_TILE_WIDTHS = (256, 224, 192, 160, 128)
GEMM_TILE_OVERHEAD = 120
# Pairs of CTAs on tiles of 256 tokens by 256 features (cta_group::2): a round of such tiles takes about 0.92 of a round
# of 128 x 256 tiles (measured at 2048 and 8192 tokens with the layer sizes of 8B and 14B models: 4 to 11 % less), and
# there are half as many places for them.
GEMM_PAIR_ROUND = 0.92
GEMM_PAIR = 4               # fifth element of a plan: the flag that asks for the pair kernel


def gemm_tc_plan(M: int, N: int, K: int, sms: int | None = None, bn_multiple: int = 16) -> tuple:
    """(swap, bn, splits, stages[, mode]) for x[M,K] @ w[N,K]^T on a device of ``sms`` multiprocessors.

    Up to 128 tokens the weight rows fill the tensor core's M = 128 and the tokens are the narrow
    side (weights stream once whatever the batch); splits of K are chosen so that the work items fill
    whole waves of the SMs (``GEMM_FEW_TOKENS_RULES``).  Above, tokens are the M side and a tile is 128
    tokens by 128..256 features: the width that needs the least rounds x width (``GEMM_TILE_WIDTHS``;
    ``bn_multiple``: widths that are multiples of this only, for an epilogue that wants whole heads),
    or, where that comes out cheaper, 256 x 256 on a pair of CTAs (``mode`` = ``GEMM_PAIR``)."""
    n_kb = -(-K // 64)
    if M <= 128:
        sms = sms or sm_count()
        bn = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128
        tiles = -(-N // 128) * -(-M // bn)
        per_sm = tiles / sms
        for t0, t1, k0, k1, b0, b1, splits, stages in GEMM_FEW_TOKENS_RULES:
            if t0 <= per_sm < t1 and k0 <= n_kb < k1 and b0 <= bn <= b1:
                return 1, bn, splits, stages
        return 1, bn, 1, 8
    if N < 256:
        return 0, (128 if N > 64 else 64), 1, 8
    sms = sms or sm_count()
    best, best_cost = 256, None
    for bn in GEMM_TILE_WIDTHS:
        if bn % bn_multiple:
            continue
        tiles = -(-M // 128) * -(-N // bn)
        cost = -(-tiles // sms) * (bn + GEMM_TILE_OVERHEAD)
        if best_cost is None or cost < 0.97 * best_cost:       # a narrower tile has to win clearly
            best, best_cost = bn, cost
    if sms >= 2 and 256 % bn_multiple == 0:
        pair_tiles = -(-M // 256) * -(-N // 256)
        if -(-pair_tiles // (sms // 2)) * (256 + GEMM_TILE_OVERHEAD) * GEMM_PAIR_ROUND < best_cost:
            return 0, 256, 1, 6, GEMM_PAIR
    return 0, best, 1, 8


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, plan: tuple | None = None,
            swiglu_pairs: bool = False, static_weights: bool = False) -> torch.Tensor:
    """out[M,N] = x[M,K] @ w[N,K]^T on tcgen05; x, w bfloat16, out bfloat16 or float32.

    ``static_weights``: w was written long before this call (a model's weights), so the kernel may
    read its first tiles while the kernel before it in the stream is still running.

    With ``swiglu_pairs`` the rows of w come in (gate, up) pairs and out is [M, N/2]:
    out[:, i] = silu(x . w[2i]) * (x . w[2i+1]), rounded as the separate kernels round."""
    _need_cuda(x, w, out)
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("gemm_tc: operands must be bfloat16 and the output bfloat16 or float32")
    n_out = N // 2 if swiglu_pairs else N
    if swiglu_pairs and (N % 2 or out.dtype != torch.bfloat16):
        raise KernelError("gemm_tc: the paired SwiGLU output needs an even number of weight rows and a bfloat16 output")
    if w.shape[1] != K or out.shape != (M, n_out) or x.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError(f"gemm_tc: shapes {tuple(x.shape)} x {tuple(w.shape)} -> {tuple(out.shape)} do not fit")
    plan = plan or gemm_tc_plan(M, N, K)
    swap, bn, splits = plan[:3]
    stages = plan[3] if len(plan) > 3 else 8
    cluster = plan[4] if len(plan) > 4 else (1 if swap and 1 < splits <= 8 else 0)
    tiles = (-(-N // 128) * -(-M // bn)) if swap else (-(-M // 128) * -(-N // bn))
    ws, cnt, status = _gemm_buffers(x.device, tiles * splits * bn * 128 if splits > 1 else 0, tiles)
    _check(library().acv_gemm_tc(_p(x), x.stride(0), _p(w), w.stride(0), _p(out), out.stride(0), M, N, K,
                                 1 if out.dtype == torch.float32 else 0, 1 if swiglu_pairs else 0, swap, bn, splits,
                                 _p(ws), ws.numel(), _p(cnt),
                                 cnt.numel(), _p(status), sm_count(x.device), stages, cluster | (2 if static_weights else 0), _stream()), "gemm_tc")
    return out


def gemm_tc_qkv_takes(x: torch.Tensor, w: torch.Tensor, head_dim: int, cos_sin: torch.Tensor | None,
                      k_pages: torch.Tensor | None) -> bool:
    """Whether the stacked q,k,v projection of x can take its epilogue (norm, rotation, append) with it: bfloat16,
    heads of 64 or 128 rotated as a whole, and either up to 32 tokens with a plan that gives every CTA one tile
    (features on the tensor-memory lanes) or more than 128 tokens (tokens on the lanes, whole heads in a tile)."""
    if k_pages is None or x.dtype != torch.bfloat16 or head_dim not in (64, 128) or not gemm_tc_takes(x, w):
        return False
    if cos_sin is not None and (cos_sin.shape[1] != head_dim or cos_sin.dtype != torch.float32):
        return False
    M, K = x.shape
    N = w.shape[0]
    swap, bn, splits = gemm_tc_plan(M, N, K, bn_multiple=head_dim if M > 128 else 16)[:3]
    if not swap:            # tokens on M (one CTA or a pair to a tile): a thread of the epilogue holds whole heads of one token
        return splits == 1 and bn >= head_dim and bn % head_dim == 0
    tiles = -(-N // 128) * -(-M // bn)
    return bn <= 32 and (1 < splits <= 8 or (splits == 1 and tiles <= sm_count(x.device)))


def gemm_tc_qkv(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                q_weight: torch.Tensor | None, k_weight: torch.Tensor | None, eps: float, cos_sin: torch.Tensor | None,
                positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor, k_pages: torch.Tensor,
                v_pages: torch.Tensor, static_weights: bool = False, table_rows: torch.Tensor | None = None,
                plan: tuple | None = None) -> torch.Tensor:
    """The stacked q,k,v projection out[M, (NH+2NKV)*D] = x @ w^T with the epilogue of ``qk_norm_rope_append``
    inside the product's kernel: the query columns of out hold the normed, rotated queries, keys and values go
    to their pages (the key and value columns of out are not written).  ``gemm_tc_qkv_takes`` says when."""
    _need_cuda(x, w, out, k_pages, v_pages)
    M, K = x.shape
    N = w.shape[0]
    plan = plan or gemm_tc_plan(M, N, K, bn_multiple=head_dim if M > 128 else 16)
    swap, bn, splits, stages = plan[:4]
    cluster = plan[4] if len(plan) > 4 else (1 if swap and 1 < splits <= 8 else 0)
    tiles = (-(-N // 128) * -(-M // bn)) if swap else (-(-M // 128) * -(-N // bn))
    ws, cnt, status = _gemm_buffers(x.device, tiles * splits * bn * 128 if splits > 1 else 0, tiles)
    _check(library().acv_gemm_tc_qkv(
        _p(x), x.stride(0), _p(w), w.stride(0), _p(out), out.stride(0), M, N, K, swap, bn, splits, _p(ws), ws.numel(),
        _p(cnt), cnt.numel(), _p(status), sm_count(x.device), stages, cluster | (2 if static_weights else 0), num_heads,
        num_kv_heads, head_dim, _p(q_weight), _p(k_weight), eps, _p(cos_sin),
        cos_sin.shape[0] if cos_sin is not None else 0, _p(positions), _p(seq_of_token), _p(block_table),
        block_table.stride(0), _p(table_rows), _p(k_pages), _p(v_pages), k_pages.shape[2], k_pages.shape[0], _stream()),
        "gemm_tc_qkv")
    return out


def gemm_tc_takes(x: torch.Tensor, w: torch.Tensor) -> bool:
    """The tensor-core kernel needs 16-byte aligned rows: K and the row strides multiples of 8."""
    return (x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0 and x.stride(1) == 1 and w.stride(1) == 1)


def status_word(device) -> torch.Tensor:
    """The int32 word (on ``device``) into which the tensor-core kernels write a code when one of their bounded
    waits runs out (0 otherwise).  The engine copies it to the host with every step's tokens."""
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return _gemm_buffers(device, 0, 0)[2]


def reset_after_failure() -> None:
    """After a step whose kernels gave up a wait: the status word back to 0, and the arrival counters of the
    split products and of the split attention back to 0 (a CTA that gave up never arrived at its tile)."""
    for _, cnt, status in _gemm_scratch.values():
        status.zero_()
        cnt.zero_()
    for _, _, cnt in _scratch.values():
        cnt.zero_()
    for buf in _layer_scratch.values():
        buf["bars"].zero_()


def gemm_tc_test_fault(wait_limit: int, skip_k_block: int) -> None:
    """For the test of the bounded waits: the next tensor-core product of this process polls each barrier at most
    ``wait_limit`` times and never loads k-block ``skip_k_block``, so it gives up, frees what it holds, returns,
    and leaves the wait's code in the status word.  Nothing faults, traps or hangs."""
    library().acv_gemm_tc_test_fault(int(wait_limit), int(skip_k_block))


def gemm_status(device=None) -> int:
    """0, or the code a bounded wait inside a tensor-core product left when it ran out (synchronises)."""
    worst = 0
    for key, (_, _, status) in _gemm_scratch.items():
        worst = max(worst, int(status.item()))
    return worst


# ----------------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r] = argmax(logits[r]) (lowest index among equals).  logits float32 [R, V]; out int32 [R]."""
    _need_cuda(logits, out)
    R, V = logits.shape
    _check(library().acv_argmax(_p(logits), logits.stride(0), R, V, _p(out), _stream()), "argmax")
    return out


def apply_penalties(logits: torch.Tensor, pen_row: torch.Tensor, pen_token: torch.Tensor, pen_count: torch.Tensor,
                    repetition: torch.Tensor, presence: torch.Tensor, frequency: torch.Tensor) -> None:
    _need_cuda(logits, pen_row)
    _check(library().acv_apply_penalties(_p(logits), logits.stride(0), logits.shape[1], _p(pen_row), _p(pen_token),
                                         _p(pen_count), pen_row.numel(), _p(repetition), _p(presence),
                                         _p(frequency), _stream()), "apply_penalties")


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, seed: torch.Tensor, counter: torch.Tensor, out_token: torch.Tensor,
           out_logprob: torch.Tensor | None = None) -> torch.Tensor:
    """One token per row.  seed, counter: int64 [R] (read as unsigned)."""
    _need_cuda(logits, out_token)
    R, V = logits.shape
    _check(library().acv_sample(_p(logits), logits.stride(0), R, V, _p(temperature), _p(top_k), _p(top_p), _p(min_p),
                                _p(seed), _p(counter), _p(out_token), _p(out_logprob), _stream()), "sample")
    return out_token


def top_logprobs(logits: torch.Tensor, k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """(ids int32 [R, k], log probabilities float32 [R, k]) of each row's k most probable tokens, most probable
    first (equal logits: the lower id first); log probability = logit - logsumexp(row).  1 <= k <= 64; where a row
    has fewer than k entries above -inf the rest is id -1 with -inf."""
    _need_cuda(logits)
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("top_logprobs: float32 rows wanted")
    R, V = logits.shape
    ids = torch.empty((R, k), device=logits.device, dtype=torch.int32)
    lp = torch.empty((R, k), device=logits.device, dtype=torch.float32)
    _check(library().acv_top_logprobs(_p(logits), logits.stride(0), R, V, k, _p(ids), _p(lp), _stream()), "top_logprobs")
    return ids, lp


# ----------------------------------------------------------------------------- tensor-core attention (bfloat16)
_scratch: dict = {}
_retired: list = []     # outgrown scratch buffers, never freed (graphs captured earlier point into them)


def _decode_scratch(device, floats: int, ml_floats: int, counters: int):
    """Scratch of the split-KV kernel, kept between calls and only ever grown (addresses that a
    captured graph holds stay valid as long as a warm-up call of the same shape came first)."""
    key = str(device)
    have = _scratch.get(key)
    if have is None or have[0].numel() < floats or have[1].numel() < ml_floats or have[2].numel() < counters:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("attention_decode: scratch would grow during a graph capture; run the shape once first")
        grow = lambda n, old: max(n, 2 * old)
        o = have or (torch.empty(0), torch.empty(0), torch.empty(0))
        have = (torch.empty(grow(floats, o[0].numel()), device=device, dtype=torch.float32),
                torch.empty(grow(ml_floats, o[1].numel()), device=device, dtype=torch.float32),
                torch.zeros(grow(counters, o[2].numel()), device=device, dtype=torch.int32))
        if key in _scratch:
            _retired.append(_scratch[key])   # a captured graph may still hold these addresses: keep them alive
        _scratch[key] = have
    return have


# What the choice of the number of splits reckons with: fitted to a sweep on a B200 over 1 to 64 requests, contexts of
# 1024 to 65536 keys (8 kv-heads of 128, 4 query heads each, pages of 64; launches that overlap as in a step, pages
# that no launch finds in L2) and every way of splitting below.  The reckoned time is within 11 % of the measured one
# (root mean square); the splits chosen took 2.7 % more time over the whole sweep than the best of each case (the rule
# before it, "CTAs for not quite twice the SMs": 9 %, and up to 60 % where clusters of 8 did not fit the device at once).
DECODE_KEY_US = 0.0117           # a CTA alone streams a key and its value in this time (its warps wait for their rings)
DECODE_KEY_US_ALONE = 0.00645    # the same where a CTA has an SM to itself and eight warps
DECODE_STREAM_BYTES_US = 6.45e6  # what all CTAs together stream from memory
DECODE_BOUNDS_NORM = 24.0        # a round takes the p-norm of the two times: with this p, the larger
DECODE_MERGE_US = (6.6, 8.0, 0.45, 8.5, 0.81)   # start to end without splits; merged inside a cluster + per split;
                                                # through scratch memory + per split
DECODE_SPLIT_KEYS = 256          # no split shorter than this
DECODE_CLUSTER_SPLITS = (2, 4, 6, 8)       # 3 and 5 were never better than their even neighbours by more than 2 %
DECODE_SCRATCH_SPLITS = (2, 4, 8, 12, 16, 24, 32)
DECODE_WIDE_CLUSTER_FIT = 0.85   # of the clusters of more than 6 CTAs that the runtime says fit at once, this part did
# Inside a step the kernel's end is what the next kernel waits for, and there shorter CTAs won where the sweep saw a tie
# (8 requests of 2100 keys: 4 splits 3.716 ms a step, 2 splits 3.743, none 3.821).  Among the ways that the reckoning
# puts within this factor of the cheapest, the one with the most splits is taken if it merges in clusters and its CTAs
# all fit the device at once.
DECODE_MORE_SPLITS_WITHIN = 1.05


@functools.lru_cache(maxsize=None)
def decode_resident(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, n_splits: int,
                    pages_of_split: int, cluster_merge: bool, alone: bool = False) -> int:
    """How many CTAs of the split-KV kernel the device holds at once (asked of the runtime: a cluster needs its CTAs
    side by side in one part of the chip).  ``alone``: how many it holds one to an SM; a grid of no more CTAs runs with
    eight warps to a CTA instead of four (0: that form does not fit these sizes)."""
    n = library().acv_attention_decode_resident(num_heads, num_kv_heads, head_dim, page_size, 0, n_splits,
                                                pages_of_split * page_size * n_splits, 1 if cluster_merge else 0,
                                                1 if alone else 0)
    if n < 0:
        raise KernelError(f"attention_decode_resident: {_ERRORS.get(n, f'refused with code {n}')}")
    return n if alone else max(1, n)


def decode_splits_cost(n_dec: int, num_kv_heads: int, max_kv: int, n_splits: int, cluster_merge: bool, resident: int,
                       row_bytes: int, resident_alone: int = 0) -> float:
    """Reckoned microseconds of the split-KV kernel: the CTAs run in rounds of ``resident``; a round takes as long as
    one CTA needs for its keys alone, or as the memory needs for the round's bytes; then the merge.  A grid of up to
    ``resident_alone`` CTAs has an SM for each, eight warps to a CTA, and streams faster."""
    ctas = n_dec * num_kv_heads * n_splits
    keys = -(-max_kv // n_splits)
    alone = keys * (DECODE_KEY_US_ALONE if ctas <= resident_alone else DECODE_KEY_US)
    p = DECODE_BOUNDS_NORM
    round_us = lambda n: (alone ** p + (n * keys * row_bytes / DECODE_STREAM_BYTES_US) ** p) ** (1.0 / p)
    full, rest = divmod(ctas, resident)
    us = full * round_us(resident) + (round_us(rest) if rest else 0.0)
    if n_splits == 1:
        return us + DECODE_MERGE_US[0]
    if cluster_merge:
        return us + DECODE_MERGE_US[1] + DECODE_MERGE_US[2] * n_splits
    return us + DECODE_MERGE_US[3] + DECODE_MERGE_US[4] * n_splits


def decode_ways(n_dec: int, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, keys: int) -> list:
    """Every way of splitting ``keys`` keys of ``n_dec`` requests that the plan chooses from, as (reckoned microseconds,
    splits, merged inside clusters?, all CTAs fit the device at once?)."""
    row_bytes = 2 * head_dim * 2                       # a key and a value of one kv-head in bfloat16
    ways = []
    for n_splits, cluster in [(1, False)] + [(s, True) for s in DECODE_CLUSTER_SPLITS] + \
                             [(s, False) for s in DECODE_SCRATCH_SPLITS]:
        if n_splits > 1 and keys < n_splits * DECODE_SPLIT_KEYS:
            continue
        if n_dec * num_kv_heads * n_splits > 65535 * 4:
            continue
        pages = -(-(-(-keys // n_splits)) // page_size)
        pages = 1 << max(0, pages - 1).bit_length()
        resident = decode_resident(num_heads, num_kv_heads, head_dim, page_size, n_splits, pages, cluster)
        alone = decode_resident(num_heads, num_kv_heads, head_dim, page_size, n_splits, pages, cluster, True)
        if cluster and n_splits > 6:
            resident = max(n_splits, int(resident * DECODE_WIDE_CLUSTER_FIT))
            alone = min(alone, resident)
        resident = max(resident, alone)
        cost = decode_splits_cost(n_dec, num_kv_heads, keys, n_splits, cluster, resident, row_bytes, alone)
        ways.append((cost, n_splits, cluster, n_dec * num_kv_heads * n_splits <= resident))
    return ways


@functools.lru_cache(maxsize=4096)
def decode_plan(n_dec: int, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, max_kv: int,
                window: int = 0) -> tuple[int, bool]:
    """(splits of the context, merged inside clusters?) for ``n_dec`` one-token requests with up to ``max_kv`` keys:
    by ``decode_splits_cost`` among no split, up to 8 splits merged inside a cluster and up to 32 merged through
    scratch memory.  A split more pays while it shortens what a CTA streams alone; it stops paying when the CTAs no
    longer fit the device at once or the memory is the limit anyway."""
    keys = min(max_kv, window) if window > 0 else max_kv
    ways = decode_ways(n_dec, num_heads, num_kv_heads, head_dim, page_size, keys)
    cheapest = min(ways)
    near = [w for w in ways if w is cheapest or (w[0] <= DECODE_MORE_SPLITS_WITHIN * cheapest[0] and w[2] and w[3])]
    best = max(near, key=lambda w: w[1])
    return best[1], best[2]


def attention_decode(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                     dec_tokens: torch.Tensor, dec_seqs: torch.Tensor, n_dec: int, kv_len: torch.Tensor,
                     block_table: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                     window: int, n_splits: int, max_kv: int = 0, cluster_merge: bool = True,
                     table_rows: torch.Tensor | None = None) -> torch.Tensor:
    """Attention of requests that bring one token each, over their pages, split over the context.

    Up to 8 splits are merged inside a thread-block cluster (through its shared memory); more, or
    ``cluster_merge=False``, go through partial results in scratch memory and a last-arriver merge."""
    n_rep = num_heads // num_kv_heads
    use_cluster = cluster_merge and 1 < n_splits <= 8
    parts = n_dec * num_kv_heads * n_splits if n_splits > 1 and not use_cluster else 0
    acc, ml, cnt = _decode_scratch(q.device, parts * n_rep * head_dim, parts * n_rep * 2, n_dec * num_kv_heads)
    _check(library().acv_attention_decode(
        _p(q), q.stride(0), _p(out), out.stride(0), _p(k_pages), _p(v_pages), _p(dec_tokens), _p(dec_seqs), n_dec,
        _p(kv_len), _p(block_table), block_table.stride(0), _p(table_rows), num_heads, num_kv_heads, head_dim,
        k_pages.shape[2], k_pages.shape[0], scale, window, n_splits, _p(acc), _p(ml), _p(cnt), acc.numel(), ml.numel(), cnt.numel(),
        max_kv or block_table.shape[1] * k_pages.shape[2], 1 if use_cluster else 0, _stream()), "attention_decode")
    return out


def attention_chunk(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                    tile_seq: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int, cu_q: torch.Tensor,
                    kv_len: torch.Tensor, block_table: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                    scale: float, window: int, table_rows: torch.Tensor | None = None, max_kv: int = 0) -> torch.Tensor:
    """Causal attention of portions of prompts (tiles of QUERY_TILE query tokens) over their requests' pages."""
    _check(library().acv_attention_chunk(
        _p(q), q.stride(0), _p(out), out.stride(0), _p(k_pages), _p(v_pages), _p(tile_seq), _p(tile_q0), n_tiles,
        _p(cu_q), _p(kv_len), _p(block_table), block_table.stride(0), _p(table_rows), num_heads, num_kv_heads, head_dim,
        k_pages.shape[2], k_pages.shape[0], scale, window, max_kv or block_table.shape[1] * k_pages.shape[2], _stream()),
        "attention_chunk")
    return out


def attention_tc(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                 tile_seq: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int, cu_q: torch.Tensor, kv_len: torch.Tensor,
                 block_table: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                 window: int, table_rows: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention of portions of prompts on tcgen05 (tiles of QUERY_TILE query tokens, pages by TMA)."""
    _, _, status = _gemm_buffers(q.device, 0, 0)
    _check(library().acv_attention_tc(
        _p(q), q.stride(0), q.shape[0], _p(out), out.stride(0), _p(k_pages), _p(v_pages), _p(tile_seq), _p(tile_q0),
        n_tiles, _p(cu_q), _p(kv_len), _p(block_table), block_table.stride(0), _p(table_rows), num_heads, num_kv_heads,
        head_dim, k_pages.shape[2], k_pages.shape[0], scale, window, _p(status), _stream()), "attention_tc")
    return out


def attention_tc_takes(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, head_dim: int) -> bool:
    page = k_pages.shape[2]
    return (head_dim in (64, 128) and page in (8, 16, 32, 64, 128) and q.stride(0) % 8 == 0 and out.stride(0) % 8 == 0
            and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0 and k_pages.is_contiguous())


def tensor_core_attention_takes(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    return dtype == torch.bfloat16 and head_dim in (64, 128) and num_heads // num_kv_heads <= 16


# ----------------------------------------------------------------------------- dispatch by shape
QUERY_TILE = 128   # query tokens per tile of the portion-attention kernels (AT_BM of attention_tc.cu)


def attention_work(q_lens, kv_lens, cu_q) -> tuple[dict, dict]:
    """Work lists of the attention kernels for a step: the requests with one token (decoding) and tiles of
    QUERY_TILE tokens of the requests with more (portions of prompts), late tiles first since they see most keys.
    Returns (int32 arrays that the kernels read on the device, counts and maxima for the launches)."""
    import numpy as np
    ql = np.asarray(q_lens, dtype=np.int32)
    dec = np.nonzero(ql == 1)[0].astype(np.int32)
    tile_seq, tile_q0, tile_keys = [], [], []
    for i in np.nonzero(ql > 1)[0]:
        starts_i = np.arange(0, q_lens[i], QUERY_TILE, dtype=np.int32)
        tile_seq.append(np.full(starts_i.size, i, dtype=np.int32))
        tile_q0.append(starts_i)
        tile_keys.append(int(kv_lens[i]) - int(q_lens[i]) + np.minimum(starts_i + QUERY_TILE, int(q_lens[i])))   # keys a tile's last query sees
    empty = np.zeros(0, np.int32)
    if tile_seq:
        # the tiles with most keys first, over all requests: the hardware hands out CTAs in this order, and the kernel
        # that gives a CTA two tiles pairs the list's front with its back
        order = np.argsort(-np.concatenate(tile_keys), kind="stable")
        tile_seq, tile_q0 = [np.concatenate(tile_seq)[order]], [np.concatenate(tile_q0)[order]]
    arrays = {"dec_tokens": np.asarray(cu_q, dtype=np.int32)[:-1][dec], "dec_seqs": dec,
              "tile_seq": np.concatenate(tile_seq) if tile_seq else empty,
              "tile_q0": np.concatenate(tile_q0) if tile_q0 else empty}
    values = {"n_dec": int(dec.size), "n_tiles": int(sum(t.size for t in tile_seq)),
              "max_dec_kv": max((k for k, q in zip(kv_lens, q_lens) if q == 1), default=0),
              "max_tile_kv": max((k for k, q in zip(kv_lens, q_lens) if q > 1), default=0)}
    return arrays, values


def attention_work_decode(padded: int, max_kv: int) -> tuple[dict, dict]:
    """The same for a batch of ``padded`` requests with one token each, made for contexts up to ``max_kv``."""
    import numpy as np
    ar = np.arange(padded, dtype=np.int32)
    return ({"dec_tokens": ar, "dec_seqs": ar, "tile_seq": np.zeros(0, np.int32), "tile_q0": np.zeros(0, np.int32)},
            {"n_dec": padded, "n_tiles": 0, "max_dec_kv": max_kv, "max_tile_kv": 0})


def attention(qkv: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, ctx,
              block_table: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
              window: int = 0, work: dict | None = None) -> torch.Tensor:
    """Attention of every token of the step over its request's pages.

    ``qkv`` is the stacked projection after norm and rotation (queries are its first
    num_heads*head_dim columns); ``ctx`` is the step's StepContext; ``work`` the step's work lists
    (``attention_work``; default: ``ctx.work``).  bfloat16 with a head size of 64 or 128 goes to the
    tensor-core kernels, requests with one token to the split-KV kernel and portions to the tiled
    one; everything else to the generic kernel."""
    rows = getattr(ctx, "table_rows", None)
    if not tensor_core_attention_takes(qkv.dtype, num_heads, num_kv_heads, head_dim):
        return attention_generic(qkv, out, k_pages, v_pages, ctx.positions, ctx.seq_of_token, block_table, num_heads,
                                 num_kv_heads, head_dim, scale, window, table_rows=rows)
    w = work if work is not None else ctx.work
    if w["n_dec"]:
        kv = min(w["max_dec_kv"], window) if window > 0 else w["max_dec_kv"]
        n_splits, in_clusters = (w["n_splits"], True) if w.get("n_splits") else \
            decode_plan(w["n_dec"], num_heads, num_kv_heads, head_dim, k_pages.shape[2], kv)
        attention_decode(qkv, out, k_pages, v_pages, w["dec_tokens"], w["dec_seqs"], w["n_dec"], ctx.kv_len,
                         block_table, num_heads, num_kv_heads, head_dim, scale, window, n_splits, w["max_dec_kv"],
                         cluster_merge=in_clusters, table_rows=rows)
    if w["n_tiles"] and attention_tc_takes(qkv, out, k_pages, head_dim):
        attention_tc(qkv, out, k_pages, v_pages, w["tile_seq"], w["tile_q0"], w["n_tiles"], ctx.cu_q, ctx.kv_len,
                     block_table, num_heads, num_kv_heads, head_dim, scale, window, table_rows=rows)
    elif w["n_tiles"]:
        attention_chunk(qkv, out, k_pages, v_pages, w["tile_seq"], w["tile_q0"], w["n_tiles"], ctx.cu_q, ctx.kv_len,
                        block_table, num_heads, num_kv_heads, head_dim, scale, window, table_rows=rows,
                        max_kv=w.get("max_tile_kv", 0))
    return out


# ----------------------------------------------------------------------------- one decoder layer of a decode step
DECODE_LAYER_TOKENS = 16     # DL_BN of decode_layer.cu
DECODE_LAYER_TRACE: torch.Tensor | None = None   # int64 [SMs, 8] on the device: every fused layer leaves its phase stamps there
_layer_scratch: dict = {}


def decode_layer_takes(T: int, H: int, I: int, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                       window: int) -> bool:
    """Whether the fused decode-layer kernel runs a layer of these sizes for a step of ``T`` one-token requests."""
    return bool(library().acv_decode_layer_takes(T, H, I, num_heads, num_kv_heads, head_dim, page_size, window))


def _layer_buffers(device, H: int, I: int, qkv_width: int, q_width: int):
    """Activations of one layer (16 rows each) and the grid barriers, kept between calls (layers run one after the
    other on one stream, and a captured graph holds the addresses)."""
    key = (str(device), H, I, qkv_width, q_width)
    have = _layer_scratch.get(key)
    if have is None:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("decode_layer: its buffers would be made during a graph capture; run the shape once first")
        n = DECODE_LAYER_TOKENS
        mk = lambda w: torch.zeros((n, w), device=device, dtype=torch.bfloat16)
        have = {"h": mk(H), "qkv": mk(qkv_width), "attn": mk(q_width), "a": mk(H), "act": mk(I),
                "bars": torch.zeros(8, device=device, dtype=torch.int32)}
        _layer_scratch[key] = have
    return have


def decode_layer(x: torch.Tensor, delta: torch.Tensor | None, delta_out: torch.Tensor, norm1_w: torch.Tensor,
                 norm2_w: torch.Tensor, eps: float, w_qkv: torch.Tensor, w_o: torch.Tensor, w_gate_up_pairs: torch.Tensor,
                 w_down: torch.Tensor, q_norm: torch.Tensor | None, k_norm: torch.Tensor | None, qk_eps: float,
                 cos_sin: torch.Tensor | None, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                 positions: torch.Tensor, seq_of_token: torch.Tensor, kv_len: torch.Tensor, block_table: torch.Tensor,
                 table_rows: torch.Tensor | None, k_pages: torch.Tensor, v_pages: torch.Tensor, max_kv: int,
                 trace: torch.Tensor | None = None) -> torch.Tensor:
    """A whole pre-norm decoder layer for a step of up to 16 one-token requests in one persistent kernel
    (csrc/decode_layer.cu): x += delta; a = attention(norm1(x)); x += a; delta_out = swiglu_mlp(norm2(x)).
    ``x`` [T, H] is updated in place, ``delta_out`` [T, H] receives what the next layer adds; the keys and values of
    the step's tokens go to their pages.  ``w_gate_up_pairs``: rows (gate_i, up_i) interleaved, as the fused SwiGLU
    product takes them.  ``decode_layer_takes`` says for which sizes.  ``trace`` (int64 [SMs, 8], optional): each CTA
    leaves the device-wide nanosecond time at which it began and at which it finished each phase (norm, q/k/v,
    attention, output product, norm, gate/up, down)."""
    _need_cuda(x, delta_out, w_qkv, k_pages)
    T, H = x.shape
    I = w_down.shape[1]
    qkv_width, q_width = w_qkv.shape[0], num_heads * head_dim
    buf = _layer_buffers(x.device, H, I, qkv_width, q_width)
    n_rep = num_heads // num_kv_heads
    sms = sm_count(x.device)
    tiles = [-(-n // 128) for n in (qkv_width, H, 2 * I, H)]
    ws, cnt, status = _gemm_buffers(x.device, max(tiles) * 16 * 16 * 128, sum(tiles))
    part, _, att_cnt = _decode_scratch(x.device, sms * n_rep * (head_dim + 2), 0, DECODE_LAYER_TOKENS * num_kv_heads)
    a = DecodeLayerArgs(
        T=T, H=H, I=I, NH=num_heads, NKV=num_kv_heads, D=head_dim, eps=eps, qk_eps=qk_eps, scale=scale,
        x=_p(x), delta_in=_p(delta), w_norm1=_p(norm1_w), w_norm2=_p(norm2_w), w_qkv=_p(w_qkv), w_o=_p(w_o),
        w_gu=_p(w_gate_up_pairs), w_down=_p(w_down), q_norm=_p(q_norm), k_norm=_p(k_norm), cos_sin=_p(cos_sin),
        table_rows=cos_sin.shape[0] if cos_sin is not None else 0, positions=_p(positions), seq_of_token=_p(seq_of_token),
        kv_len=_p(kv_len), block_table=_p(block_table), bt_stride=block_table.stride(0), bt_rows=_p(table_rows),
        k_pages=_p(k_pages), v_pages=_p(v_pages), page_size=k_pages.shape[2], num_pages=k_pages.shape[0],
        h=_p(buf["h"]), qkv=_p(buf["qkv"]), attn_out=_p(buf["attn"]), a_out=_p(buf["a"]), act=_p(buf["act"]),
        delta_out=_p(delta_out), workspace=_p(ws), workspace_floats=ws.numel(), counters=_p(cnt), n_counters=cnt.numel(),
        part=_p(part), part_floats=part.numel(), att_counters=_p(att_cnt), n_att_counters=att_cnt.numel(),
        bars=_p(buf["bars"]), status=_p(status), sm_count=sms, max_kv=max(1, max_kv),
        trace=_p(trace if trace is not None else DECODE_LAYER_TRACE))
    _check(library().acv_decode_layer(ctypes.byref(a), _stream()), "decode_layer")
    return delta_out


def linear_bf16(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, static_weights: bool = False) -> torch.Tensor:
    """out = x @ w^T in bfloat16 with float accumulation: the tcgen05 kernel; rows that are not 16-byte
    aligned (K or a stride no multiple of 8) go to the library product, as all do in the reference."""
    if gemm_tc_takes(x, w):
        return gemm_tc(x, w, out, static_weights=static_weights)
    return torch.mm(x, w.t(), out=out)


def linear_bf16_swiglu(x: torch.Tensor, w_pairs: torch.Tensor, out: torch.Tensor,
                       static_weights: bool = False) -> torch.Tensor:
    """out[M, I] = silu(x @ Wg^T) * (x @ Wu^T) in one kernel; w_pairs [2I, K] holds (gate_i, up_i) in rows 2i, 2i+1."""
    return gemm_tc(x, w_pairs, out, swiglu_pairs=True, static_weights=static_weights)


def linear_bf16_f32out(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, static_weights: bool = False) -> torch.Tensor:
    """out (float32) = x @ w^T from bfloat16 operands, accumulated in float32."""
    if gemm_tc_takes(x, w):
        return gemm_tc(x, w, out, static_weights=static_weights)
    return gemm_simt(x, w, out)
