"""Python side of the CUDA kernels: loads each module's shared library (building it at first
use), checks shapes, types and devices, and calls the C entry points on torch's current
stream.  Nothing here computes on the CPU and nothing falls back to a library kernel: a
missing extension or a refused size raises.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Dict, Optional

import torch

from . import build
from .build import ExtensionError

PAGE = 64                      # tokens per cache page; equals kl::PAGE in common.cuh

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

_ERRORS = {-1: "unsupported dtype", -2: "unsupported size", -3: "misaligned pointer or stride",
           -4: "the kernel reported an error through its status word", -5: "set-up failed"}


class KernelError(RuntimeError):
    pass


_libs: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def lib(name: str) -> ctypes.CDLL:
    """The loaded shared library of one kernel module."""
    got = _libs.get(name)
    if got is not None:
        return got
    with _lock:
        if name not in _libs:
            path = build.ensure_built(name)
            try:
                _libs[name] = ctypes.CDLL(path)
            except OSError as e:
                raise ExtensionError(f"cannot load {path}: {e}") from None
        return _libs[name]


def loaded_libraries() -> Dict[str, str]:
    return {n: l._name for n, l in _libs.items()}


launch_count = 0       # kernels of this package launched so far (counted per entry-point call)


def _check(code: int, what: str, launches: int = 1) -> None:
    global launch_count
    if code == 0:
        launch_count += launches
        return
    if code in _ERRORS:
        raise KernelError(f"{what}: {_ERRORS[code]}")
    raise KernelError(f"{what}: CUDA error {code}")


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} is not supported by the kernels (float32, bfloat16)") from None


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


# The current stream's handle, once per launch: torch.cuda.current_stream() builds a Stream object and
# looks the device up three times (7 us); the raw call behind it takes a fraction of a microsecond.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> ctypes.c_void_p:
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel arguments must live on a CUDA device; there is no CPU path")


def _i32(t: Optional[torch.Tensor], name: str) -> None:
    if t is not None:
        _need(t.dtype == torch.int32 and t.is_contiguous(), f"{name} must be a contiguous int32 tensor")


# --------------------------------------------------------------------------- row-wise

def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, error_flag: torch.Tensor,
              scale: float = 1.0) -> None:
    """out[t] = scale * float32(table[ids[t]]); ids outside the table set error_flag[0] = 1."""
    _cuda(ids, table, out, error_flag)
    _i32(ids, "ids"); _i32(error_flag, "error_flag")
    n, (vocab, hidden) = ids.numel(), table.shape
    _need(table.is_contiguous() and out.is_contiguous() and out.dtype == torch.float32, "embedding: bad layout")
    _need(out.shape[0] >= n and out.shape[1] == hidden, "embedding: output shape")
    _check(lib("rowwise").kl_embedding(_ptr(ids), n, _ptr(table), dtype_code(table.dtype), vocab, hidden,
                                       ctypes.c_float(scale), _ptr(out), _ptr(error_flag), _stream()), "embedding")


def logit_transform(logits: torch.Tensor, scale: float = 1.0, softcap: float = 0.0) -> None:
    """In place on float32 logits [rows, vocab]: x = scale * x, then with ``softcap`` c > 0
    x = c * tanh(x / c)."""
    _cuda(logits)
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1, "logit_transform: float32 rows")
    _need(softcap >= 0.0, "logit_transform: the soft cap must not be negative")
    rows, vocab = logits.shape
    _check(lib("rowwise").kl_logit_transform(_ptr(logits), ctypes.c_longlong(logits.stride(0)), rows, vocab,
                                             ctypes.c_float(scale), ctypes.c_float(softcap), _stream()), "logit_transform")


def _partials(delta: Optional[torch.Tensor]) -> bool:
    """A delta given as float32 partial sums [S, rows, width] (the pieces of a product whose K
    range was cut), to be added in ascending order by the kernel that consumes it."""
    return delta is not None and delta.dim() == 3


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, out: torch.Tensor,
                eps: float, rows: Optional[torch.Tensor] = None) -> None:
    """x = residual (+ delta); out = weight * x * rsqrt(mean(x^2) + eps).

    ``delta`` is [rows, hidden] in the output's dtype, or float32 partial sums
    [S, rows, hidden].  Without ``rows`` every row is processed and, when ``delta`` is given,
    the sum is written back to ``residual``.  With ``rows`` (int32 indices) only those rows
    are read, into out[0..len(rows)), and ``residual`` is left as it is."""
    _cuda(residual, delta, weight, out, rows)
    _i32(rows, "rows")
    hidden = residual.shape[-1]
    n = rows.numel() if rows is not None else residual.shape[0]
    _need(residual.dtype == torch.float32 and residual.is_contiguous(), "add_rmsnorm: the residual stream is float32")
    _need(weight.dtype == torch.float32 and weight.numel() == hidden, "add_rmsnorm: weight must be float32 [hidden]")
    _need(out.is_contiguous() and out.shape[-1] == hidden and out.shape[0] >= n, "add_rmsnorm: output shape")
    plain, parts, n_parts, stride = delta, None, 0, 0
    if _partials(delta):
        _need(delta.dtype == torch.float32 and delta.is_contiguous() and tuple(delta.shape[1:]) == tuple(residual.shape),
              "add_rmsnorm: partial sums must be float32 [S, rows, hidden]")
        plain, parts, n_parts, stride = None, delta, delta.shape[0], delta.shape[1] * delta.shape[2]
    elif delta is not None:
        _need(delta.dtype == out.dtype and delta.is_contiguous() and delta.shape == residual.shape,
              "add_rmsnorm: delta must match the residual's shape and the output's dtype")
    _check(lib("rowwise").kl_add_rmsnorm(_ptr(residual), _ptr(plain), _ptr(parts), n_parts, ctypes.c_longlong(stride),
                                         _ptr(weight), _ptr(out), _ptr(rows), n, hidden, ctypes.c_float(eps),
                                         dtype_code(out.dtype), _stream()), "add_rmsnorm")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    _cuda(gate_up, out)
    tokens, two_i = gate_up.shape
    _need(two_i % 2 == 0 and out.shape == (tokens, two_i // 2), "swiglu: shapes")
    _need(gate_up.is_contiguous() and out.is_contiguous() and gate_up.dtype == out.dtype, "swiglu: layout")
    _check(lib("rowwise").kl_swiglu(_ptr(gate_up), _ptr(out), tokens, two_i // 2, dtype_code(out.dtype), _stream()),
           "swiglu")


# --------------------------------------------------------------------------- position encoding + cache write

def rope_kv_write(qkv: torch.Tensor, inv_freq: Optional[torch.Tensor], rotary_dim: int, positions: torch.Tensor,
                  token_slot: torch.Tensor, block_table: torch.Tensor, k_cache: Optional[torch.Tensor],
                  v_cache: Optional[torch.Tensor], num_heads: int, num_kv_heads: int, head_dim: int,
                  partials: Optional[torch.Tensor] = None) -> None:
    """Rotate the query heads of ``qkv`` [tokens, (H + 2 KV) * hd] in place; rotate the key
    heads and store them, and the value heads, into the paged cache
    [pages, KV, PAGE, hd] (skipped when both caches are None).  With ``partials`` (float32
    [S, tokens, width]) the projections are the sum of those pieces and ``qkv`` only receives
    the rotated queries."""
    _cuda(qkv, inv_freq, positions, token_slot, block_table, k_cache, v_cache, partials)
    n_parts, stride = 0, 0
    if partials is not None:
        _need(partials.dtype == torch.float32 and partials.is_contiguous() and tuple(partials.shape[1:]) == tuple(qkv.shape),
              "rope_kv_write: partial sums must be float32 [S, tokens, width]")
        n_parts, stride = partials.shape[0], partials.shape[1] * partials.shape[2]
    _i32(positions, "positions"); _i32(token_slot, "token_slot"); _i32(block_table, "block_table")
    n = qkv.shape[0]
    _need(qkv.is_contiguous() and qkv.shape[1] == (num_heads + 2 * num_kv_heads) * head_dim, "rope_kv_write: qkv shape")
    _need(positions.numel() >= n and token_slot.numel() >= n, "rope_kv_write: one position and slot per token")
    write = k_cache is not None
    if write:
        _need(v_cache is not None and k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype, "rope_kv_write: cache dtype")
        _need(k_cache.is_contiguous() and v_cache.is_contiguous()
              and tuple(k_cache.shape[1:]) == (num_kv_heads, PAGE, head_dim) and k_cache.shape == v_cache.shape,
              "rope_kv_write: cache layout must be [pages, kv_heads, 64, head_dim]")
    if rotary_dim:
        _need(inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rotary_dim // 2,
              "rope_kv_write: inv_freq must be float32 [rotary_dim / 2]")
    _check(lib("rope_kv").kl_rope_kv_write(_ptr(qkv), _ptr(partials), n_parts, ctypes.c_longlong(stride),
                                           _ptr(inv_freq), rotary_dim, _ptr(positions), _ptr(token_slot),
                                           _ptr(block_table), block_table.shape[1], _ptr(k_cache), _ptr(v_cache), n,
                                           num_heads, num_kv_heads, head_dim, int(write), dtype_code(qkv.dtype),
                                           _stream()), "rope_kv_write")


# --------------------------------------------------------------------------- attention

def attention_simt(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                   block_table: torch.Tensor, positions: torch.Tensor, token_slot: torch.Tensor, n_tokens: int,
                   num_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: int = 0) -> None:
    """out[t, h] = softmax(scale * q[t, h] . K[slot_t, lo..pos_t]) V over the paged cache."""
    _cuda(q, out, k_cache, v_cache, block_table, positions, token_slot)
    _i32(positions, "positions"); _i32(token_slot, "token_slot"); _i32(block_table, "block_table")
    _need(out.is_contiguous() and out.shape[0] >= n_tokens and out.shape[1] == num_heads * head_dim, "attention: out shape")
    _need(q.dtype == out.dtype == k_cache.dtype == v_cache.dtype, "attention: dtypes differ")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous()
          and tuple(k_cache.shape[1:]) == (num_kv_heads, PAGE, head_dim), "attention: cache layout")
    _need(head_dim % 16 == 0 and head_dim <= 256, f"attention: head_dim {head_dim} must be a multiple of 16 up to 256")
    _need(num_heads % num_kv_heads == 0, "attention: heads must be a multiple of kv heads")
    _check(lib("attention_simt").kl_attention_simt(_ptr(q), q_stride, _ptr(out), _ptr(k_cache), _ptr(v_cache),
                                                   _ptr(block_table), block_table.shape[1], _ptr(positions),
                                                   _ptr(token_slot), n_tokens, num_heads, num_kv_heads, head_dim,
                                                   ctypes.c_float(scale), int(window or 0), dtype_code(q.dtype),
                                                   _stream()), "attention_simt")


# --------------------------------------------------------------------------- matrix products

def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T in plain 32-bit FMA arithmetic; any size."""
    _cuda(a, w, out)
    (M, K), (N, K2) = a.shape, w.shape
    _need(K == K2 and out.shape[0] >= M and out.shape[1] == N, f"gemm: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    _need(a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1, "gemm: rows must be contiguous")
    _need(a.dtype == w.dtype, "gemm: operand dtypes differ")
    _check(lib("gemm_simt").kl_gemm_simt(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), M, N, K,
                                         dtype_code(a.dtype), dtype_code(out.dtype), _stream()), "gemm_simt")


# --------------------------------------------------------------------------- sampling

def argmax_rows(logits: torch.Tensor, out: torch.Tensor) -> None:
    _cuda(logits, out)
    _i32(out, "out")
    rows, vocab = logits.shape
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1 and out.numel() >= rows, "argmax: layout")
    L = lib("sampling")
    sv = si = None
    launches = 1
    if vocab >= 16384:                                              # wide rows: many CTAs per row, then one pick
        chunks = L.kl_argmax_chunks(vocab)
        sv = torch.empty((rows, chunks), dtype=torch.float32, device=logits.device)
        si = torch.empty((rows, chunks), dtype=torch.int32, device=logits.device)
        launches = 2
    _check(L.kl_argmax_rows(_ptr(logits), ctypes.c_longlong(logits.stride(0)), rows, vocab, _ptr(out), _ptr(sv), _ptr(si),
                            _stream()), "argmax_rows", launches)


def sample_rows(logits: torch.Tensor, temperature: float, top_k: int, seed: int, request_ids: torch.Tensor,
                steps: torch.Tensor, out: torch.Tensor) -> None:
    _cuda(logits, request_ids, steps, out)
    _i32(out, "out"); _i32(request_ids, "request_ids"); _i32(steps, "steps")
    rows, vocab = logits.shape
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "sample: layout")
    _need(request_ids.numel() >= rows and steps.numel() >= rows and out.numel() >= rows, "sample: one id and step per row")
    _need(temperature > 0, "sample: temperature must be positive (0 means argmax)")
    _check(lib("sampling").kl_sample_rows(_ptr(logits), ctypes.c_longlong(logits.stride(0)), rows, vocab,
                                          ctypes.c_float(temperature), int(top_k or 0),
                                          ctypes.c_ulonglong(seed & (2**64 - 1)), _ptr(request_ids), _ptr(steps),
                                          _ptr(out), _stream()), "sample_rows")


def token_logprob(logits: torch.Tensor, tokens: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """float32 [rows]: log softmax(logits[row])[tokens[row]]."""
    _cuda(logits, tokens, out)
    _i32(tokens, "tokens")
    rows, vocab = logits.shape
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1 and tokens.numel() >= rows, "token_logprob: layout")
    if out is None:
        out = torch.empty(rows, dtype=torch.float32, device=logits.device)
    _need(out.dtype == torch.float32 and out.is_contiguous() and out.numel() >= rows, "token_logprob: out")
    _check(lib("sampling").kl_token_logprob(_ptr(logits), ctypes.c_longlong(logits.stride(0)), rows, vocab, _ptr(tokens),
                                            _ptr(out), _stream()), "token_logprob")
    return out


# --------------------------------------------------------------------------- dispatch by dtype and shape

_device_words: Dict[int, torch.Tensor] = {}


def device_words(device: torch.device) -> torch.Tensor:
    """Two int32 words per device through which kernels report what the host must not miss:
    word 0 is the status word (kernels with bounded waits write a non-zero code into it when a
    wait runs out), word 1 the flag that the embedding kernel sets when it meets a token id
    outside the vocabulary.  ``check_device_words`` reads both with one copy."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _device_words:
        _device_words[idx] = torch.zeros(2, dtype=torch.int32, device=device)
    return _device_words[idx]


def status_word(device: torch.device) -> torch.Tensor:
    return device_words(device)[0:1]


def _status_ptr(device: torch.device) -> ctypes.c_void_p:
    """The status word's address (word 0 of ``device_words``) for a launch, without a tensor view."""
    return ctypes.c_void_p(device_words(device).data_ptr())


def error_word(device: torch.device) -> torch.Tensor:
    return device_words(device)[1:2]


class TokenIdError(ValueError):
    """A token id outside the vocabulary reached the embedding kernel."""


def check_device_words(device: torch.device) -> None:
    """Read both words (that synchronises), clear what was set, and raise for it: ``KernelError``
    for a wait that ran out (whatever the kernels wrote after it is not to be trusted),
    ``TokenIdError`` for a bad token id."""
    words = device_words(device)
    status, bad_id = words.tolist()
    if status or bad_id:
        words.zero_()
    if status:
        raise KernelError(f"a tensor-core kernel gave up waiting (code {status}: 1 = loader, 2 = MMA issuer, 3 = epilogue); "
                          "the results of this run are not valid")
    if bad_id:
        raise TokenIdError("a token id outside the vocabulary reached the embedding kernel")


def check_status(device: torch.device) -> None:
    """The status word alone (the token-id flag is left as it is)."""
    word = status_word(device)
    code = int(word.item())
    if code:
        word.zero_()
        raise KernelError(f"a tensor-core kernel gave up waiting (code {code}: 1 = loader, 2 = MMA issuer, 3 = epilogue)")


def _tc_ok(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor]) -> bool:
    """Whether the TMA-fed tensor-core kernels take these operands: bfloat16, rows that start
    on 16-byte boundaries (K and the row strides multiples of 8 elements).  ``out`` None: the
    kernel's own float32 pieces."""
    K = a.shape[1]
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and (out is None or (out.dtype in (torch.bfloat16, torch.float32) and out.stride(1) == 1))
            and K % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and a.stride(1) == 1 and w.stride(1) == 1)


_sm_counts: Dict[int, int] = {}


def sm_count(device: Optional[torch.device] = None) -> int:
    """Streaming multiprocessors of ``device`` (default: the current one), asked of the driver once."""
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    if idx not in _sm_counts:
        _sm_counts[idx] = int(torch.cuda.get_device_properties(idx).multi_processor_count)
    return _sm_counts[idx]


def skinny_splits(N: int, K: int, M: int = 1) -> int:
    """Into how many pieces the K range is cut for a product with few tokens, so that about two
    CTAs per SM stream weights: 128 output features per CTA, at least 4 k-blocks of 64 each.
    Every piece is written as float32 [M, N] and read again by the kernel that adds the pieces, so
    with many tokens and a short k range fewer pieces are better: their bytes stay under a quarter
    of the weights' (pieces * M * 4 <= K * 2 / 4)."""
    tiles = ((N + 127) // 128) * max(1, (M + 127) // 128)    # CTAs per cut: weight tiles x token tiles (of 128 beyond 64 tokens)
    k_blocks = (K + 63) // 64
    # never more CTAs than the two per SM that are resident at once: one CTA too many is a second round
    want = max(1, min((2 * sm_count()) // tiles, k_blocks // 4, 32, max(1, K // (8 * max(M, 1)))))
    per = (k_blocks + want - 1) // want
    return (k_blocks + per - 1) // per


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, swiglu: bool = False) -> None:
    """out[M, N] = a @ w^T on the tensor cores, tokens as tile rows (any M; pairs of CTAs on tiles of
    256 tokens where the token count suits, single CTAs on tiles of 128 otherwise).  With ``swiglu``
    the rows of ``w`` alternate 64 gate rows and 64 up rows and out[M, N / 2] receives
    silu(gate) * up."""
    _cuda(a, w, out)
    (M, K), (N, K2) = a.shape, w.shape
    _need(K == K2 and out.shape[0] >= M and out.shape[1] == (N // 2 if swiglu else N), "gemm_tcgen05: shapes")
    _need(not swiglu or (N % 128 == 0 and out.dtype == torch.bfloat16), "gemm_tcgen05: swiglu needs N % 128 == 0 and bf16 out")
    _need(_tc_ok(a, w, out), "gemm_tcgen05: operands must be bfloat16 with 16-byte aligned rows")
    _check(lib("gemm_tcgen05").kl_gemm_tcgen05(_ptr(a), ctypes.c_longlong(a.stride(0)), _ptr(w),
                                               ctypes.c_longlong(w.stride(0)), _ptr(out), ctypes.c_longlong(out.stride(0)),
                                               M, N, K, int(out.dtype == torch.float32), int(swiglu),
                                               _status_ptr(a.device), _stream()), "gemm_tcgen05")


# arguments of kl_gemm_tcgen05_skinny that switch the residual-stream forms off
_NO_STREAM_FUSION = (ctypes.c_void_p(0), 0, ctypes.c_float(0.0), ctypes.c_void_p(0), ctypes.c_void_p(0), ctypes.c_void_p(0),
                     ctypes.c_void_p(0), ctypes.c_void_p(0))

STREAM_FUSION_MAX_ROWS = 64
STREAM_SINK_MAX_ROWS = 4        # measured on the 8B shape: faster than a norm kernel of its own up to 4 rows, slower from 8


def stream_fusable(rows: int, w: torch.Tensor) -> bool:
    """Whether a product of ``rows`` tokens with ``w`` can add its result into the float32 residual
    stream, or apply a norm's 1 / rms to its rows, inside the kernel (decode steps, bfloat16)."""
    return (rows <= STREAM_FUSION_MAX_ROWS and w.dtype == torch.bfloat16 and w.is_cuda and w.shape[1] % 8 == 0
            and w.stride(1) == 1 and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0)


def gemm_skinny_stream(w: torch.Tensor, a: torch.Tensor, row_scale=None, sink=None, swiglu: bool = False,
                       splits: Optional[int] = None):
    """A decode step's product with the residual stream folded in (see gemm_tcgen05.cu).

    ``a``: bfloat16 [M, K].  ``row_scale`` = (ss float32 [pieces, 64], eps): row m of the result is
    multiplied by rsqrt(sum_p ss[p, m] / K + eps); with a = bf16(x * norm_weight) that is the
    product of the normalised rows of x.
    Result: with ``sink`` = (stream float32 [M, N], next norm's weight float32 [N] or None) the
    product is added into the stream and (ss float32 [N / 128 tiles, 64], bf16(stream * weight)
    [M, N] or None) comes back; with ``swiglu`` a bfloat16 [M, N / 2] tensor; else float32 pieces
    [S, M, N]."""
    N, K = w.shape
    M = a.shape[0]
    _cuda(a, w)
    _need(a.dtype == torch.bfloat16 and a.shape[1] == K and a.stride(1) == 1 and a.stride(0) % 8 == 0
          and a.data_ptr() % 16 == 0, "gemm_skinny_stream: activations")
    _need(stream_fusable(M, w), "gemm_skinny_stream: shape or layout not supported")
    if row_scale is not None:
        ss, eps = row_scale
        _cuda(ss)
        _need(ss.dtype == torch.float32 and ss.is_contiguous() and ss.dim() == 2 and ss.shape[1] == 64,
              "gemm_skinny_stream: sums of squares")
        scale_args = (_ptr(ss), ss.shape[0], ctypes.c_float(eps))
    else:
        scale_args = (ctypes.c_void_p(0), 0, ctypes.c_float(0.0))
    dev = w.device
    L = lib("gemm_tcgen05")
    st = _status_ptr(dev)
    null = ctypes.c_void_p(0)
    if swiglu:
        _need(sink is None and N % 128 == 0, "gemm_skinny_stream: swiglu")
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=dev)
        _check(L.kl_gemm_tcgen05_skinny(_ptr(a), ctypes.c_longlong(a.stride(0)), _ptr(w), ctypes.c_longlong(w.stride(0)), _ptr(out),
                                        ctypes.c_longlong(out.stride(0)), M, N, K, 1, 0, 1, *scale_args, null, null, null, null,
                                        null, st, _stream()), "gemm_skinny_stream")
        return out
    splits = skinny_splits(N, K, M) if splits is None else splits
    partial = torch.empty((splits, M, N), dtype=torch.float32, device=dev)
    result = partial
    sink_args = (null, null, null, null, null)
    if sink is not None:
        stream, next_w = sink
        _cuda(stream)
        _need(stream.dtype == torch.float32 and stream.is_contiguous() and tuple(stream.shape) == (M, N), "gemm_skinny_stream: sink")
        tiles = (N + 127) // 128
        ss_out = torch.empty((tiles, 64), dtype=torch.float32, device=dev)
        scaled = None
        if next_w is not None:
            _cuda(next_w)
            _need(next_w.dtype == torch.float32 and next_w.is_contiguous() and next_w.numel() == N, "gemm_skinny_stream: norm weight")
            scaled = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        sink_args = (_ptr(stream), _ptr(ss_out), _ptr(_zero_counters(dev, tiles, "gemm")),
                     _ptr(next_w) if next_w is not None else null, _ptr(scaled) if scaled is not None else null)
        result = (ss_out, scaled)
    _check(L.kl_gemm_tcgen05_skinny(_ptr(a), ctypes.c_longlong(a.stride(0)), _ptr(w), ctypes.c_longlong(w.stride(0)), _ptr(partial),
                                    ctypes.c_longlong(N), M, N, K, splits, 1, 0, *scale_args, *sink_args, st, _stream()),
           "gemm_skinny_stream")
    return result


# Which way round a product of M tokens and N features runs.  Weights as tile rows (tiles of 128
# features x 16 to 128 tokens, the K range cut so that all SMs stream): every weight crosses from HBM
# once and 16 KB of it per CTA and k block.  Tokens as tile rows (128 x 256 or 256 x 256): both operands
# are reused, but a product of 128 tokens and 4,096 features has 16 tiles for 148 SMs (8B shape, 96
# sequences: 7.6 ms per decode step that way, 5.5 ms with weights as rows).  Measured per product on
# the 8B shape, us with tokens / weights as rows:
#   128 tokens: q/k/v (24 tiles) 29.2 / 18.2, output (16) 26.7 / 13.9, gate/up (112) 43.1 / 53.6, down (16) 82.9 / 28.9
#   384 tokens: q/k/v (72) 29.6 / 23.2, output (48) 26.8 / 21.7, gate/up (336) 85.0 / -, down (48) 82.6 / 46.1
#   512 tokens: q/k/v (96) 27.6 / 34.1, output (64) 24.2 / 21.9, down (64) 70.2 / 58.5
# and on the 1B shape at 128 tokens: gate/up (64 tiles) 18.0 / 25.9.  So beyond 64 tokens: weights as rows
# while the other way has fewer tiles than 0.6 of the SMs; the gate/up product, whose K range cannot be
# cut (its epilogue needs whole sums), while it has fewer than a third of them, and already from 33 tokens on
# (8B shape, ms per decode step with the gate/up product's weights / tokens as rows: 48 sequences 4.06 / 4.02,
# 64 sequences 4.44 / 4.36; 24 and 32 sequences, were they included: 3.42 / 3.49 and 3.52 / 3.62).
SKINNY_MAX_ROWS = 512


SWIGLU_WEIGHT_ROWS_MAX = 32     # tokens up to which the gate/up product takes the weights as tile rows


def weights_as_rows(M: int, N: int, swiglu: bool = False) -> bool:
    if M <= (SWIGLU_WEIGHT_ROWS_MAX if swiglu else 64):
        return True
    if M > SKINNY_MAX_ROWS:
        return False
    tiles = ((M + 127) // 128) * ((N + 255) // 256)
    return tiles * 3 < sm_count() if swiglu else tiles * 5 < sm_count() * 3


def gemm_skinny_partials(a: torch.Tensor, w: torch.Tensor, splits: Optional[int] = None) -> Optional[torch.Tensor]:
    """The pieces of a @ w^T for few tokens (``weights_as_rows``) as float32 [S, M, N], for a consumer that adds
    them itself (the norm after a projection, the rotary kernel after q/k/v); None when the
    product is not cut (S == 1) or the operands do not fit the tensor-core kernel."""
    (M, K), (N, K2) = a.shape, w.shape
    if not weights_as_rows(M, N) or a.dtype != torch.bfloat16 or K != K2:
        return None
    if not _tc_ok(a, w, None):
        return None
    splits = skinny_splits(N, K, M) if splits is None else splits
    if splits <= 1:
        return None
    partial = torch.empty((splits, M, N), dtype=torch.float32, device=a.device)
    _check(lib("gemm_tcgen05").kl_gemm_tcgen05_skinny(
        _ptr(a), ctypes.c_longlong(a.stride(0)), _ptr(w), ctypes.c_longlong(w.stride(0)), _ptr(partial),
        ctypes.c_longlong(N), M, N, K, splits, 1, 0, *_NO_STREAM_FUSION, _status_ptr(a.device), _stream()),
        "gemm_skinny")
    return partial


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, splits: Optional[int] = None,
                swiglu: bool = False) -> None:
    """out[M, N] = a @ w^T for M <= SKINNY_MAX_ROWS tokens: weights as tile rows, each weight read once, the
    K range cut into ``splits`` pieces whose float32 partial sums are added in a fixed order.
    With ``swiglu`` (rows of ``w`` alternate 64 gate and 64 up rows; no cut) out[M, N / 2]
    receives silu(gate) * up."""
    _cuda(a, w, out)
    (M, K), (N, K2) = a.shape, w.shape
    _need(K == K2 and out.shape[0] >= M and out.shape[1] == (N // 2 if swiglu else N) and M <= SKINNY_MAX_ROWS, "gemm_skinny: shapes")
    _need(_tc_ok(a, w, out), "gemm_skinny: operands must be bfloat16 with 16-byte aligned rows")
    _need(not swiglu or (N % 128 == 0 and out.dtype == torch.bfloat16), "gemm_skinny: swiglu needs N % 128 == 0 and bf16 out")
    splits = 1 if swiglu else (skinny_splits(N, K, M) if splits is None else splits)
    L = lib("gemm_tcgen05")
    st = _status_ptr(a.device)
    if splits == 1:
        _check(L.kl_gemm_tcgen05_skinny(_ptr(a), ctypes.c_longlong(a.stride(0)), _ptr(w), ctypes.c_longlong(w.stride(0)),
                                        _ptr(out), ctypes.c_longlong(out.stride(0)), M, N, K, 1,
                                        int(out.dtype == torch.float32), int(swiglu), *_NO_STREAM_FUSION, st, _stream()),
               "gemm_skinny")
        return
    partial = torch.empty((splits, M, N), dtype=torch.float32, device=a.device)
    _check(L.kl_gemm_tcgen05_skinny(_ptr(a), ctypes.c_longlong(a.stride(0)), _ptr(w), ctypes.c_longlong(w.stride(0)),
                                    _ptr(partial), ctypes.c_longlong(N), M, N, K, splits, 1, 0, *_NO_STREAM_FUSION, st,
                                    _stream()), "gemm_skinny")
    _check(L.kl_splitk_reduce(_ptr(partial), splits, M, N, _ptr(out), ctypes.c_longlong(out.stride(0)),
                              int(out.dtype == torch.float32), _stream()), "splitk_reduce")


def matmul(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out = a @ w^T with the kernel that fits the dtype and the shape.  float32 operands
    always take the plain 32-bit kernel; bfloat16 operands take the tensor-core kernels when
    their rows are 16-byte aligned (few tokens: weights as tile rows), else the plain kernel."""
    if a.dtype == torch.bfloat16 and _tc_ok(a, w, out):
        if weights_as_rows(a.shape[0], w.shape[0]):
            gemm_skinny(a, w, out)
        else:
            gemm_tcgen05(a, w, out)
    else:
        gemm_simt(a, w, out)


DECODE_HEAD_DIMS = (16, 32, 64, 128, 256)


def decode_splits(rows: int, num_heads: int, num_kv_heads: int) -> int:
    """Into how many pieces each sequence's keys are cut in decode attention: enough CTAs for
    about two per SM, from the batch size alone (never from the lengths, so that a captured
    graph stays valid while the sequences grow)."""
    group = num_heads // num_kv_heads
    tiles = (group + 3) // 4 if group >= 3 else 1
    ctas = max(1, rows * num_kv_heads * tiles)
    return max(1, min(32, (2 * sm_count() + ctas - 1) // ctas))


def attention_decode(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     block_table: torch.Tensor, positions: torch.Tensor, token_slot: torch.Tensor, rows: int,
                     num_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: int = 0,
                     splits: Optional[int] = None) -> None:
    """One query token per row against its sequence's cache, keys cut over ``splits`` CTAs."""
    _cuda(q, out, k_cache, v_cache, block_table, positions, token_slot)
    _i32(positions, "positions"); _i32(token_slot, "token_slot"); _i32(block_table, "block_table")
    _need(q.dtype == out.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16, "attention_decode: bfloat16 only")
    _need(head_dim in DECODE_HEAD_DIMS, f"attention_decode: head_dim {head_dim} not in {DECODE_HEAD_DIMS}")
    _need(out.is_contiguous() and out.shape[0] >= rows and out.shape[1] == num_heads * head_dim, "attention_decode: out shape")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous()
          and tuple(k_cache.shape[1:]) == (num_kv_heads, PAGE, head_dim), "attention_decode: cache layout")
    _need(num_heads % num_kv_heads == 0, "attention_decode: heads must be a multiple of kv heads")
    splits = decode_splits(rows, num_heads, num_kv_heads) if splits is None else splits
    po = pml = None
    if splits > 1:
        po = torch.empty((rows, num_heads, splits, head_dim), dtype=torch.float32, device=q.device)
        pml = torch.empty((rows, num_heads, splits, 2), dtype=torch.float32, device=q.device)
    _check(lib("attention_decode").kl_attention_decode(
        _ptr(q), q_stride, _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
        _ptr(positions), _ptr(token_slot), _ptr(po), _ptr(pml), rows, num_heads, num_kv_heads, head_dim,
        ctypes.c_float(scale), int(window or 0), splits, _stream()), "attention_decode", 2 if splits > 1 else 1)


MMA_HEAD_DIMS = (64, 128)


def attention_mma(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  block_table: torch.Tensor, cu_tokens: torch.Tensor, seq_slots: torch.Tensor, seq_starts: torch.Tensor,
                  seq_new: torch.Tensor, n_seqs: int, max_new: int, n_rows: int, num_heads: int, num_kv_heads: int,
                  head_dim: int, scale: float, window: int = 0, splits: int = 1, few_rows: bool = False) -> None:
    """Tensor-core attention of a ragged batch over the paged cache (bfloat16, head sizes 64
    and 128).  ``few_rows``: the layout for one token per sequence; ``splits``: pieces each
    sequence's pages are cut into."""
    _cuda(q, out, k_cache, v_cache, block_table, cu_tokens, seq_slots, seq_starts, seq_new)
    for t, nm in ((block_table, "block_table"), (cu_tokens, "cu_tokens"), (seq_slots, "seq_slots"),
                  (seq_starts, "seq_starts"), (seq_new, "seq_new")):
        _i32(t, nm)
    _need(q.dtype == out.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16, "attention_mma: bfloat16 only")
    _need(head_dim in MMA_HEAD_DIMS, f"attention_mma: head_dim {head_dim} not in {MMA_HEAD_DIMS}")
    _need(out.is_contiguous() and out.shape[0] >= n_rows and out.shape[1] == num_heads * head_dim, "attention_mma: out shape")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous()
          and tuple(k_cache.shape[1:]) == (num_kv_heads, PAGE, head_dim), "attention_mma: cache layout")
    _need(num_heads % num_kv_heads == 0 and num_heads // num_kv_heads <= 16, "attention_mma: group size up to 16")
    po = pml = None
    if splits > 1:
        po = torch.empty((n_rows, num_heads, splits, head_dim), dtype=torch.float32, device=q.device)
        pml = torch.empty((n_rows, num_heads, splits, 2), dtype=torch.float32, device=q.device)
    _check(lib("attention_mma").kl_attention_mma(
        _ptr(q), q_stride, _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
        _ptr(cu_tokens), _ptr(seq_slots), _ptr(seq_starts), _ptr(seq_new), _ptr(po), _ptr(pml), n_seqs, max_new, n_rows,
        num_heads, num_kv_heads, head_dim, ctypes.c_float(scale), int(window or 0), splits, int(few_rows), _stream()),
        "attention_mma", 2 if splits > 1 else 1)


def swiglu_fusable(hidden: int, inter: int, dtype: torch.dtype) -> bool:
    """Whether gate and up can be one product whose epilogue applies silu(gate) * up: bfloat16,
    rows on 16-byte boundaries, and an intermediate size that is a multiple of 64 (the weights
    are then stored as alternating blocks of 64 gate rows and 64 up rows)."""
    return dtype == torch.bfloat16 and inter % 64 == 0 and hidden % 8 == 0


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[I, K] and [I, K] -> [2 I, K]: 64 gate rows, the 64 up rows of the same features, and so on."""
    inter, k = gate.shape
    return torch.stack([gate.view(inter // 64, 64, k), up.view(inter // 64, 64, k)], dim=1).reshape(2 * inter, k).contiguous()


def matmul_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, I] = silu(a @ gate^T) * (a @ up^T) in one kernel; ``w_gate_up`` from ``interleave_gate_up``."""
    if weights_as_rows(a.shape[0], w_gate_up.shape[0], swiglu=True):
        gemm_skinny(a, w_gate_up, out, swiglu=True)
    else:
        gemm_tcgen05(a, w_gate_up, out, swiglu=True)


def attention_tcgen05(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      block_table: torch.Tensor, cu_tokens: torch.Tensor, seq_slots: torch.Tensor, seq_starts: torch.Tensor,
                      seq_new: torch.Tensor, n_seqs: int, max_new: int, n_rows: int, num_heads: int, num_kv_heads: int,
                      head_dim: int, scale: float) -> None:
    """Prefill attention with both products on tcgen05 (bfloat16, head size 64 or 128, no window)."""
    _cuda(q, out, k_cache, v_cache, block_table, cu_tokens, seq_slots, seq_starts, seq_new)
    for t, nm in ((block_table, "block_table"), (cu_tokens, "cu_tokens"), (seq_slots, "seq_slots"),
                  (seq_starts, "seq_starts"), (seq_new, "seq_new")):
        _i32(t, nm)
    _need(q.dtype == out.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16, "attention_tcgen05: bfloat16 only")
    _need(head_dim in (64, 128) and q_stride % 8 == 0 and q.data_ptr() % 16 == 0, "attention_tcgen05: head_dim 64 or 128, aligned rows")
    _need(out.is_contiguous() and out.shape[0] >= n_rows and out.shape[1] == num_heads * head_dim, "attention_tcgen05: out shape")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous()
          and tuple(k_cache.shape[1:]) == (num_kv_heads, PAGE, head_dim), "attention_tcgen05: cache layout")
    _need(q.shape[0] >= n_rows, "attention_tcgen05: q rows")
    cache_rows = k_cache.shape[0] * num_kv_heads * PAGE
    _check(lib("attention_tcgen05").kl_attention_tcgen05(
        _ptr(q), q_stride, _ptr(out), _ptr(k_cache), _ptr(v_cache), ctypes.c_longlong(cache_rows), _ptr(block_table),
        block_table.shape[1], _ptr(cu_tokens), _ptr(seq_slots), _ptr(seq_starts), _ptr(seq_new), n_seqs, max_new,
        q.shape[0], num_heads, num_kv_heads, head_dim, ctypes.c_float(scale), _status_ptr(q.device), _stream()),
        "attention_tcgen05")


# Which kernel prefill steps of the bfloat16 path use for head sizes 64 and 128: "tcgen05", or "mma"
# (the kernel that serves windows and other group sizes).  Kept as a switch so that tests can run
# whole models through the second kernel too (tests/test_gpu_schedules.py).
PREFILL_KERNEL = "tcgen05"

_counters: Dict[tuple, torch.Tensor] = {}


COUNTERS = 1 << 18     # int32 counters per device and use (1 MiB): one per (sequence, kv head) or per tile


def _zero_counters(device: torch.device, n: int, use: str = "attention") -> torch.Tensor:
    """int32 counters that kernels leave at zero (the last CTA of a group resets its own); one
    buffer per device and per use, so that kernels of different kinds never share a counter.
    The buffer is made once and never replaced: captured graphs and kernels in flight hold its
    address."""
    idx = (device.index if device.index is not None else torch.cuda.current_device(), use)
    have = _counters.get(idx)
    if have is None:
        have = _counters[idx] = torch.zeros(COUNTERS, dtype=torch.int32, device=device)
    _need(n <= COUNTERS, f"{use}: {n} counters wanted, {COUNTERS} exist")
    return have


def decode_attention_splits(n_seqs: int, num_kv_heads: int, head_dim: int = 128, context_class: int = 0) -> int:
    """Pieces a sequence's keys are cut into for the tensor-core decode kernel.

    Up to 1,024 tokens (``context_class`` 0; the engine's class of the longest sequence: 16 pages,
    then one class per doubling): as many as keep all CTAs in one round (three CTAs fit an SM, four
    with a head size of 64), at most 16.  A CTA's time is its chain of pages, so a second round
    costs more than longer chains (32 sequences of 8 kv heads, 512 tokens: 27 us with one piece,
    35 us with two).  For longer sequences, measured on the 8B shape inside the decode step:

    * where one round has room for two pieces or more per (sequence, kv head) pair: still one
      round, but up to a piece per four pages (1 sequence of 32,768 tokens: 55 pieces 166 us per
      layer, 16 pieces 200 us; 2 sequences: 27 pieces 169 us, 16 pieces 197 us);
    * where it has not, but two pieces per pair fit the light CTAs' round of four per SM: two
      pieces beyond 4,096 tokens (32 sequences of 8,300 tokens: 307 against 334 us per layer; of
      2,100 tokens: 192 against 191 us; more pieces in more rounds were never faster)."""
    pairs = max(1, n_seqs * num_kv_heads)
    places = (4 if head_dim == 64 else 3) * sm_count()
    one_round = max(1, places // pairs)
    if context_class <= 0:
        return min(16, one_round)
    pages = 16 << context_class                          # the class's longest sequence
    if one_round >= 2:
        return max(1, min(one_round, max(16, pages // 4)))
    if context_class >= 3 and head_dim == 128 and pairs * 2 <= 4 * sm_count():
        return 2
    return 1


def decode_fusable(dtype: torch.dtype, head_dim: int, rotary_dim: int, num_heads: int, num_kv_heads: int) -> bool:
    """Whether a decode step's rotation, cache write, attention and split merge run as one kernel."""
    return (dtype == torch.bfloat16 and head_dim in MMA_HEAD_DIMS and rotary_dim == head_dim
            and num_heads % num_kv_heads == 0 and num_heads // num_kv_heads <= 16)


def attention_decode_fused(qkv: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor,
                           v_cache: torch.Tensor, block_table: torch.Tensor, step, num_heads: int, num_kv_heads: int,
                           head_dim: int, scale: float, window: int = 0, splits: Optional[int] = None) -> None:
    """One token per sequence (a decode step, rows in sequence order, no padding rows).  ``qkv``
    is the q/k/v projection, bfloat16 [rows, (H + 2 KV) * hd] or float32 pieces [S, rows, width].
    Rotates q and k, appends k and v to the cache, attends, merges the splits: one kernel."""
    _cuda(qkv, inv_freq, out, k_cache, v_cache, block_table)
    n = step.n_seqs
    _need(step.is_decode and step.n_tokens == n, "attention_decode_fused: one token per sequence and no padding rows")
    _need(decode_fusable(out.dtype, head_dim, 2 * inv_freq.numel(), num_heads, num_kv_heads), "attention_decode_fused: not fusable")
    width = (num_heads + 2 * num_kv_heads) * head_dim
    parts, plain, n_parts, stride = None, None, 0, 0
    if qkv.dim() == 3:
        _need(qkv.dtype == torch.float32 and qkv.is_contiguous() and tuple(qkv.shape[1:]) == (n, width), "attention_decode_fused: pieces")
        parts, n_parts, stride = qkv, qkv.shape[0], n * width
    else:
        _need(qkv.dtype == torch.bfloat16 and qkv.is_contiguous() and tuple(qkv.shape) == (n, width), "attention_decode_fused: qkv")
        plain = qkv
    _need(out.is_contiguous() and out.shape[0] >= n and out.shape[1] == num_heads * head_dim, "attention_decode_fused: out shape")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.dtype == torch.bfloat16
          and tuple(k_cache.shape[1:]) == (num_kv_heads, PAGE, head_dim), "attention_decode_fused: cache layout")
    _need(inv_freq.dtype == torch.float32 and inv_freq.numel() == head_dim // 2, "attention_decode_fused: inv_freq")
    _need(all(t.data_ptr() % 16 == 0 for t in (qkv, inv_freq, out, k_cache, v_cache)), "attention_decode_fused: 16-byte aligned operands")
    if splits is None:
        splits = decode_attention_splits(n, num_kv_heads, head_dim, getattr(step, "context_class", 0))
    po = pml = None
    if splits > 1:
        po = torch.empty((n, num_heads, splits, head_dim), dtype=torch.float32, device=out.device)
        pml = torch.empty((n, num_heads, splits, 2), dtype=torch.float32, device=out.device)
    counters = _zero_counters(out.device, n * num_kv_heads)
    _check(lib("attention_mma").kl_attention_decode_fused(
        _ptr(plain), _ptr(parts), n_parts, ctypes.c_longlong(stride), _ptr(inv_freq), _ptr(out), _ptr(k_cache), _ptr(v_cache),
        _ptr(block_table), block_table.shape[1], _ptr(step.cu_tokens), _ptr(step.seq_slots), _ptr(step.seq_starts),
        _ptr(step.seq_new), _ptr(po), _ptr(pml), _ptr(counters), n, num_heads, num_kv_heads, head_dim, ctypes.c_float(scale),
        int(window or 0), splits, _stream()), "attention_decode_fused")


# Which kernel decode steps of the bfloat16 path use when both fit: "mma" (tensor cores) or
# "simt" (attention_decode.cu, which otherwise serves head sizes 16, 32 and 256); a switch for tests.
DECODE_KERNEL = "mma"


def attention(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
              block_table: torch.Tensor, step, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
              window: int = 0) -> None:
    """Attention of every token of ``step`` over its sequence's cache.  The bfloat16 path
    takes the tensor-core kernel (head sizes 64 and 128) or, for decode steps with other head
    sizes, the split-KV kernel; float32 and everything else takes the plain kernel."""
    bf = q.dtype == torch.bfloat16
    group = num_heads // num_kv_heads
    if (bf and not step.is_decode and PREFILL_KERNEL == "tcgen05" and head_dim in (64, 128) and not window and group <= 128
            and q_stride % 8 == 0 and q.data_ptr() % 16 == 0 and step.max_new >= 8):
        attention_tcgen05(q, q_stride, out, k_cache, v_cache, block_table, step.cu_tokens, step.seq_slots, step.seq_starts,
                          step.seq_new, step.n_seqs, step.max_new, step.n_tokens, num_heads, num_kv_heads, head_dim, scale)
    elif bf and head_dim in MMA_HEAD_DIMS and group <= 16 and (not step.is_decode or DECODE_KERNEL == "mma"):
        splits = 1
        if step.is_decode:
            splits = decode_attention_splits(step.n_seqs, num_kv_heads, head_dim, getattr(step, "context_class", 0))
        attention_mma(q, q_stride, out, k_cache, v_cache, block_table, step.cu_tokens, step.seq_slots, step.seq_starts,
                      step.seq_new, step.n_seqs, step.max_new, step.n_tokens, num_heads, num_kv_heads, head_dim, scale,
                      window, splits, few_rows=step.is_decode)
    elif bf and step.is_decode and head_dim in DECODE_HEAD_DIMS and q_stride % 8 == 0:
        attention_decode(q, q_stride, out, k_cache, v_cache, block_table, step.positions, step.token_slot, step.n_tokens,
                         num_heads, num_kv_heads, head_dim, scale, window)
    else:
        attention_simt(q, q_stride, out, k_cache, v_cache, block_table, step.positions, step.token_slot, step.n_tokens,
                       num_heads, num_kv_heads, head_dim, scale, window)
