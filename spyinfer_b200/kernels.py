"""Python faces of the CUDA kernels: argument checks, then one C call on the current stream.

Every function takes CUDA tensors, checks device, dtype, shape and contiguity (a kernel
never sees a tensor it cannot index), and raises ``KernelError`` with the module's message
if the C side refuses the sizes.  Nothing here falls back to a library or to the CPU.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc import build

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

STATUS_MESSAGES = {
    1: "a token id outside the vocabulary (batch token index {detail})",
    2: "a position beyond the position table (batch token index {detail})",
    3: "a block-table entry that is no page of the pool (batch token index {detail})",
    4: "a wait inside it ran out of its time limit (code {detail})",
}
STATUS_WAIT_TIMEOUT = 4


class KernelError(RuntimeError):
    pass


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device is visible: this engine runs its kernels on the GPU only and has no CPU path")


def _code(t: torch.Tensor, what: str) -> int:
    if t.dtype not in _CODES:
        raise KernelError(f"{what}: dtype {t.dtype} is not supported (float32 or bfloat16)")
    return _CODES[t.dtype]


def _check(t: torch.Tensor, what: str, dtype=None, ndim=None) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{what}: expected a CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what}: expected {dtype}, found {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{what}: expected {ndim} dimensions, found shape {tuple(t.shape)}")
    if not t.is_contiguous():
        raise KernelError(f"{what}: expected a contiguous tensor, found strides {t.stride()} for shape {tuple(t.shape)}")


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


_launches = 0


def launch_count() -> int:
    """How many kernel launches this process has made through this module (a replayed CUDA
    graph counts the launches it holds)."""
    return _launches


def count_launches(n: int) -> None:
    global _launches
    _launches += n


def _call(module: str, fn: str, *args) -> None:
    global _launches
    _launches += 1
    lib = build.load(module)
    f = getattr(lib, fn)
    f.restype = ctypes.c_int
    if f(*args) != 0:
        raise KernelError(build.last_error(module))


def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = table[ids[t]]`` widened to float32.  table [V, H]; ids [T] int32; out [T, H] float32."""
    _check(table, "embedding table", ndim=2)
    _check(ids, "token ids", torch.int32, 1)
    _check(out, "embedding output", torch.float32, 2)
    T, (V, H) = ids.shape[0], table.shape
    if tuple(out.shape) != (T, H):
        raise KernelError(f"embedding output: expected shape {(T, H)}, found {tuple(out.shape)}")
    _call("embedding", "spy_embedding", _ptr(table), _code(table, "embedding table"), _ptr(ids), _ptr(out), T, H, V, _ptr(status), _stream())
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, delta: Optional[torch.Tensor] = None,
            rows: Optional[torch.Tensor] = None, write_back: bool = False) -> torch.Tensor:
    """``out = rmsnorm(x [+ delta]) * weight`` row by row; with ``write_back`` the sum is stored
    into ``x`` (the residual stream); ``rows`` gathers rows of x (and delta) into out.
    ``delta`` has x's shape, or is a stack ``[splits, rows, len]`` of partial sums (the
    unreduced output of a split-K product) that are added in order."""
    _check(x, "rmsnorm input", ndim=2)
    _check(weight, "rmsnorm weight", ndim=1)
    _check(out, "rmsnorm output", ndim=2)
    H = x.shape[1]
    if weight.shape[0] != H or out.shape[1] != H:
        raise KernelError(f"rmsnorm: row lengths differ: input {H}, weight {weight.shape[0]}, output {out.shape[1]}")
    splits, split_stride = 0, 0
    if delta is not None:
        if delta.dim() == 3:
            _check(delta, "rmsnorm delta", ndim=3)
            splits, split_stride = delta.shape[0], delta.shape[1] * delta.shape[2]
            if tuple(delta.shape[1:]) != tuple(x.shape):
                raise KernelError(f"rmsnorm: stacked delta shape {tuple(delta.shape)} does not fit input shape {tuple(x.shape)}")
        else:
            _check(delta, "rmsnorm delta", ndim=2)
            splits = 1
            if tuple(delta.shape) != tuple(x.shape):
                raise KernelError(f"rmsnorm: delta shape {tuple(delta.shape)} differs from input shape {tuple(x.shape)}")
    if rows is not None:
        _check(rows, "rmsnorm rows", torch.int32, 1)
        n = rows.shape[0]
    else:
        n = x.shape[0]
    if out.shape[0] != n:
        raise KernelError(f"rmsnorm: output has {out.shape[0]} rows, expected {n}")
    _call("rmsnorm", "spy_rmsnorm", _ptr(x), _code(x, "rmsnorm input"), _ptr(delta), _code(delta, "rmsnorm delta") if delta is not None else 0,
          splits, ctypes.c_longlong(split_stride), _ptr(rows), _ptr(weight), _code(weight, "rmsnorm weight"), _ptr(out),
          _code(out, "rmsnorm output"), n, H, ctypes.c_float(eps), int(bool(write_back)), _stream())
    return out


def build_rope_table(inv_freq: torch.Tensor, rows: int) -> torch.Tensor:
    """(cos, sin) of ``position * inv_freq[j]`` as float32 ``[rows, len(inv_freq), 2]``."""
    _check(inv_freq, "inverse frequencies", torch.float32, 1)
    table = torch.empty((rows, inv_freq.shape[0], 2), dtype=torch.float32, device=inv_freq.device)
    _call("qk_rope_store", "spy_build_rope_table", _ptr(table), _ptr(inv_freq), rows, inv_freq.shape[0], _stream())
    return table


def qk_rope_store(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, q_weight: Optional[torch.Tensor],
                  k_weight: Optional[torch.Tensor], eps: float, rope_table: Optional[torch.Tensor], positions: torch.Tensor,
                  seq_of_token: torch.Tensor, block_table: Optional[torch.Tensor], pages: Optional[torch.Tensor], store: bool = True,
                  status: Optional[torch.Tensor] = None, q_out: Optional[torch.Tensor] = None, pairing: str = "half") -> torch.Tensor:
    """Per-head RMSNorm (if weights are given) and rotation (if a table is given) of the q and k
    heads of ``qkv [T, (nh + 2 nkv) hd]``, or of a stack ``[splits, T, ...]`` of float32 partial
    products that is summed on the way.  q goes to ``q_out [T, nh hd]`` (default: in place,
    which a stack does not allow).  With ``store`` the k heads (normed, rotated) and the v heads
    go to ``pages [num_pages, 2, nkv, page_size, hd]`` through ``block_table [S, width]``.
    ``pairing``: which elements the angle ``j`` of the table rotates: ``"half"`` ``(j, j + r)``,
    ``"interleaved"`` ``(2j, 2j + 1)``.
    Returns the tensor that holds q (rows may be wider than ``nh hd``)."""
    if pairing not in ("half", "interleaved"):
        raise KernelError(f"qk_rope_store: unknown pairing rule {pairing!r}")
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if qkv.dim() == 3:
        _check(qkv, "qkv partial products", torch.float32, 3)
        splits, T = qkv.shape[0], qkv.shape[1]
        split_stride = qkv.shape[1] * qkv.shape[2]
        if q_out is None:
            raise KernelError("qk_rope_store: a stack of partial products needs q_out")
    else:
        _check(qkv, "qkv", ndim=2)
        splits, T, split_stride = 1, qkv.shape[0], 0
    if qkv.shape[-1] != width:
        raise KernelError(f"qkv: expected {width} columns, found {qkv.shape[-1]}")
    if q_out is None:
        q_out = qkv
    else:
        _check(q_out, "q output", ndim=2)
        if q_out.shape[0] != T or q_out.shape[1] < num_heads * head_dim:
            raise KernelError(f"q output: expected [{T}, >= {num_heads * head_dim}], found {tuple(q_out.shape)}")
    _check(positions, "positions", torch.int32, 1)
    _check(seq_of_token, "seq_of_token", torch.int32, 1)
    if positions.shape[0] != T or seq_of_token.shape[0] != T:
        raise KernelError("qk_rope_store: positions and seq_of_token must have one entry per token")
    w_code = 0
    if (q_weight is None) != (k_weight is None):
        raise KernelError("qk_rope_store: q and k norm weights must both be given or both be None")
    if q_weight is not None:
        _check(q_weight, "q norm weight", ndim=1)
        _check(k_weight, "k norm weight", q_weight.dtype, 1)
        if q_weight.shape[0] != head_dim or k_weight.shape[0] != head_dim:
            raise KernelError(f"qk_rope_store: norm weights must have head_dim={head_dim} elements")
        w_code = _code(q_weight, "q norm weight")
    rot_half = table_rows = 0
    if rope_table is not None:
        _check(rope_table, "rope table", torch.float32, 3)
        table_rows, rot_half = rope_table.shape[0], rope_table.shape[1]
    page_size = num_pages = table_width = cache_code = 0
    if store:
        if pages is None or block_table is None:
            raise KernelError("qk_rope_store: storing needs pages and a block table")
        _check(pages, "cache pages", ndim=5)
        _check(block_table, "block table", torch.int32, 2)
        num_pages, two, nkv, page_size, hd = pages.shape
        if two != 2 or nkv != num_kv_heads or hd != head_dim:
            raise KernelError(f"cache pages: expected [pages, 2, {num_kv_heads}, page_size, {head_dim}], found {tuple(pages.shape)}")
        table_width = block_table.shape[1]
        cache_code = _code(pages, "cache pages")
    _call("qk_rope_store", "spy_qk_rope_store", _ptr(qkv), _code(qkv, "qkv"), splits, ctypes.c_longlong(split_stride), _ptr(q_out),
          _code(q_out, "q output"), ctypes.c_longlong(q_out.shape[1]), T, num_heads, num_kv_heads, head_dim, _ptr(q_weight), _ptr(k_weight),
          w_code, ctypes.c_float(eps), _ptr(rope_table), rot_half, table_rows, _ptr(positions), _ptr(seq_of_token),
          _ptr(block_table if store else None), table_width, _ptr(pages if store else None), cache_code, page_size, num_pages,
          int(bool(store)), 0 if pairing == "half" else 1, _ptr(status), _stream())
    return q_out


def attention_generic(q: torch.Tensor, num_heads: int, head_dim: int, out: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor,
                      positions: torch.Tensor, seq_of_token: torch.Tensor, scale: float, window: Optional[int] = None,
                      status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of every token of the batch over its sequence's pages (any mix of prompt
    portions and single tokens).  ``q [T, >= nh*hd]`` (only the first nh*hd columns are read),
    ``out [T, nh*hd]``."""
    _check(q, "attention queries", ndim=2)
    _check(out, "attention output", q.dtype, 2)
    _check(pages, "cache pages", ndim=5)
    _check(block_table, "block table", torch.int32, 2)
    _check(positions, "positions", torch.int32, 1)
    _check(seq_of_token, "seq_of_token", torch.int32, 1)
    T = q.shape[0]
    num_pages, two, nkv, page_size, hd = pages.shape
    if two != 2 or hd != head_dim:
        raise KernelError(f"cache pages: expected [pages, 2, nkv, page_size, {head_dim}], found {tuple(pages.shape)}")
    if q.shape[1] < num_heads * head_dim or tuple(out.shape) != (T, num_heads * head_dim):
        raise KernelError(f"attention: q {tuple(q.shape)} / out {tuple(out.shape)} do not fit {num_heads} heads of {head_dim}")
    if positions.shape[0] != T or seq_of_token.shape[0] != T:
        raise KernelError("attention: positions and seq_of_token must have one entry per token")
    _call("attention_generic", "spy_attention_generic", _ptr(q), ctypes.c_longlong(q.shape[1]), _ptr(out), _code(q, "attention queries"),
          _ptr(pages), _code(pages, "cache pages"), _ptr(block_table), block_table.shape[1], page_size, num_pages, num_heads, nkv, head_dim,
          _ptr(positions), _ptr(seq_of_token), T, int(window or 0), ctypes.c_float(scale), _ptr(status), _stream())
    return out


_attn_scratch = {}


def attention_scratch(device, floats: int) -> torch.Tensor:
    """A float32 buffer of at least ``floats`` for the split attention kernel's partial
    results.  Buffers are kept for the life of the process (captured graphs point at them);
    a larger request makes a new one."""
    key = str(torch.device(device))
    buf = _attn_scratch.get(key)
    if buf is None or buf[-1].numel() < floats:
        size = max(floats, 1 << 20)
        _attn_scratch.setdefault(key, []).append(torch.empty(size, dtype=torch.float32, device=device))
        buf = _attn_scratch[key]
    return buf[-1]


def attention_mma_takes(num_heads: int, num_kv_heads: int, head_dim: int, dtype: torch.dtype) -> bool:
    """Whether the tensor-core attention kernel takes these sizes: bfloat16, head size 64 or
    128, at most 16 query heads per key/value head."""
    return dtype == torch.bfloat16 and head_dim in (64, 128) and num_heads % num_kv_heads == 0 and num_heads // num_kv_heads <= 16


def attention_mma(q: torch.Tensor, num_heads: int, head_dim: int, out: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor,
                  positions: torch.Tensor, q_start: torch.Tensor, num_seqs: int, scale: float, window: Optional[int] = None,
                  split_keys: int = 0, max_splits: int = 0, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Tensor-core attention of a batch over its pages.  ``split_keys == 0``: tiles mode, any
    mix of portions and single tokens.  ``split_keys > 0``: every sequence brings one token
    and its keys are cut into splits of ``split_keys`` (a multiple of 64), at most
    ``max_splits`` of them, merged through scratch memory."""
    _check(q, "attention queries", torch.bfloat16, 2)
    _check(out, "attention output", torch.bfloat16, 2)
    _check(pages, "cache pages", torch.bfloat16, 5)
    _check(block_table, "block table", torch.int32, 2)
    _check(positions, "positions", torch.int32, 1)
    _check(q_start, "q_start", torch.int32, 1)
    T = q.shape[0]
    num_pages, two, nkv, page_size, hd = pages.shape
    if two != 2 or hd != head_dim:
        raise KernelError(f"cache pages: expected [pages, 2, nkv, page_size, {head_dim}], found {tuple(pages.shape)}")
    if q.shape[1] < num_heads * head_dim or tuple(out.shape) != (T, num_heads * head_dim):
        raise KernelError(f"attention: q {tuple(q.shape)} / out {tuple(out.shape)} do not fit {num_heads} heads of {head_dim}")
    if positions.shape[0] != T or q_start.shape[0] != num_seqs + 1 or block_table.shape[0] < num_seqs:
        raise KernelError("attention: positions need one entry per token, q_start one per sequence plus one, the block table a row per sequence")
    mode = 1 if split_keys > 0 else 0
    scratch, floats = None, 0
    if mode == 1 and max_splits > 1:
        floats = num_seqs * num_heads * max_splits * (head_dim + 2)
        scratch = attention_scratch(q.device, floats)
        floats = scratch.numel()
    if status is None:
        status = status_word(q.device)
    _call("attention_mma", "spy_attention_mma", _ptr(q), ctypes.c_longlong(q.shape[1]), _ptr(out), _ptr(pages), _ptr(block_table),
          block_table.shape[1], page_size, num_pages, num_heads, nkv, head_dim, _ptr(positions), _ptr(q_start), T, num_seqs,
          int(window or 0), ctypes.c_float(scale), mode, int(split_keys), int(max_splits), _ptr(scratch), ctypes.c_longlong(floats),
          _ptr(status), _stream())
    return out


def attention_tc(q: torch.Tensor, num_heads: int, head_dim: int, out: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor,
                 positions: torch.Tensor, q_start: torch.Tensor, num_seqs: int, scale: float, window: Optional[int] = None,
                 status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of a batch over its pages on tcgen05 (blocks of two 128-row query tiles that share
    every key and value tile, scores and output in tensor memory, pages brought in by TMA): prompt
    portions, any mix.  Page sizes 8 .. 128."""
    _check(q, "attention queries", torch.bfloat16, 2)
    _check(out, "attention output", torch.bfloat16, 2)
    _check(pages, "cache pages", torch.bfloat16, 5)
    _check(block_table, "block table", torch.int32, 2)
    _check(positions, "positions", torch.int32, 1)
    _check(q_start, "q_start", torch.int32, 1)
    T = q.shape[0]
    num_pages, two, nkv, page_size, hd = pages.shape
    if two != 2 or hd != head_dim:
        raise KernelError(f"cache pages: expected [pages, 2, nkv, page_size, {head_dim}], found {tuple(pages.shape)}")
    if q.shape[1] < num_heads * head_dim or tuple(out.shape) != (T, num_heads * head_dim):
        raise KernelError(f"attention: q {tuple(q.shape)} / out {tuple(out.shape)} do not fit {num_heads} heads of {head_dim}")
    if positions.shape[0] != T or q_start.shape[0] != num_seqs + 1 or block_table.shape[0] < num_seqs:
        raise KernelError("attention: positions need one entry per token, q_start one per sequence plus one, the block table a row per sequence")
    if status is None:
        status = status_word(q.device)
    _call("attention_tc", "spy_attention_tc", _ptr(q), ctypes.c_longlong(q.shape[1]), _ptr(out), _ptr(pages), _ptr(block_table),
          block_table.shape[1], page_size, num_pages, num_heads, nkv, head_dim, _ptr(positions), _ptr(q_start), T, num_seqs,
          int(window or 0), ctypes.c_float(scale), _ptr(status), _stream())
    return out


ATTENTION_DECODE_MAX_SEQS = 1024
ATTENTION_DECODE_MAX_PAIRS = 65536   # sequences x key/value heads


ATTENTION_TMA_PAGE_SIZES = (8, 16, 32, 64, 128)   # a page of the cache is one TMA box


def attention_tc_takes(num_heads: int, num_kv_heads: int, head_dim: int, dtype: torch.dtype) -> bool:
    """Whether the tcgen05 attention kernels (prompt portions and decoding) take these sizes: bfloat16, a
    head size that is a multiple of 8 up to 128 (their tiles are 64 or 128 wide; the TMA boxes fill what
    lies beyond the head size with zeros), at most 16 query heads per key/value head.  The page size must
    be one of ``ATTENTION_TMA_PAGE_SIZES`` besides."""
    return (dtype == torch.bfloat16 and 8 <= head_dim <= 128 and head_dim % 8 == 0 and num_kv_heads > 0 and num_heads % num_kv_heads == 0
            and num_heads // num_kv_heads <= 16)


def attention_decode_takes(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, dtype: torch.dtype) -> bool:
    """Whether the persistent tcgen05 decode-attention kernel takes these sizes: those of
    ``attention_tc_takes`` and pages of 8 .. 128 tokens (a power of two)."""
    return attention_tc_takes(num_heads, num_kv_heads, head_dim, dtype) and page_size in ATTENTION_TMA_PAGE_SIZES


def attention_decode(q: torch.Tensor, num_heads: int, head_dim: int, out: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor,
                     positions: torch.Tensor, q_start: torch.Tensor, num_seqs: int, scale: float, window: Optional[int] = None,
                     status: Optional[torch.Tensor] = None, share: str = "auto") -> torch.Tensor:
    """Attention of a decoding batch (one token per sequence) over its pages: one persistent block
    per SM, keys in the rows of tcgen05 tiles, pages brought in by TMA, the batch's tiles shared out
    evenly over the blocks and merged through scratch memory.  At most 1024 sequences.  ``positions``,
    ``q_start`` and ``block_table`` are read while kernels launched earlier may still be running: they
    must be complete before those start (the engine copies them at the start of a step).  Launches
    on different streams must not overlap (they share the counters of the merge).  ``share``: how
    the work is dealt out, "auto" (the kernel decides), "split" (tiles split evenly, merged) or
    "whole" ((sequence, kv head) pairs whole)."""
    if share not in ("auto", "split", "whole"):
        raise KernelError(f"attention_decode: share {share!r} is not 'auto', 'split' or 'whole'")
    _check(q, "attention queries", torch.bfloat16, 2)
    _check(out, "attention output", torch.bfloat16, 2)
    _check(pages, "cache pages", torch.bfloat16, 5)
    _check(block_table, "block table", torch.int32, 2)
    _check(positions, "positions", torch.int32, 1)
    _check(q_start, "q_start", torch.int32, 1)
    T = q.shape[0]
    num_pages, two, nkv, page_size, hd = pages.shape
    if two != 2 or hd != head_dim:
        raise KernelError(f"cache pages: expected [pages, 2, nkv, page_size, {head_dim}], found {tuple(pages.shape)}")
    if q.shape[1] < num_heads * head_dim or tuple(out.shape) != (T, num_heads * head_dim):
        raise KernelError(f"attention: q {tuple(q.shape)} / out {tuple(out.shape)} do not fit {num_heads} heads of {head_dim}")
    if positions.shape[0] != T or q_start.shape[0] != num_seqs + 1 or block_table.shape[0] < num_seqs or T < num_seqs:
        raise KernelError("attention: positions need one entry per token, q_start one per sequence plus one, the block table a row per sequence")
    lib = build.load("attention_decode")
    lib.spy_attention_decode_scratch_floats.restype = ctypes.c_longlong
    floats = int(lib.spy_attention_decode_scratch_floats(num_seqs, num_heads, nkv, head_dim))
    scratch = attention_scratch(q.device, floats)
    if status is None:
        status = status_word(q.device)
    _call("attention_decode", "spy_attention_decode", _ptr(q), ctypes.c_longlong(q.shape[1]), _ptr(out), _ptr(pages), _ptr(block_table),
          block_table.shape[1], page_size, num_pages, num_heads, nkv, head_dim, _ptr(positions), _ptr(q_start), T, num_seqs,
          int(window or 0), ctypes.c_float(scale), ("auto", "split", "whole").index(share), _ptr(scratch), ctypes.c_longlong(scratch.numel()),
          _ptr(status), _stream())
    return out


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[M, N] = a[M, K] @ w[N, K]^T`` on the CUDA cores in 32-bit, any sizes and dtypes."""
    _check(a, "gemm input", ndim=2)
    _check(w, "gemm weight", ndim=2)
    _check(out, "gemm output", ndim=2)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm: shapes do not fit: input {tuple(a.shape)}, weight {tuple(w.shape)}, output {tuple(out.shape)}")
    _call("gemm_simt", "spy_gemm_simt", _ptr(a), _code(a, "gemm input"), ctypes.c_longlong(K), _ptr(w), _code(w, "gemm weight"),
          ctypes.c_longlong(K), _ptr(out), _code(out, "gemm output"), ctypes.c_longlong(N), M, N, K, _stream())
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]``; gate_up [T, 2I], out [T, I]."""
    _check(gate_up, "swiglu input", ndim=2)
    _check(out, "swiglu output", gate_up.dtype, 2)
    T, two_i = gate_up.shape
    if two_i % 2 != 0 or tuple(out.shape) != (T, two_i // 2):
        raise KernelError(f"swiglu: input {tuple(gate_up.shape)} and output {tuple(out.shape)} do not fit")
    _call("swiglu", "spy_swiglu", _ptr(gate_up), _ptr(out), _code(gate_up, "swiglu input"), T, two_i // 2, _stream())
    return out


def add_bias(out: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """``out[t, c] += bias[c]`` in place (32-bit sum); out [T, C] float32 or bfloat16, bias [C]."""
    _check(out, "bias target", ndim=2)
    _check(bias, "bias", ndim=1)
    if bias.shape[0] != out.shape[1]:
        raise KernelError(f"add_bias: a bias of {bias.shape[0]} does not fit rows of {out.shape[1]}")
    _call("swiglu", "spy_add_bias", _ptr(out), _code(out, "bias target"), _ptr(bias), _code(bias, "bias"), out.shape[0], out.shape[1], _stream())
    return out


def sample(logits: torch.Tensor, tokens: torch.Tensor, temperature: Optional[torch.Tensor] = None, seed: Optional[torch.Tensor] = None,
           draw: Optional[torch.Tensor] = None, top_k: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of ``logits [R, V]`` float32 into ``tokens [R]`` int32: argmax where the
    row's temperature is 0 (or no temperatures are given), else a seeded draw from
    ``softmax(logits / temperature)``, among the row's ``top_k[r]`` largest logits only where
    that is positive (logits equal to the k-th largest all stay)."""
    _check(logits, "logits", torch.float32, 2)
    _check(tokens, "sampled tokens", torch.int32, 1)
    R, V = logits.shape
    if tokens.shape[0] != R:
        raise KernelError("sample: one output token per row of logits is needed")
    if temperature is not None:
        _check(temperature, "temperatures", torch.float32, 1)
        _check(seed, "seeds", torch.int64, 1)
        _check(draw, "draw counters", torch.int64, 1)
        if not (temperature.shape[0] == seed.shape[0] == draw.shape[0] == R):
            raise KernelError("sample: temperature, seed and draw need one entry per row")
    floor_v = None
    if top_k is not None:
        if temperature is None:
            raise KernelError("sample: top_k is for rows with a temperature; give the temperatures too")
        _check(top_k, "top_k", torch.int32, 1)
        if top_k.shape[0] != R:
            raise KernelError("sample: top_k needs one entry per row")
        floor_v = torch.empty(R, dtype=torch.float32, device=logits.device)
    lib = build.load("sampling")
    slices = lib.spy_sample_slices(V)
    slice_v = torch.empty(R * slices, dtype=torch.float32, device=logits.device)
    slice_i = torch.empty(R * slices, dtype=torch.int32, device=logits.device)
    _call("sampling", "spy_sample", _ptr(logits), ctypes.c_longlong(V), R, V, _ptr(temperature), _ptr(seed), _ptr(draw), _ptr(top_k),
          _ptr(floor_v), _ptr(tokens), _ptr(slice_v), _ptr(slice_i), _stream())
    return tokens


def tensor_core_gemm_takes(out_features: int, in_features: int) -> bool:
    """Whether the tcgen05 kernel takes a weight of this shape: its rows must be 16 bytes
    aligned for TMA, so ``in_features`` must be a multiple of 8.  Any ``out_features``."""
    return in_features % 8 == 0 and in_features > 0


_status_words = {}


def status_word(device) -> torch.Tensor:
    """The device's status word: two int32 (code, detail), zero while all is well.  Kernels
    that meet an index outside their buffers, or whose bounded waits run out, store a code
    here and skip the access; the engine reads it after a step."""
    key = str(torch.device(device))
    if key not in _status_words:
        _status_words[key] = torch.zeros(2, dtype=torch.int32, device=device)
    return _status_words[key]


GEMM_SCRATCH_FLOATS = 16 * 1024 * 1024
_gemm_scratch = {}


def _scratch(device) -> torch.Tensor:
    """The split-K scratch of a device: one fixed buffer (64 MB), made at first use, so that
    captured graphs keep pointing at live memory.  Products on one stream use it in turn."""
    key = str(device)
    if key not in _gemm_scratch:
        _gemm_scratch[key] = torch.empty(GEMM_SCRATCH_FLOATS, dtype=torch.float32, device=device)
    return _gemm_scratch[key]


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None,
                 out_dtype: Optional[torch.dtype] = None, epilogue: Optional[str] = None, defer: bool = False,
                 prefetch: Optional[torch.Tensor] = None, prefetch_bytes: int = 0) -> torch.Tensor:
    """``a[M, K] @ w[N, K]^T`` on the tensor cores: bfloat16 operands, 32-bit accumulation,
    bfloat16 or float32 output.  K must be a multiple of 8.

    ``epilogue="swiglu"``: ``w``'s rows alternate gate and up rows and the result is
    ``silu(gate) * up``, ``[M, N / 2]``.  ``defer=True``: when the kernel splits K, the float32
    partial products are returned unsummed as ``[splits, M, N]`` for a consumer that adds them
    (``rmsnorm``'s delta, ``qk_rope_store``'s input); otherwise the result is ``[M, N]``.
    ``prefetch``: a tensor that a later kernel will read (the next product's weights); with up to 256
    rows in ``a`` the blocks ask for its first ``prefetch_bytes`` bytes (0: all) to be brought into L2
    once their own loads are on their way."""
    _check(a, "gemm input", torch.bfloat16, 2)
    _check(w, "gemm weight", torch.bfloat16, 2)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm: shapes do not fit: input {tuple(a.shape)}, weight {tuple(w.shape)}")
    if epilogue not in (None, "swiglu"):
        raise KernelError(f"gemm: unknown epilogue {epilogue!r}")
    n_out = N // 2 if epilogue == "swiglu" else N
    if status is None:
        status = status_word(a.device)
    lib = build.load("gemm_tcgen05")
    pf_ptr, pf_bytes = None, 0
    if prefetch is not None and M <= 256:
        total = prefetch.numel() * prefetch.element_size()
        pf_ptr, pf_bytes = _ptr(prefetch), min(total, prefetch_bytes) if prefetch_bytes > 0 else total
    if defer and epilogue is None and out is None:
        splits, need = ctypes.c_int(1), ctypes.c_longlong(0)
        lib.spy_gemm_tcgen05_plan(M, N, K, ctypes.c_longlong(1 << 40), ctypes.byref(splits), ctypes.byref(need))
        if splits.value > 1:
            stack = torch.empty((splits.value, M, N), dtype=torch.float32, device=a.device)
            used = ctypes.c_int(0)
            _call("gemm_tcgen05", "spy_gemm_tcgen05_ex", _ptr(a), ctypes.c_longlong(K), _ptr(w), ctypes.c_longlong(K), None, BF16,
                  ctypes.c_longlong(N), M, N, K, _ptr(stack), ctypes.c_longlong(stack.numel()), 0, 1, ctypes.byref(used), _ptr(status),
                  _stream(), pf_ptr, ctypes.c_longlong(pf_bytes))
            if used.value != splits.value:
                raise KernelError(f"gemm: planned {splits.value} splits, the kernel used {used.value}")
            return stack
    if out is None:
        out = torch.empty((M, n_out), dtype=out_dtype or torch.bfloat16, device=a.device)
    else:
        _check(out, "gemm output", ndim=2)
        if tuple(out.shape) != (M, n_out):
            raise KernelError(f"gemm: output {tuple(out.shape)} does not fit [{M}, {n_out}]")
    scratch = _scratch(a.device)
    _call("gemm_tcgen05", "spy_gemm_tcgen05_ex", _ptr(a), ctypes.c_longlong(K), _ptr(w), ctypes.c_longlong(K), _ptr(out),
          _code(out, "gemm output"), ctypes.c_longlong(n_out), M, N, K, _ptr(scratch), ctypes.c_longlong(scratch.numel()),
          1 if epilogue == "swiglu" else 0, 0, None, _ptr(status), _stream(), pf_ptr, ctypes.c_longlong(pf_bytes))
    return out


def gemm_tcgen05_reset() -> None:
    """Lowers the flags that the blocks of a product with shared K blocks signal one another by.
    To be called after a status word of 4 (a wait ran out): the product that gave up may have left
    flags raised, which the next such product would take for partial tiles that are ready."""
    _call("gemm_tcgen05", "spy_gemm_tcgen05_reset", _stream())


def wait_selftest(limit_ns: int, status: Optional[torch.Tensor] = None) -> int:
    """Runs the kernels' bounded wait on a barrier that nothing arrives at, with ``limit_ns`` as its
    limit (at most 100 ms).  The kernel returns by itself and leaves code 4 in the status word; the
    nanoseconds its first thread waited are returned.  A health check of the mechanism that keeps a
    lost signal inside a tensor-core kernel from holding the GPU."""
    dev = torch.device("cuda", torch.cuda.current_device()) if status is None else status.device
    if status is None:
        status = status_word(dev)
    waited = torch.zeros(1, dtype=torch.int64, device=dev)
    _call("gemm_tcgen05", "spy_tcgen05_wait_selftest", ctypes.c_ulonglong(int(limit_ns)), _ptr(status), _ptr(waited), _stream())
    return int(waited.item())

