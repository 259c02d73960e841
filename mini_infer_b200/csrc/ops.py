"""Python faces of the CUDA kernels.

Each function checks its tensors (device, dtype, layout), passes raw pointers and the
current CUDA stream to an ``extern "C"`` entry point, and raises ``KernelError`` with the
library's message if the arguments were refused or the launch failed.  There is no CPU
path: a tensor that is not on a CUDA device is an error.

``launch_count`` counts the kernels launched through this module (the bench reports it).
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_void_p

import torch

from . import build

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}

launch_count = 0


class KernelError(RuntimeError):
    pass


def _ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _cuda(*tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels run on CUDA tensors only (got a tensor on %s)" % t.device)


def _code(dtype: torch.dtype) -> int:
    try:
        return DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"unsupported dtype {dtype}; kernels take float32 or bfloat16") from None


def _finish(lib: ctypes.CDLL, rc: int, what: str) -> None:
    global launch_count
    if rc != 0:
        msg = lib.mi_error_message().decode("utf-8", "replace")
        raise KernelError(f"{what}: {msg or ('status %d' % rc)}")
    launch_count += 1


class KernelWaitError(KernelError):
    """A kernel gave up one of its bounded waits: what it wrote since is not to be trusted."""


_configured: set[str] = set()

# Libraries whose kernels have bounded waits.  Their give-ups are reported into one int32 word
# per device (``status_word``), which the engine copies to the host with every step's result;
# on their own the libraries would each keep a word that only a synchronising call can read.
_WAITING_LIBRARIES = ("attention_mma", "attention_tc", "gemm_tma")
_status_words: dict[int, torch.Tensor] = {}
_status_shared: set[tuple[str, int]] = set()


def _lib(name: str) -> ctypes.CDLL:
    lib = build.library(name)
    if name not in _configured:
        _SIGNATURES[name](lib)
        _configured.add(name)
    return lib


def _device_index(device: torch.device) -> int:
    return device.index if device.index is not None else torch.cuda.current_device()


def status_word(device: torch.device) -> torch.Tensor:
    """The int32 word (on ``device``) that the kernels with bounded waits set to 1 when a wait
    gave up.  Zero means every such kernel launched through this module has waited out its
    copies; the engine reads it with each step's tokens."""
    idx = _device_index(device)
    word = _status_words.get(idx)
    if word is None:
        word = _status_words[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return word


def _waiting_lib(name: str, device: torch.device) -> ctypes.CDLL:
    """``_lib`` for a library with bounded waits: the first use on a device points the
    library's give-up reports at that device's shared status word."""
    lib = _lib(name)
    idx = _device_index(device)
    if (name, idx) not in _status_shared:
        with torch.cuda.device(idx):
            rc = lib.mi_set_status_word(_ptr(status_word(device)))
        if rc != 0:
            raise KernelError(f"{name}: cannot share the status word: {lib.mi_error_message().decode()}")
        _status_shared.add((name, idx))
    return lib


def recover_from_wait_failure(device: torch.device) -> None:
    """After a give-up: clear the status word and the arrival counters that the interrupted
    kernels may have left non-zero (they are zero between calls otherwise).  Synchronises."""
    torch.cuda.synchronize(device)
    with torch.inference_mode():      # the buffers were made inside a step, which runs in inference mode
        status_word(device).zero_()
        idx = _device_index(device)
        for buf in _decode_counter_bufs.get(idx, []):
            buf.zero_()
        for _partials, counters in _tma_ws.get(idx, []):
            counters.zero_()
    torch.cuda.synchronize(device)


def _sig_elementwise(lib: ctypes.CDLL) -> None:
    lib.mi_embedding.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
    lib.mi_add_rmsnorm.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_int, c_int, c_float, c_int, c_int, c_void_p]
    lib.mi_rope_write.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
    lib.mi_silu_mul.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    lib.mi_silu_mul_pairs.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    lib.mi_table_update.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p]
    lib.mi_rope_table.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]


def _sig_gemm_f32(lib: ctypes.CDLL) -> None:
    lib.mi_gemm_f32.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                c_int, c_void_p]


def _sig_attention_generic(lib: ctypes.CDLL) -> None:
    lib.mi_attention_generic.argtypes = [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
        c_float, c_int, c_int, c_void_p]
    lib.mi_attention_generic_tile_tokens.restype = c_int


def _sig_sampling(lib: ctypes.CDLL) -> None:
    lib.mi_sample.argtypes = [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                              c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]


def _sig_attention_mma(lib: ctypes.CDLL) -> None:
    lib.mi_attention_decode.argtypes = [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
        c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p,
        c_void_p, c_void_p]
    lib.mi_attention_decode_sliced.argtypes = [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
        c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p,
        c_void_p, c_void_p]
    lib.mi_attention_decode_counters.argtypes = [c_int, c_int, c_int]
    lib.mi_attention_decode_balanced_scratch.argtypes = [c_int, c_int, c_int, c_int, c_int, ctypes.POINTER(c_int),
                                                         ctypes.POINTER(ctypes.c_longlong),
                                                         ctypes.POINTER(ctypes.c_longlong), ctypes.POINTER(c_int)]
    lib.mi_attention_decode_balanced.argtypes = [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
        c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]
    lib.mi_attention_decode_balanced_unit_cost.argtypes = [c_int]
    lib.mi_attention_wait_status.argtypes = [c_int]
    lib.mi_set_status_word.argtypes = [c_void_p]
    lib.mi_attention_prefill.argtypes = [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
        c_float, c_int, c_void_p]
    lib.mi_attention_prefill_tile_tokens.argtypes = [c_int]
    lib.mi_attention_prefill_tile_tokens.restype = c_int


def _sig_gemm_tma(lib: ctypes.CDLL) -> None:
    lib.mi_gemm_tma.argtypes = [c_void_p, ctypes.c_longlong, c_void_p, c_void_p, ctypes.c_longlong, c_int, c_int,
                                c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]
    lib.mi_gemm_tma_fused.argtypes = [c_void_p, ctypes.c_longlong, c_void_p, c_void_p, ctypes.c_longlong, c_int, c_int,
                                      c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
                                      c_void_p, c_void_p, c_void_p, c_void_p]
    lib.mi_gemm_tma_workspace.argtypes = [c_int, c_int, c_int, ctypes.POINTER(ctypes.c_longlong),
                                          ctypes.POINTER(c_int)]
    lib.mi_gemm_tma_status.argtypes = [c_int]
    lib.mi_set_status_word.argtypes = [c_void_p]


def _sig_attention_tc(lib: ctypes.CDLL) -> None:
    lib.mi_attention_prefill_tc.argtypes = [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_int, c_void_p, c_int,
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
        c_void_p]
    lib.mi_attention_prefill_tc_supported.argtypes = [c_int, c_int, c_int, c_int]
    lib.mi_attention_tc_status.argtypes = [c_int]
    lib.mi_set_status_word.argtypes = [c_void_p]


_SIGNATURES = {
    "attention_tc": _sig_attention_tc,
    "gemm_tma": _sig_gemm_tma,
    "attention_mma": _sig_attention_mma,
    "elementwise": _sig_elementwise,
    "gemm_f32": _sig_gemm_f32,
    "attention_generic": _sig_attention_generic,
    "sampling": _sig_sampling,
}


def register_signatures(name: str, fn) -> None:
    _SIGNATURES[name] = fn


# ---------------------------------------------------------------------------------------


def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out[t] = table[ids[t]]``; ``ids`` int32 ``[M]``, ``table`` ``[V, H]``."""
    _cuda(table, ids, out)
    if ids.dtype != torch.int32 or ids.dim() != 1 or not ids.is_contiguous():
        raise KernelError("embedding: ids must be a contiguous int32 vector")
    if table.dim() != 2 or not table.is_contiguous():
        raise KernelError("embedding: table must be a contiguous [V, H] matrix")
    V, H = table.shape
    M = ids.shape[0]
    if out is None:
        out = torch.empty((M, H), dtype=table.dtype, device=table.device)
    elif out.shape != (M, H) or out.dtype != table.dtype or not out.is_contiguous():
        raise KernelError("embedding: bad output tensor")
    lib = _lib("elementwise")
    rc = lib.mi_embedding(_ptr(table), _ptr(ids), _ptr(out), M, H, V, _code(table.dtype), _stream())
    _finish(lib, rc, "embedding")
    return out


def add_rmsnorm(
    x: torch.Tensor,
    weight: torch.Tensor,
    eps: float,
    *,
    residual_in: torch.Tensor | None = None,
    residual_out: torch.Tensor | None = None,
    rows: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """RMS norm of ``x (+ residual_in)`` with fp32 statistics.

    ``r = float(x[src]) + residual_in[src]`` (``src = rows[i]`` if ``rows`` is given, else
    ``i``); ``residual_out[i] = r`` if given (fp32; may alias ``residual_in`` when no
    ``rows``); returns ``weight * r * rsqrt(mean(r*r) + eps)`` in ``x``'s dtype.
    """
    _cuda(x, weight, residual_in, residual_out, rows, out)
    if x.dim() != 2 or not x.is_contiguous():
        raise KernelError("rmsnorm: x must be a contiguous [M, H] matrix")
    H = x.shape[1]
    M = x.shape[0] if rows is None else rows.shape[0]
    if weight.shape != (H,) or not weight.is_contiguous():
        raise KernelError(f"rmsnorm: weight must have shape ({H},)")
    for name, r in (("residual_in", residual_in), ("residual_out", residual_out)):
        if r is not None and (r.dtype != torch.float32 or r.dim() != 2 or r.shape[1] != H
                              or not r.is_contiguous()):
            raise KernelError(f"rmsnorm: {name} must be a contiguous fp32 [*, {H}] matrix")
    if residual_in is not None and residual_in.shape[0] != x.shape[0]:
        raise KernelError("rmsnorm: residual_in must have x's rows")
    if residual_out is not None and residual_out.shape[0] != M:
        raise KernelError("rmsnorm: residual_out must have one row per output row")
    if rows is not None and (rows.dtype != torch.int32 or rows.dim() != 1 or not rows.is_contiguous()):
        raise KernelError("rmsnorm: rows must be a contiguous int32 vector")
    if out is None:
        out = torch.empty((M, H), dtype=x.dtype, device=x.device)
    elif out.shape != (M, H) or out.dtype != x.dtype or not out.is_contiguous():
        raise KernelError("rmsnorm: bad output tensor")
    lib = _lib("elementwise")
    rc = lib.mi_add_rmsnorm(_ptr(x), _ptr(residual_in), _ptr(residual_out), _ptr(weight), _ptr(out),
                            _ptr(rows), M, H, float(eps), _code(x.dtype), _code(weight.dtype), _stream())
    _finish(lib, rc, "rmsnorm")
    return out


def rope_write(
    qkv: torch.Tensor,
    nq: int,
    nkv: int,
    head_dim: int,
    *,
    positions: torch.Tensor | None = None,
    inv_freq: torch.Tensor | None = None,
    rotary_dim: int = 0,
    slots: torch.Tensor | None = None,
    kcache: torch.Tensor | None = None,
    vcache: torch.Tensor | None = None,
) -> None:
    """Rotate q and k inside ``qkv [M, (nq + 2 nkv) * d]`` (half layout, fp32 angles) and
    store k and v at ``slots`` (page * page_size + offset) of ``kcache`` / ``vcache``
    ``[pages, nkv, page_size, d]``."""
    _cuda(qkv, positions, inv_freq, slots, kcache, vcache)
    M = qkv.shape[0]
    if qkv.dim() != 2 or qkv.shape[1] != (nq + 2 * nkv) * head_dim or not qkv.is_contiguous():
        raise KernelError("rope: qkv must be contiguous [M, (nq + 2 nkv) * d]")
    if rotary_dim:
        if positions is None or positions.dtype != torch.int32 or positions.shape != (M,):
            raise KernelError("rope: positions must be int32 [M]")
        if inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.shape != (rotary_dim // 2,):
            raise KernelError("rope: inv_freq must be fp32 [rotary_dim / 2]")
    if kcache is not None:
        if slots is None or slots.dtype != torch.int32 or slots.shape != (M,):
            raise KernelError("rope: slots must be int32 [M]")
        for c in (kcache, vcache):
            if (c is None or c.dtype != qkv.dtype or c.dim() != 4 or c.shape[1] != nkv or c.shape[3] != head_dim
                    or not c.is_contiguous()):
                raise KernelError("rope: caches must be contiguous [pages, nkv, page_size, d] in qkv's dtype")
    page_size = int(kcache.shape[2]) if kcache is not None else 0
    lib = _lib("elementwise")
    rc = lib.mi_rope_write(_ptr(qkv), _ptr(positions), _ptr(inv_freq), _ptr(slots), _ptr(kcache),
                           _ptr(vcache), M, nq, nkv, head_dim, rotary_dim, page_size, _code(qkv.dtype),
                           _stream())
    _finish(lib, rc, "rope")


def table_update(table: torch.Tensor, updates: torch.Tensor, count: torch.Tensor, capacity: int) -> None:
    """Scatter new page ids into a block table: ``table[slot, index] = page`` for the first
    ``count[0]`` (at most ``capacity``) triples ``(slot, index, page)`` of ``updates``; all int32
    on the device.  ``count`` is read when the kernel runs, so a captured step can replay it."""
    _cuda(table, updates, count)
    if table.dtype != torch.int32 or table.dim() != 2 or not table.is_contiguous():
        raise KernelError("table_update: the table must be a contiguous int32 matrix")
    if updates.dtype != torch.int32 or updates.numel() < 3 * capacity or count.dtype != torch.int32 or count.numel() < 1:
        raise KernelError("table_update: updates must hold 3 * capacity int32 values and count one")
    lib = _lib("elementwise")
    rc = lib.mi_table_update(_ptr(table), table.shape[1], table.shape[0], _ptr(updates), _ptr(count),
                             int(capacity), _stream())
    _finish(lib, rc, "table_update")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor | None = None, pairs: bool = False) -> torch.Tensor:
    """``silu(gate) * up`` with fp32 arithmetic, for ``gate_up [M, 2 I]`` laid out as halves
    (``gate = gate_up[:, :I]``, ``up = gate_up[:, I:]``) or, with ``pairs``, interleaved
    (``gate = gate_up[:, 0::2]``, ``up = gate_up[:, 1::2]``)."""
    _cuda(gate_up, out)
    if gate_up.dim() != 2 or gate_up.shape[1] % 2 or not gate_up.is_contiguous():
        raise KernelError("silu_mul: input must be contiguous [M, 2 I]")
    M, I2 = gate_up.shape
    I = I2 // 2
    if out is None:
        out = torch.empty((M, I), dtype=gate_up.dtype, device=gate_up.device)
    elif out.shape != (M, I) or out.dtype != gate_up.dtype or not out.is_contiguous():
        raise KernelError("silu_mul: bad output tensor")
    lib = _lib("elementwise")
    fn = lib.mi_silu_mul_pairs if pairs else lib.mi_silu_mul
    rc = fn(_ptr(gate_up), _ptr(out), M, I, _code(gate_up.dtype), _stream())
    _finish(lib, rc, "silu_mul")
    return out


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``a [M, K] @ w [N, K]^T`` in true fp32 (CUDA cores, fixed summation order)."""
    _cuda(a, w, out)
    if a.dtype != torch.float32 or w.dtype != torch.float32:
        raise KernelError("gemm_f32: operands must be float32")
    if a.dim() != 2 or w.dim() != 2 or a.shape[1] != w.shape[1]:
        raise KernelError(f"gemm_f32: shapes {tuple(a.shape)} x {tuple(w.shape)}^T do not match")
    if a.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError("gemm_f32: operands must be K-contiguous")
    M, K = a.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    elif out.shape != (M, N) or out.dtype != torch.float32 or out.stride(1) != 1:
        raise KernelError("gemm_f32: bad output tensor")
    lib = _lib("gemm_f32")
    rc = lib.mi_gemm_f32(_ptr(a), _ptr(w), _ptr(out), M, N, K, a.stride(0) if M > 1 else K,
                         w.stride(0) if N > 1 else K, out.stride(0) if M > 1 else N, _stream())
    _finish(lib, rc, "gemm_f32")
    return out


def cache_swizzle_mask(head_dim: int, dtype: torch.dtype) -> int:
    """The chunk permutation mask of cache rows (``mi_swizzle_mask`` in common.cuh)."""
    n = head_dim * torch.empty((), dtype=dtype).element_size() // 16
    if n < 2 or n & (n - 1):
        return 0
    return min(n, 8) - 1


def _chunk_permutation(page_size: int, head_dim: int, dtype: torch.dtype) -> torch.Tensor:
    """``perm[t, k]``: where element ``k`` of the row at in-page offset ``t`` is stored."""
    epc = 16 // torch.empty((), dtype=dtype).element_size()
    mask = cache_swizzle_mask(head_dim, dtype)
    t = torch.arange(page_size).view(-1, 1)
    k = torch.arange(head_dim).view(1, -1)
    return ((k // epc) ^ (t & mask)) * epc + k % epc


def pack_cache_pages(by_slot: torch.Tensor, page_size: int) -> torch.Tensor:
    """``[pages * page_size, kv_heads, d]`` (one row per slot) -> the cache layout
    ``[pages, kv_heads, page_size, d]`` with each row's 16-byte chunks permuted by its in-page
    offset.  For tests and tools; the engine writes the cache with the rope/store kernel."""
    n, nkv, d = by_slot.shape
    pages = by_slot.view(n // page_size, page_size, nkv, d).permute(0, 2, 1, 3).contiguous()
    perm = _chunk_permutation(page_size, d, by_slot.dtype).to(by_slot.device)
    out = torch.empty_like(pages)
    out.scatter_(3, perm.view(1, 1, page_size, d).expand_as(pages), pages)
    return out


def unpack_cache_pages(pages: torch.Tensor) -> torch.Tensor:
    """The inverse of ``pack_cache_pages``: ``[pages * page_size, kv_heads, d]`` by slot."""
    n_pages, nkv, page_size, d = pages.shape
    perm = _chunk_permutation(page_size, d, pages.dtype).to(pages.device)
    plain = torch.gather(pages, 3, perm.view(1, 1, page_size, d).expand_as(pages))
    return plain.permute(0, 2, 1, 3).reshape(n_pages * page_size, nkv, d)


# Query tokens per tile of the CUDA-core attention kernel (BQ in attention_generic.cu).
ATTENTION_TILE_TOKENS = 16


def prefill_tile_tokens(group: int) -> int:
    """Tokens per tile of the tensor-core prefill kernel for ``group`` query heads per
    key/value head: 128 rows of (token, head in group) per block (attention_mma.cu)."""
    return 128 // min(group, 128)


PREFILL_TC_TILES = 1      # 128-row tiles per block of the tcgen05 prefill kernel (NTILE in attention_tc.cu)


def prefill_tc_tile_tokens(group: int) -> int:
    """Tokens per block of the tcgen05 prefill kernel: tiles of 128 rows of (token, head in
    group) (attention_tc.cu)."""
    return 128 * PREFILL_TC_TILES // min(group, 128)


def attention_tile_sizes(group: int) -> frozenset[int]:
    """The query tile sizes a step must plan for an attention mixer with this group size."""
    return frozenset({ATTENTION_TILE_TOKENS, prefill_tile_tokens(group), prefill_tc_tile_tokens(group)})


_sm_count: dict[int, int] = {}


def _sms(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _sm_count:
        _sm_count[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _sm_count[idx]


def sm_count(device: torch.device) -> int:
    return _sms(device)


def decode_splits(n_requests: int, nq: int, nkv: int, max_kv_len: int, window: int, device) -> int:
    """For the sliced decode kernel (``attention_decode``), which the engine itself no longer
    uses: how many slices of the keys each (request, key/value head) is cut into: enough blocks
    for about two per SM, but at least four 64-key chunks per slice (a slice costs a fixed
    prologue and a merge, measured at roughly ten chunks' worth of time)."""
    blocks = n_requests * nkv * ((nq // nkv + 7) // 8)
    span = min(max_kv_len, window + 63) if window else max_kv_len
    chunks = max(1, -(-span // 64))
    return max(1, min(2 * _sms(device) // blocks, chunks // 4, 64))


FUSE_DECODE_ROPE = os.environ.get("MINI_INFER_FUSE_ROPE", "1") != "0"
SPLIT_MIXED_STEPS = os.environ.get("MINI_INFER_SPLIT_MIXED", "1") != "0"


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """``[tokens, 2 * len(inv_freq)]`` fp32: per token the sines, then the cosines, of
    ``position * inv_freq``, computed as the rotary kernels compute them (elementwise.cu)."""
    _cuda(positions, inv_freq)
    if positions.dtype != torch.int32 or inv_freq.dtype != torch.float32:
        raise KernelError("rope_table: int32 positions and fp32 frequencies")
    half = inv_freq.numel()
    out = torch.empty((positions.numel(), 2 * half), dtype=torch.float32, device=positions.device)
    lib = _lib("elementwise")
    rc = lib.mi_rope_table(_ptr(positions), _ptr(inv_freq), _ptr(out), positions.numel(), half, _stream())
    _finish(lib, rc, "rope_table")
    return out


FUSE_DECODE_ROPE_MAX_REQUESTS = 16


def decode_rope_fusable(q_dtype: torch.dtype, head_dim: int, decode_only: bool, n_requests: int) -> bool:
    """Whether ``attention`` should rotate q and store the new key and value itself (the decode
    kernel of bfloat16 steps in which every request brings one token).  Measured inside the
    captured step at Llama 3.1 8B sizes: one kernel boundary less per layer is worth 0.5 % at
    batch 8; at batch 64 the separate kernel is 1 % faster (while it runs, the attention kernel's
    copy warps are already fetching pages), hence the limit."""
    return (FUSE_DECODE_ROPE and decode_only and q_dtype == torch.bfloat16 and head_dim in (64, 128, 256)
            and n_requests <= FUSE_DECODE_ROPE_MAX_REQUESTS)


def attention(q: torch.Tensor, q_stride: int, out: torch.Tensor, cache, ctx, nq: int, nkv: int,
              head_dim: int, scale: float, window: int = 0, rope_table: torch.Tensor | None = None) -> None:
    """Attention of this step's queries over one cache layer.

    ``cache`` is a ``LayerCache`` (its ``k``/``v`` pages and group index), ``ctx`` the
    ``StepContext`` (block tables, lengths, query tiles).  float32 runs the CUDA-core kernel;
    bfloat16 runs the tensor-core kernels: the balanced decode kernel when every request brings
    one token, otherwise the tcgen05 prefill kernel where it takes the sizes and the mma.sync
    prefill kernel elsewhere.  ``rope_table`` (only where ``decode_rope_fusable``): q, k, v are
    un-rotated and not yet stored; the decode kernel does both.
    """
    group = ctx.groups[cache.group]
    if q.dtype == torch.bfloat16:
        if ctx.decode_only:
            attention_decode_balanced(q, q_stride, out, cache.k, cache.v, group.block_table, group.page_size,
                                      ctx.q_start, ctx.kv_len, ctx.n_requests, nq, nkv, head_dim, scale, window,
                                      table_rows=group.table_rows, rope_table=rope_table,
                                      store_kv=bool(cache.writes))
        else:
            if rope_table is not None:
                raise KernelError("attention: only the decode kernel rotates and stores by itself")
            tc = USE_TC_PREFILL and prefill_tc_supported(nq, nkv, head_dim, group.page_size)
            tt = (prefill_tc_tile_tokens if tc else prefill_tile_tokens)(nq // nkv)
            tile_req, tile_tok0, n_tiles = ctx.q_tiles(tt)
            if SPLIT_MIXED_STEPS and ctx.n_single and tt in ctx.tiles_multi:
                # a mixed step: the single tokens through the decode kernel (their keys spread over
                # all blocks), the prompt portions through the prefill kernel; disjoint rows of `out`
                attention_decode_balanced(q, q_stride, out, cache.k, cache.v, group.block_table, group.page_size,
                                          ctx.single_q_start, ctx.single_kv_len, ctx.n_single, nq, nkv, head_dim,
                                          scale, window, table_rows=ctx.single_rows)
                tile_req, tile_tok0, n_tiles = ctx.tiles_multi[tt]
            (attention_prefill_tc if tc else attention_prefill)(
                q, q_stride, out, cache.k, cache.v, group.block_table, group.page_size,
                ctx.q_start, ctx.q_len, ctx.kv_len, tile_req, tile_tok0, n_tiles, tt,
                nq, nkv, head_dim, scale, window, table_rows=group.table_rows)
        return
    tile_req, tile_tok0, n_tiles = ctx.q_tiles(ATTENTION_TILE_TOKENS)
    attention_generic(q, q_stride, out, cache.k, cache.v, group.block_table, group.page_size,
                      ctx.q_start, ctx.q_len, ctx.kv_len, tile_req, tile_tok0, n_tiles,
                      nq, nkv, head_dim, scale, window, table_rows=group.table_rows)


def _check_attention_args(q, out, kcache, vcache, block_table, nq, nkv, head_dim, page_size, ints):
    for name, t in ints:
        if t is not None and t.dtype != torch.int32:
            raise KernelError(f"attention: {name} must be int32")
    if kcache.dtype != q.dtype or vcache.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelError("attention: q, out and caches must share a dtype")
    if kcache.dim() != 4 or kcache.shape[1:] != (nkv, page_size, head_dim) or not kcache.is_contiguous() \
            or vcache.shape != kcache.shape or not vcache.is_contiguous():
        raise KernelError("attention: caches must be contiguous [pages, nkv, page_size, d]")
    if out.dim() != 2 or out.shape[1] != nq * head_dim or not out.is_contiguous():
        raise KernelError("attention: out must be contiguous [tokens, nq * d]")
    if block_table.dim() != 2 or block_table.stride(1) != 1:
        raise KernelError("attention: block_table must be [rows, pages] with unit inner stride")


# Arrival counters of the split-key decode kernel, per device: zero between calls (the kernel
# resets them).  Never freed once handed out: a captured CUDA graph may hold the address.
_decode_counter_bufs: dict[int, list[torch.Tensor]] = {}


def _decode_counters(device: torch.device, n: int) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    stack = _decode_counter_bufs.setdefault(idx, [])
    if not stack or stack[-1].numel() < n:
        stack.append(torch.zeros(max(n, 16384), dtype=torch.int32, device=device))
    return stack[-1]


def attention_decode(q, q_stride, out, kcache, vcache, block_table, page_size, q_start, kv_len,
                     n_requests, nq, nkv, head_dim, scale, window=0, n_splits=1, slice_chunks=None,
                     table_rows=None) -> None:
    """bfloat16 decode attention: one query token per request, keys cut into ``n_splits``
    slices whose partial results are merged through scratch memory (attention_mma.cu).
    Request ``b`` reads row ``table_rows[b]`` of ``block_table`` (row ``b`` without ``table_rows``).
    ``slice_chunks`` (an int32 tensor of one element on the device, read when the kernel
    runs) makes every slice that many 64-key chunks for all requests; without it every
    request's own keys are cut into ``n_splits`` equal slices."""
    _cuda(q, out, kcache, vcache, block_table, q_start, kv_len, slice_chunks, table_rows)
    if slice_chunks is not None and (slice_chunks.dtype != torch.int32 or slice_chunks.numel() < 1):
        raise KernelError("attention_decode: slice_chunks must be an int32 tensor of one element")
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_decode: bfloat16 only")
    _check_attention_args(q, out, kcache, vcache, block_table, nq, nkv, head_dim, page_size,
                          (("block_table", block_table), ("q_start", q_start), ("kv_len", kv_len),
                           ("table_rows", table_rows)))
    part_o = part_ml = counters = None
    lib = _waiting_lib("attention_mma", q.device)
    if n_splits > 1:
        part_o = torch.empty((n_requests * nq * n_splits, head_dim), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n_requests * nq * n_splits, 2), dtype=torch.float32, device=q.device)
        counters = _decode_counters(q.device, lib.mi_attention_decode_counters(int(n_requests), nq, nkv))
    rc = lib.mi_attention_decode_sliced(
        _ptr(q), int(q_stride), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache), _ptr(block_table),
        block_table.stride(0), _ptr(table_rows), int(page_size), _ptr(q_start), _ptr(kv_len), int(n_requests), nq, nkv,
        head_dim, float(scale), int(window), int(n_splits), _ptr(slice_chunks), _ptr(part_o), _ptr(part_ml),
        _ptr(counters), _stream())
    _finish(lib, rc, "attention_decode")


# Scratch of the balanced decode kernel, per device: partial results, their (max, sum) pairs and
# the per-unit chunk counters (zero between calls).  Never freed once handed out: a captured
# CUDA graph may hold the addresses.
_balanced_ws: dict[int, list[tuple[torch.Tensor, torch.Tensor, torch.Tensor]]] = {}


def _balanced_workspace(device: torch.device, o_floats: int, ml_floats: int, counters: int):
    idx = _device_index(device)
    stack = _balanced_ws.setdefault(idx, [])
    if not stack or stack[-1][0].numel() < o_floats or stack[-1][1].numel() < ml_floats or stack[-1][2].numel() < counters:
        stack.append((torch.empty(max(o_floats, 1 << 20), dtype=torch.float32, device=device),
                      torch.empty(max(ml_floats, 1 << 14), dtype=torch.float32, device=device),
                      torch.zeros(max(counters, 4096), dtype=torch.int32, device=device)))
    return stack[-1]


def attention_decode_balanced(q, q_stride, out, kcache, vcache, block_table, page_size, q_start, kv_len,
                              n_requests, nq, nkv, head_dim, scale, window=0, table_rows=None,
                              rope_table: torch.Tensor | None = None, store_kv: bool = True) -> None:
    """bfloat16 decode attention with the keys of all requests spread evenly over persistent
    blocks, whatever the requests' lengths (attention_decode_balanced_kernel): no plan from the
    host, the blocks read the lengths themselves.  With ``rope_table`` (``rope_table()`` of the
    step's positions) q, k and v come as the projection left them (one row per token: q heads, k
    heads, v heads): the kernel rotates q itself and, with ``store_kv``, rotates the new key and
    writes it and the new value into their page before it reads them."""
    _cuda(q, out, kcache, vcache, block_table, q_start, kv_len, table_rows, rope_table)
    if rope_table is not None and (rope_table.dtype != torch.float32 or not rope_table.is_contiguous()
                                   or rope_table.shape[-1] != head_dim):
        raise KernelError("attention_decode: the rotary table must be contiguous fp32 [tokens, head_dim]")
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_decode: bfloat16 only")
    _check_attention_args(q, out, kcache, vcache, block_table, nq, nkv, head_dim, page_size,
                          (("block_table", block_table), ("q_start", q_start), ("kv_len", kv_len),
                           ("table_rows", table_rows)))
    lib = _waiting_lib("attention_mma", q.device)
    grid, o_floats, ml_floats, counters = c_int(0), ctypes.c_longlong(0), ctypes.c_longlong(0), c_int(0)
    rc = lib.mi_attention_decode_balanced_scratch(int(n_requests), nq, nkv, head_dim, _sms(q.device), ctypes.byref(grid),
                                                  ctypes.byref(o_floats), ctypes.byref(ml_floats), ctypes.byref(counters))
    if rc != 0:
        raise KernelError("attention_decode: " + lib.mi_error_message().decode("utf-8", "replace"))
    part_o, part_ml, count = _balanced_workspace(q.device, int(o_floats.value), int(ml_floats.value), int(counters.value))
    rc = lib.mi_attention_decode_balanced(
        _ptr(q), int(q_stride), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache), _ptr(block_table),
        block_table.stride(0), _ptr(table_rows), int(page_size), _ptr(q_start), _ptr(kv_len), int(n_requests), nq, nkv,
        head_dim, float(scale), int(window), int(grid.value), _ptr(part_o), _ptr(part_ml), _ptr(count),
        _ptr(rope_table), 1 if store_kv else 0, _stream())
    _finish(lib, rc, "attention_decode")


def decode_unit_cost(chunks: int | None = None) -> int:
    """What the balanced decode kernel reckons a block pays for taking up one (request, head
    group) unit, in 64-key chunks, when it cuts the requests' keys into equal stretches (so that a
    block with many short requests gets fewer keys than one inside a long request).  Sets it when
    given; returns the value that was in force before."""
    return int(_lib("attention_mma").mi_attention_decode_balanced_unit_cost(-1 if chunks is None else int(chunks)))


def attention_wait_status(reset: bool = True) -> int:
    """1 if a tensor-core attention kernel gave up waiting for a copy since the last reset
    (its output was then invalid); synchronises the device."""
    return int(_lib("attention_mma").mi_attention_wait_status(1 if reset else 0))


def attention_prefill(q, q_stride, out, kcache, vcache, block_table, page_size, q_start, q_len, kv_len,
                      tile_req, tile_tok0, n_tiles, tile_tokens, nq, nkv, head_dim, scale, window=0,
                      table_rows=None) -> None:
    """bfloat16 attention of query portions of any length over the paged cache (attention_mma.cu)."""
    _cuda(q, out, kcache, vcache, block_table, q_start, q_len, kv_len, tile_req, tile_tok0, table_rows)
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_prefill: bfloat16 only")
    _check_attention_args(q, out, kcache, vcache, block_table, nq, nkv, head_dim, page_size,
                          (("block_table", block_table), ("q_start", q_start), ("q_len", q_len),
                           ("kv_len", kv_len), ("tile_req", tile_req), ("tile_tok0", tile_tok0),
                           ("table_rows", table_rows)))
    lib = _waiting_lib("attention_mma", q.device)
    rc = lib.mi_attention_prefill(
        _ptr(q), int(q_stride), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache), _ptr(block_table),
        block_table.stride(0), _ptr(table_rows), int(page_size), _ptr(q_start), _ptr(q_len), _ptr(kv_len), _ptr(tile_req),
        _ptr(tile_tok0), int(n_tiles), int(tile_tokens), nq, nkv, head_dim, float(scale), int(window),
        _stream())
    _finish(lib, rc, "attention_prefill")


USE_TC_PREFILL = os.environ.get("MINI_INFER_TC_PREFILL", "1") != "0"


def prefill_tc_supported(nq: int, nkv: int, head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 prefill kernel (attention_tc.cu) takes these sizes: head size 64 or
    128, a power-of-two page of 8 to 64 keys, a group size that divides 128.  (The same test as
    the library's own ``mi_attention_prefill_tc_supported``, made here so that a model the
    kernel does not take never compiles it.)"""
    if head_dim not in (64, 128) or page_size < 8 or page_size > 64 or page_size & (page_size - 1):
        return False
    if nq <= 0 or nkv <= 0 or nq % nkv:
        return False
    return 128 % min(nq // nkv, 128) == 0


def attention_prefill_tc(q, q_stride, out, kcache, vcache, block_table, page_size, q_start, q_len, kv_len,
                         tile_req, tile_tok0, n_tiles, tile_tokens, nq, nkv, head_dim, scale, window=0,
                         table_rows=None) -> None:
    """bfloat16 attention of query portions over the paged cache on tcgen05 (attention_tc.cu);
    same arguments as ``attention_prefill``."""
    _cuda(q, out, kcache, vcache, block_table, q_start, q_len, kv_len, tile_req, tile_tok0, table_rows)
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_prefill_tc: bfloat16 only")
    _check_attention_args(q, out, kcache, vcache, block_table, nq, nkv, head_dim, page_size,
                          (("block_table", block_table), ("q_start", q_start), ("q_len", q_len),
                           ("kv_len", kv_len), ("tile_req", tile_req), ("tile_tok0", tile_tok0),
                           ("table_rows", table_rows)))
    lib = _waiting_lib("attention_tc", q.device)
    rc = lib.mi_attention_prefill_tc(
        _ptr(q), int(q_stride), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache), int(kcache.shape[0]),
        _ptr(block_table), block_table.stride(0), _ptr(table_rows), int(page_size), _ptr(q_start), _ptr(q_len), _ptr(kv_len),
        _ptr(tile_req), _ptr(tile_tok0), int(n_tiles), int(tile_tokens), nq, nkv, head_dim, float(scale),
        int(window), _stream())
    _finish(lib, rc, "attention_prefill_tc")


def attention_tc_status(reset: bool = True) -> int:
    """Non-zero when a block of the tcgen05 prefill kernel gave up a bounded wait since the
    last reset (its output is then wrong).  Synchronises the device."""
    return int(_lib("attention_tc").mi_attention_tc_status(1 if reset else 0))


def attention_generic(
    q: torch.Tensor,
    q_stride: int,
    out: torch.Tensor,
    kcache: torch.Tensor,
    vcache: torch.Tensor,
    block_table: torch.Tensor,
    page_size: int,
    q_start: torch.Tensor,
    q_len: torch.Tensor,
    kv_len: torch.Tensor,
    tile_req: torch.Tensor,
    tile_tok0: torch.Tensor,
    n_tiles: int,
    nq: int,
    nkv: int,
    head_dim: int,
    scale: float,
    window: int = 0,
    table_rows: torch.Tensor | None = None,
) -> None:
    """Causal attention of query portions over the paged cache (see attention_generic.cu).

    ``q`` is any tensor whose element ``(token t, head h, k)`` lies at
    ``t * q_stride + h * head_dim + k`` from its first element.
    """
    _cuda(q, out, kcache, vcache, block_table, q_start, q_len, kv_len, tile_req, tile_tok0, table_rows)
    for name, t in (("block_table", block_table), ("q_start", q_start), ("q_len", q_len),
                    ("kv_len", kv_len), ("tile_req", tile_req), ("tile_tok0", tile_tok0),
                    ("table_rows", table_rows)):
        if t is not None and t.dtype != torch.int32:
            raise KernelError(f"attention: {name} must be int32")
    if kcache.dtype != q.dtype or vcache.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelError("attention: q, out and caches must share a dtype")
    if kcache.dim() != 4 or kcache.shape[1:] != (nkv, page_size, head_dim) or not kcache.is_contiguous() \
            or vcache.shape != kcache.shape or not vcache.is_contiguous():
        raise KernelError("attention: caches must be contiguous [pages, nkv, page_size, d]")
    if out.dim() != 2 or out.shape[1] != nq * head_dim or not out.is_contiguous():
        raise KernelError("attention: out must be contiguous [tokens, nq * d]")
    if block_table.dim() != 2 or block_table.stride(1) != 1:
        raise KernelError("attention: block_table must be [requests, pages] with unit inner stride")
    lib = _lib("attention_generic")
    if lib.mi_attention_generic_tile_tokens() != ATTENTION_TILE_TOKENS:
        raise KernelError("attention: the kernel's tile size differs from ATTENTION_TILE_TOKENS")
    rc = lib.mi_attention_generic(
        _ptr(q), int(q_stride), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache),
        _ptr(block_table), block_table.stride(0), _ptr(table_rows), int(page_size), _ptr(q_start), _ptr(q_len),
        _ptr(kv_len), _ptr(tile_req), _ptr(tile_tok0), int(n_tiles), nq, nkv, head_dim,
        float(scale), int(window), _code(q.dtype), _stream())
    _finish(lib, rc, "attention")


def sample(
    logits: torch.Tensor,
    out: torch.Tensor,
    *,
    temperature: torch.Tensor | None = None,
    top_k: torch.Tensor | None = None,
    top_p: torch.Tensor | None = None,
    seed_lo: torch.Tensor | None = None,
    seed_hi: torch.Tensor | None = None,
    draw_index: torch.Tensor | None = None,
) -> torch.Tensor:
    """One token id per row of fp32 ``logits [B, V]`` into int32 ``out [B]`` (see sampling.cu)."""
    _cuda(logits, out, temperature, top_k, top_p, seed_lo, seed_hi, draw_index)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be fp32 [B, V] with unit inner stride")
    B, V = logits.shape
    if out.dtype != torch.int32 or out.shape != (B,) or not out.is_contiguous():
        raise KernelError("sample: out must be int32 [B]")
    for name, t, dt in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                        ("top_p", top_p, torch.float32), ("seed_lo", seed_lo, torch.int32),
                        ("seed_hi", seed_hi, torch.int32), ("draw_index", draw_index, torch.int32)):
        if t is not None and (t.dtype != dt or t.shape != (B,) or not t.is_contiguous()):
            raise KernelError(f"sample: {name} must be {dt} [B]")
    lib = _lib("sampling")
    rc = lib.mi_sample(_ptr(logits), logits.stride(0) if B > 1 else V, B, V, _ptr(temperature),
                       _ptr(top_k), _ptr(top_p), _ptr(seed_lo), _ptr(seed_hi), _ptr(draw_index),
                       _ptr(out), _stream())
    _finish(lib, rc, "sample")
    return out


TMA_GEMM_MAX_ROWS = 128            # what gemm_tma.cu takes
# ``linear`` routes inputs of up to this many rows to gemm_tma.  Measured on a B200 inside a
# captured decode step (Llama 3.1 8B sizes, milliseconds per step, own product against the
# library's): up to 16 rows the own product is ahead, because it marks the weights to leave the
# L2 first and does the block's additions and norms in its epilogues (batch 8: 3.74 vs 4.05;
# batch 16: 4.17 vs 4.42); from 32 rows on the library is (5.23 vs 5.15; 64 rows: 7.34 vs 6.63).
TMA_GEMM_DISPATCH_ROWS = 16
USE_TMA_GEMM = os.environ.get("MINI_INFER_TMA_GEMM", "1") != "0"
_tma_ws: dict[int, list[tuple[torch.Tensor, torch.Tensor]]] = {}


def _tma_workspace(device: torch.device, floats: int, counters: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Partial tiles and per-tile arrival counters (zero between calls) of the streaming
    product, per device; never freed once handed out (a captured graph may hold the address)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    stack = _tma_ws.setdefault(idx, [])
    if not stack or stack[-1][0].numel() < floats or stack[-1][1].numel() < counters:
        stack.append((
            torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=device),
            torch.zeros(max(counters, 4096), dtype=torch.int32, device=device),
        ))
    return stack[-1]


def gemm_tma_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether ``gemm_tma`` takes these operands (few rows, 16-byte aligned rows)."""
    return (x.dim() == 2 and w.dim() == 2 and 0 < x.shape[0] <= TMA_GEMM_MAX_ROWS and x.shape[1] % 8 == 0
            and x.stride(1) == 1 and w.is_contiguous() and (x.shape[0] == 1 or x.stride(0) % 8 == 0)
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


TMA_GEMM_FUSED_ROWS = 16    # the fused epilogues of gemm_tma take one group of 16 token columns
TMA_GEMM_STAT_TOKENS = 16   # columns of a statistics table
TMA_GEMM_TILE_ROWS = 128    # rows of W per tile: one row of a statistics table


class RowStats:
    """Sums of squares of the rows of an fp32 stream ``[M, width]``, 128 features at a time
    (``sums [ceil(width / 128), 16]``, column = row of the stream), as the residual epilogue of
    ``gemm_tma`` leaves them, with the ``eps`` of the norm they are meant for."""

    __slots__ = ("sums", "width", "eps")

    def __init__(self, sums: torch.Tensor, width: int, eps: float) -> None:
        self.sums, self.width, self.eps = sums, int(width), float(eps)


def gemm_tma(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
             swiglu: bool = False, row_stats: RowStats | None = None,
             residual: torch.Tensor | None = None, gain: torch.Tensor | None = None,
             eps: float = 0.0):
    """``x [M <= 128, K] @ w [N, K]^T`` for bfloat16 operands on the tcgen05 tensor cores,
    streaming ``w`` once through TMA (gemm_tma.cu); the result is bfloat16 or float32.  With
    ``swiglu`` the rows of ``w`` alternate gate, up and the result is ``[M, N / 2]``:
    ``silu(gate) * up`` computed on the fp32 accumulators in the product's epilogue.

    Two fused forms for at most 16 rows.  ``row_stats``: every row of the product is first
    scaled by ``rsqrt(sum of its squares / width + eps)`` (the input was multiplied by a norm's
    gain, not yet divided by its root mean square).  ``residual [M, N]`` fp32 with ``gain [N]``
    fp32: the product is added to ``residual`` in place, the result is ``residual * gain`` and a
    second value is returned, the ``RowStats`` of the new residual for a norm with ``eps``."""
    _cuda(x, w)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tma: operands must be bfloat16")
    if x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1] or x.stride(1) != 1 or not w.is_contiguous():
        raise KernelError(f"gemm_tma: shapes {tuple(x.shape)} x {tuple(w.shape)}^T do not match")
    M, K = x.shape
    N = w.shape[0]
    lib = _waiting_lib("gemm_tma", x.device)
    blocks = _sms(x.device)
    floats, counters = ctypes.c_longlong(0), c_int(0)
    lib.mi_gemm_tma_workspace(M, N, blocks, ctypes.byref(floats), ctypes.byref(counters))
    partial, count = _tma_workspace(x.device, int(floats.value), int(counters.value))
    if swiglu and N % 2:
        raise KernelError("gemm_tma: the gate/up epilogue needs an even number of rows")
    n_out = N // 2 if swiglu else N
    out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
    sums_in = tiles_in = width = None
    if row_stats is not None:
        sums_in, width = row_stats.sums, row_stats.width
        tiles_in = -(-width // TMA_GEMM_TILE_ROWS)
        if (width != K or sums_in.dtype != torch.float32 or not sums_in.is_contiguous()
                or tuple(sums_in.shape) != (tiles_in, TMA_GEMM_STAT_TOKENS)):
            raise KernelError(f"gemm_tma: row statistics {tuple(sums_in.shape)} of width {width} do not fit K = {K}")
    stats_out = None
    if residual is not None:
        if (gain is None or gain.dtype != torch.float32 or gain.numel() != N or not gain.is_contiguous()
                or residual.dtype != torch.float32 or tuple(residual.shape) != (M, N) or not residual.is_contiguous()):
            raise KernelError("gemm_tma: the residual epilogue needs a contiguous fp32 stream [M, N] and an fp32 gain [N]")
        _cuda(residual, gain)
        stats_out = torch.empty((-(-N // TMA_GEMM_TILE_ROWS), TMA_GEMM_STAT_TOKENS), dtype=torch.float32,
                                device=x.device)
    rc = lib.mi_gemm_tma_fused(_ptr(x), x.stride(0) if M > 1 else K, _ptr(w), _ptr(out), n_out, M, N, K,
                               _code(out_dtype), 1 if swiglu else 0, blocks, _ptr(partial), _ptr(count),
                               _ptr(sums_in), tiles_in or 0, width or 0, row_stats.eps if row_stats else 0.0,
                               _ptr(residual), _ptr(gain), _ptr(stats_out), _stream())
    _finish(lib, rc, "gemm_tma")
    if residual is not None:
        return out, RowStats(stats_out, N, eps)
    return out


def gemm_tma_status(reset: bool = True) -> int:
    """Non-zero when a block of the streaming product gave up a bounded wait since the last
    reset (its output is then wrong).  Synchronises the device."""
    return int(_lib("gemm_tma").mi_gemm_tma_status(1 if reset else 0))


def fused_norms_enabled() -> bool:
    """Whether additions and norms may ride on the streaming product's epilogues
    (``MINI_INFER_FUSED_NORMS=0`` keeps them as kernels of their own, for comparisons)."""
    return USE_TMA_GEMM and os.environ.get("MINI_INFER_FUSED_NORMS", "1") != "0"


def linear_fusable(n_rows: int, w: torch.Tensor) -> bool:
    """Whether a product of ``n_rows`` rows with ``w`` has the fused forms of ``gemm_tma``
    (``row_stats`` on its input side, ``linear_into_stream`` on its output side)."""
    return (fused_norms_enabled() and 0 < n_rows <= min(TMA_GEMM_DISPATCH_ROWS, TMA_GEMM_FUSED_ROWS)
            and w.is_cuda and w.dtype == torch.bfloat16 and w.dim() == 2 and w.is_contiguous()
            and w.shape[1] % 8 == 0 and w.data_ptr() % 16 == 0)


def linear_into_stream(x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor, gain: torch.Tensor,
                       eps: float) -> tuple[torch.Tensor, "RowStats"]:
    """``residual += x w^T`` in place (fp32); returns ``residual * gain`` in bfloat16 and the row
    statistics a product with ``row_stats`` needs to finish an RMS norm with ``eps``."""
    if not linear_fusable(x.shape[0], w) or not gemm_tma_ok(x, w):
        raise KernelError("linear_into_stream: these operands have no fused form (ask linear_fusable first)")
    return gemm_tma(x, w, torch.bfloat16, residual=residual, gain=gain, eps=eps)


def linear_swiglu(x: torch.Tensor, w_pairs: torch.Tensor, row_stats: "RowStats | None" = None) -> torch.Tensor:
    """``silu(x Wg^T) * (x Wu^T)`` for a merged projection whose rows alternate gate, up
    (``w_pairs [2 I, K]``).  Decode-sized bfloat16 inputs run the product and the activation
    as one kernel (gemm_tma with its gate/up epilogue); everything else runs ``linear`` and
    the SiLU-multiply kernel on the interleaved result.  ``row_stats``: see ``gemm_tma``."""
    if (x.dtype == torch.bfloat16 and USE_TMA_GEMM and x.shape[0] <= TMA_GEMM_DISPATCH_ROWS
            and w_pairs.dtype == torch.bfloat16 and gemm_tma_ok(x, w_pairs)):
        return gemm_tma(x, w_pairs, torch.bfloat16, swiglu=True, row_stats=row_stats)
    if row_stats is not None:
        raise KernelError("linear_swiglu: row statistics need the streaming product (ask linear_fusable first)")
    return silu_mul(linear(x, w_pairs), pairs=True)


_MM_OUT_DTYPE: bool | None = None


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None,
           row_stats: "RowStats | None" = None) -> torch.Tensor:
    """``x [M, K] @ w [N, K]^T``.

    float32 operands run the true-fp32 CUDA-core kernel (never a library product, which
    could pick a reduced-precision mode).  bfloat16 operands with few rows (decode) run the
    weight-streaming tcgen05 kernel of gemm_tma.cu, which starts streaming weights while the
    kernel before it still runs; other bfloat16 operands use the library product with fp32
    accumulation, as the reference does for every linear layer (``distributed/linear.py:167``).
    ``out_dtype=float32`` keeps the accumulator's precision in the result (used for logits).
    ``row_stats`` (streaming product only): see ``gemm_tma``.
    """
    global _MM_OUT_DTYPE, launch_count
    if row_stats is not None:
        if not linear_fusable(x.shape[0], w) or not gemm_tma_ok(x, w):
            raise KernelError("linear: row statistics need the streaming product (ask linear_fusable first)")
        return gemm_tma(x, w, out_dtype or torch.bfloat16, row_stats=row_stats)
    if x.dtype == torch.float32:
        if w.dtype != torch.float32:
            raise KernelError("linear: fp32 activations need fp32 weights")
        return gemm_f32(x, w)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"linear: unsupported dtypes {x.dtype} x {w.dtype}")
    _cuda(x, w)
    if out_dtype not in (None, torch.bfloat16, torch.float32):
        raise KernelError(f"linear: unsupported output dtype {out_dtype}")
    if USE_TMA_GEMM and x.shape[0] <= TMA_GEMM_DISPATCH_ROWS and gemm_tma_ok(x, w):
        return gemm_tma(x, w, out_dtype or torch.bfloat16)
    launch_count += 1
    if out_dtype in (None, torch.bfloat16):
        return torch.mm(x, w.t())
    if out_dtype != torch.float32:
        raise KernelError(f"linear: unsupported output dtype {out_dtype}")
    if _MM_OUT_DTYPE is None:
        try:
            torch.mm(x[:1], w[:1].t(), out_dtype=torch.float32)
            _MM_OUT_DTYPE = True
        except (TypeError, RuntimeError):
            _MM_OUT_DTYPE = False
    if _MM_OUT_DTYPE:
        return torch.mm(x, w.t(), out_dtype=torch.float32)
    return torch.mm(x, w.t()).float()
