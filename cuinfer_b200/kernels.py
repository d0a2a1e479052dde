"""Python face of the CUDA kernels: one thin function per exported entry point.

The shared library is compiled from ``cuinfer_b200/csrc`` on first use (see ``csrc/build.py``) and
loaded with ctypes.  Every function takes torch CUDA tensors, checks dtypes, shapes and contiguity,
and launches on torch's current stream, so that calls are ordered with torch's own work and are
recorded when a CUDA graph is being captured.  There is no CPU or library fallback: if the library
cannot be built or loaded, or a tensor is not on a CUDA device, the call raises.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

_lib_handle: Optional[ctypes.CDLL] = None
_lib_lock = threading.Lock()

# Number of kernel launches issued through this module (each wrapper call launches one kernel unless
# it says otherwise).  The benchmark reads it.
launch_count = 0


class KernelError(RuntimeError):
    pass


def library() -> ctypes.CDLL:
    """The loaded kernel library; built first if it is missing or stale."""
    global _lib_handle
    if _lib_handle is not None:
        return _lib_handle
    with _lib_lock:
        if _lib_handle is not None:
            return _lib_handle
        try:
            path = _build.build(verbose=True)
            lib = ctypes.CDLL(path)
        except Exception as exc:  # noqa: BLE001 - anything here means the product path cannot run
            raise KernelError(
                "the CUDA kernel library of cuinfer_b200 is not available, and there is no fallback: "
                f"{type(exc).__name__}: {exc}"
            ) from exc
        lib.cib_last_error.restype = ctypes.c_char_p
        _declare(lib)
        lib.cib_set_prompt_pdl.argtypes = [ctypes.c_int]
        lib.cib_set_prompt_pdl.restype = None
        lib.cib_set_prompt_pdl(1 if os.environ.get("CUINFER_B200_PROMPT_PDL", "1") != "0" and os.environ.get("CUINFER_B200_PDL", "1") != "0" else 0)
        _lib_handle = lib
        return lib


def library_path() -> str:
    library()
    return _build.library_path()


_P, _I, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


def _declare(lib: ctypes.CDLL) -> None:
    sig = {
        "cib_embedding_gather": [_P, _P, _I, _P, _I, _I, _I, _P, _P],
        "cib_add_rmsnorm": [_P, _P, _I, _P, _I, _F, _P, _I, _I, _I, _P],
        "cib_gather_rows": [_P, _P, _I, _P, _P, _I, _I, _I, _P],
        "cib_silu_mul": [_P, _P, _I, _I, _I, _P],
        "cib_qk_norm_rope_kv_write": [_P, _I, _I, _P, _P, _P, _P, _I, _I, _F, _P, _I, _I, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P],
        "cib_paged_attention_generic": [_P, _I, _I, _P, _I, _P, _I, _I, _P, _I, _P, _P, _P, _I, _I, _I, _I, _F, _I, _P],
        "cib_paged_attention_decode": [_P, _I, _P, _I, _P, _I, _I, _P, _I, _P, _I, _I, _I, _I, _F, _I, _I, _P, _P, _I, _P, _P, ctypes.c_longlong, _P],
        "cib_paged_attention_prefill": [_P, _I, _P, _I, _P, _I, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P],
        "cib_attention_tcgen05": [_P, _I, _P, _I, _P, _I, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P, _P],
        "cib_gemm_skinny": [_P, _I, _I, _I, _P, _I, _P, _P, _I, _P, _I, _F, _P, _P, _I, _I, _I, _I, _I, _P, ctypes.c_longlong, _P],
        "cib_gemm_tcgen05": [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _P, _P],
        "cib_gemm_wstream": [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _P, _P],
        "cib_gemm_generic": [_P, _I, _P, _I, _I, _P, _I, _I, _I, _I, _I, _P],
        "cib_sample": [_P, _I, _I, _I, _P, _P, _P],
        "cib_argmax_rows": [_P, _I, _I, _I, _P, _P],
        "cib_selftest_bounded_wait": [ctypes.c_longlong, _P, _P, _P],
        "cib_fill_random": [_P, _I, ctypes.c_longlong, ctypes.c_ulonglong, ctypes.c_double, ctypes.c_double, _F, _I, _P],
    }
    for name, argtypes in sig.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = _I
    lib.cib_paged_attention_decode_supports.argtypes = [_I, _I, _I]
    lib.cib_paged_attention_decode_supports.restype = _I
    lib.cib_gemm_tcgen05_supports.argtypes = [_I, _I, _I]
    lib.cib_gemm_tcgen05_supports.restype = _I
    lib.cib_attention_tcgen05_supports.argtypes = [_I, _I, _I, _I]
    lib.cib_attention_tcgen05_supports.restype = _I
    lib.cib_gemm_wstream_supports.argtypes = [_I, _I, _I]
    lib.cib_gemm_wstream_supports.restype = _I
    lib.cib_gemm_skinny_supports.argtypes = [_I, _I, _I, _I]
    lib.cib_gemm_skinny_supports.restype = _I
    lib.cib_paged_attention_prefill_supports.argtypes = [_I, _I, _I]
    lib.cib_paged_attention_prefill_supports.restype = _I
    lib.cib_paged_attention_decode_scratch_floats.argtypes = [_I, _I, _I, _I]
    lib.cib_paged_attention_decode_scratch_floats.restype = ctypes.c_longlong


def _check(rc: int, name: str) -> None:
    if rc != 0:
        msg = library().cib_last_error()
        raise KernelError(f"{name} failed ({rc}): {msg.decode() if msg else 'no message'}")


# torch's current stream as a raw pointer.  The private accessors skip the construction of a Stream object, which is
# a microsecond and a half on every launch; without them the public call is used.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _code(t: torch.Tensor, what: str) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise KernelError(f"{what}: dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _cuda(t: torch.Tensor, what: str, dtype: torch.dtype | None = None, contiguous: bool = True) -> int:
    if not t.is_cuda:
        raise KernelError(f"{what} must be a CUDA tensor; cuinfer_b200 has no CPU path")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")
    return t.data_ptr()


def _count() -> None:
    global launch_count
    launch_count += 1


# ---- row-wise kernels ----------------------------------------------------------------------------

def embedding_gather(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, bad_flag: torch.Tensor | None = None) -> None:
    """out[t] = table[ids[t]] as float32 rows."""
    T = ids.numel()
    V, H = table.shape
    if out.shape != (T, H):
        raise KernelError(f"embedding_gather: out must be [{T}, {H}], got {list(out.shape)}")
    rc = library().cib_embedding_gather(
        _cuda(ids, "ids", torch.int32), _cuda(table, "table"), _code(table, "table"), _cuda(out, "out", torch.float32),
        T, H, V, _cuda(bad_flag, "bad_flag", torch.int32) if bad_flag is not None else None, _stream())
    _check(rc, "embedding_gather")
    _count()


def add_rmsnorm(residual: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor | None, eps: float,
                out: torch.Tensor | None) -> None:
    """residual += delta (if given); out = rmsnorm(residual) * weight (if out given)."""
    rows, H = residual.shape
    if delta is not None and delta.shape != residual.shape:
        raise KernelError(f"add_rmsnorm: delta {list(delta.shape)} does not match residual {list(residual.shape)}")
    if out is not None:
        if out.shape != residual.shape:
            raise KernelError(f"add_rmsnorm: out {list(out.shape)} does not match residual {list(residual.shape)}")
        if weight is None or weight.numel() != H:
            raise KernelError(f"add_rmsnorm: weight must have {H} elements")
    rc = library().cib_add_rmsnorm(
        _cuda(residual, "residual", torch.float32),
        _cuda(delta, "delta") if delta is not None else None, _code(delta, "delta") if delta is not None else 0,
        _cuda(weight, "weight") if weight is not None else None, _code(weight, "weight") if weight is not None else 0,
        float(eps), _cuda(out, "out") if out is not None else None, _code(out, "out") if out is not None else 0,
        rows, H, _stream())
    _check(rc, "add_rmsnorm")
    _count()


def gather_rows(residual: torch.Tensor, delta: torch.Tensor | None, indices: torch.Tensor, out: torch.Tensor) -> None:
    """out[s] = residual[indices[s]] (+ delta[indices[s]]), float32."""
    rows, H = residual.shape
    S = indices.numel()
    if out.shape != (S, H):
        raise KernelError(f"gather_rows: out must be [{S}, {H}]")
    rc = library().cib_gather_rows(
        _cuda(residual, "residual", torch.float32),
        _cuda(delta, "delta") if delta is not None else None, _code(delta, "delta") if delta is not None else 0,
        _cuda(indices, "indices", torch.int32), _cuda(out, "out", torch.float32), S, H, rows, _stream())
    _check(rc, "gather_rows")
    _count()


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, j] = silu(gate_up[t, j]) * gate_up[t, I + j]."""
    rows, two_i = gate_up.shape
    inter = two_i // 2
    if two_i != 2 * inter or out.shape != (rows, inter) or out.dtype != gate_up.dtype:
        raise KernelError(f"silu_mul: gate_up {list(gate_up.shape)} / out {list(out.shape)} do not fit")
    rc = library().cib_silu_mul(_cuda(gate_up, "gate_up"), _cuda(out, "out"), _code(gate_up, "gate_up"), rows, inter, _stream())
    _check(rc, "silu_mul")
    _count()


# ---- attention -------------------------------------------------------------------------------------

def qk_norm_rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, slot_mapping: torch.Tensor | None,
                          q_weight: torch.Tensor | None, k_weight: torch.Tensor | None, eps: float,
                          rope_table: torch.Tensor | None, rotary_dim: int, cache: torch.Tensor | None,
                          num_q_heads: int, num_kv_heads: int, head_dim: int) -> None:
    """Per-head RMSNorm (if weights are given) and rotary encoding (if a table is given) of the query and
    key heads of the packed ``qkv`` rows; queries are rewritten in place, keys and values are written to
    ``cache[page, 0|1, kv head, slot, :]`` (if a cache is given)."""
    T, stride = qkv.shape
    has_norm = q_weight is not None
    if has_norm and (k_weight is None or q_weight.dtype != k_weight.dtype):
        raise KernelError("qk_norm_rope: q and k norm weights must both be given, in one dtype")
    write_cache = cache is not None
    if write_cache:
        if cache.dim() != 5 or cache.shape[1] != 2 or cache.shape[2] != num_kv_heads or cache.shape[4] != head_dim:
            raise KernelError(f"qk_norm_rope: cache must be [pages, 2, {num_kv_heads}, page_size, {head_dim}], got {list(cache.shape)}")
        if cache.dtype != qkv.dtype:
            raise KernelError("qk_norm_rope: cache and qkv must have one dtype")
        if slot_mapping is None:
            raise KernelError("qk_norm_rope: a cache write needs slot_mapping")
    if rope_table is not None and (rope_table.dim() != 3 or rope_table.shape[1] * 2 != rotary_dim or rope_table.shape[2] != 2):
        raise KernelError(f"qk_norm_rope: rope table must be [positions, {rotary_dim // 2}, 2], got {list(rope_table.shape)}")
    rc = library().cib_qk_norm_rope_kv_write(
        _cuda(qkv, "qkv"), _code(qkv, "qkv"), stride, _cuda(positions, "positions", torch.int32),
        _cuda(slot_mapping, "slot_mapping", torch.int32) if slot_mapping is not None else None,
        _cuda(q_weight, "q_weight") if has_norm else None, _cuda(k_weight, "k_weight") if has_norm else None,
        _code(q_weight, "q_weight") if has_norm else 0, 1 if has_norm else 0, float(eps),
        _cuda(rope_table, "rope_table", torch.float32) if rope_table is not None else None,
        rotary_dim if rope_table is not None else 0, rope_table.shape[0] if rope_table is not None else 0,
        _cuda(cache, "cache") if write_cache else None, cache.shape[0] if write_cache else 0,
        cache.shape[3] if write_cache else 0, T, num_q_heads, num_kv_heads, head_dim, 1 if write_cache else 0,
        1 if use_pdl else 0, _stream())
    _check(rc, "qk_norm_rope_kv_write")
    _count()


def paged_attention_generic(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                            query_start_loc: torch.Tensor, seq_lens: torch.Tensor, token_request: torch.Tensor,
                            num_q_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: int = 0) -> None:
    """Causal attention of the packed query rows ``q[:, :nq*d]`` over the paged cache; out[T, nq*d]."""
    T = q.shape[0]
    if q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("paged_attention: q and out rows must be dense")
    if out.shape != (T, num_q_heads * head_dim) or out.dtype != q.dtype or cache.dtype != q.dtype:
        raise KernelError("paged_attention: out/cache do not fit q")
    rc = library().cib_paged_attention_generic(
        _cuda(q, "q", contiguous=False), _code(q, "q"), q.stride(0), _cuda(out, "out", contiguous=False), out.stride(0),
        _cuda(cache, "cache"), cache.shape[0], cache.shape[3],
        _cuda(block_table, "block_table", torch.int32), block_table.stride(0),
        _cuda(query_start_loc, "query_start_loc", torch.int32), _cuda(seq_lens, "seq_lens", torch.int32),
        _cuda(token_request, "token_request", torch.int32), T, num_q_heads, num_kv_heads, head_dim, float(scale),
        int(window), _stream())
    _check(rc, "paged_attention_generic")
    _count()


_decode_counters: dict = {}
_retired: list = []


def paged_attention_decode_supports(head_dim: int, num_q_heads: int, num_kv_heads: int) -> bool:
    return bool(library().cib_paged_attention_decode_supports(head_dim, num_q_heads, num_kv_heads))


# CUINFER_B200_DECODE_TMA=0 keeps the decode attention kernel on its cp.async path (for comparisons).
decode_tma = os.environ.get("CUINFER_B200_DECODE_TMA", "1") != "0"


DECODE_TMA_MIN_KEYS = int(os.environ.get("CUINFER_B200_DECODE_TMA_MIN_KEYS", "1024"))      # keys per CTA from which the TMA path of the decode kernel pays inside a step (measured)


def decode_tma_takes(page_size: int, head_dim: int, window: int) -> bool:
    """Whether the decode attention can stream its keys and values as TMA page boxes for this cache layout (else
    cp.async only): whole 16-slot blocks inside a page, 64-column panels, no window."""
    return decode_tma and page_size % 16 == 0 and head_dim % 64 == 0 and window <= 0


def decode_uses_tma(max_seq_len: int, splits: int) -> bool:
    """The TMA path streams faster, but it starts later after the kernel before it in a step (the cp.async path asks
    for its first blocks before that kernel has ended): timed alone it wins at every size, inside a decode step only
    for long streams per CTA (batch 1 with 26 CTAs of 160 keys per head: 919 tokens/s against 974 on cp.async)."""
    return -(-max_seq_len // splits) >= DECODE_TMA_MIN_KEYS


def decode_slots(head_dim: int) -> int:
    """CTAs of the decode attention kernel that the GPU runs at a time: its key and value rings take 768 bytes per
    value of the head size, so one CTA per SM at head size 256, two at 128, and three (by registers) below."""
    return 148 * (1 if head_dim > 128 else 2 if head_dim > 64 else 3)


def decode_splits(num_requests: int, num_kv_heads: int, max_seq_len: int, slots: int = 296, tma: bool = False,
                  head_dim: int = 128) -> int:
    """How many CTAs share the keys of one (request, kv head).  ``tma``: the cache layout allows the TMA path, which
    a split then takes if it leaves a CTA ``DECODE_TMA_MIN_KEYS`` keys or more.

    The GPU runs ``slots`` CTAs of this kernel at a time (two on each of the 148 SMs); a CTA's four warps take
    16-key blocks in turn, so a CTA's share counts in steps of 64 keys.  A launch is estimated, in nanoseconds, round
    of CTAs by round: a round of n CTAs takes keys per CTA x (the larger of a CTA's own pace per key and n x 0.072, the
    memory's pace when n CTAs stream at once) plus a fixed cost for a CTA's start and its partial results; splitting
    adds 3000 for the combine and 40 per split.  A CTA's own pace is 16 per key and 3000 fixed on the TMA path, 18 and
    4000 on the cp.async path.  The constants were fitted to timings at batch 1 to 128 with 300 to 9000 keys of head
    size 128 (largest miss 1.7 us, 9 % r.m.s. error of the estimate); for another head size the costs per key scale
    with the bytes of a key.  The smallest estimate wins.
    """
    pairs = max(1, num_requests * num_kv_heads)
    width = head_dim / 128.0
    best, best_cost = 1, None
    for s in range(1, 65):
        keys = -(-(-(-max_seq_len // s)) // 64) * 64
        if s > 1 and (s - 1) * keys >= max_seq_len:
            continue                                   # the last CTA would get nothing: a smaller s does the same
        per_key, fixed = (16.0 * width, 3000.0) if tma and decode_uses_tma(max_seq_len, s) else (18.0 * width, 4000.0)
        full, rest = divmod(pairs * s, slots)
        cost = full * (keys * max(per_key, 0.072 * width * slots) + fixed)
        if rest:
            cost += keys * max(per_key, 0.072 * width * rest) + fixed
        if s > 1:
            cost += 3000.0 + 40.0 * s
        if best_cost is None or cost < best_cost:
            best, best_cost = s, cost
    return best


# A kernel of the decode chain may ask for the weights of the kernel after it to be fetched into the L2 while it runs.
# That pays where the chain is bound by latencies and the weights are small beside the 126 MB L2 (every matrix of the
# 0.6B layer sizes is under 13 MB).  Matrices of 33 to 200 MB (the 8B layer sizes) would compete with the running
# kernel's own stream and could not stay in the L2 until they are used, so larger ones are not asked for.
L2_HINT_MAX_BYTES = 16 << 20


def _l2_hint(warm: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    if warm is None or warm.numel() * warm.element_size() > L2_HINT_MAX_BYTES:
        return None
    return warm


def paged_attention_decode(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                           seq_lens: torch.Tensor, num_q_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                           window: int, splits: int, tma: bool | None = None, warm: torch.Tensor | None = None) -> None:
    """bfloat16 attention of one query token per request (``q[r, :nq*d]``) over the paged cache, the keys of
    every (request, kv head) split over ``splits`` CTAs.  Allocates the partial-result scratch with torch.
    ``tma``: let the kernel fetch the cache through TMA where the geometry allows it (default: yes).  That path
    streams faster but starts slower, so callers that know the keys per CTA pass False for short streams.
    ``warm``: a tensor that the kernel after this one reads first; fetched into the L2 when the stream of keys ends."""
    R = q.shape[0]
    warm = _l2_hint(warm)
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("paged_attention_decode: bfloat16 only")
    if q.stride(1) != 1 or out.stride(1) != 1 or out.shape != (R, num_q_heads * head_dim):
        raise KernelError("paged_attention_decode: q/out rows must be dense and out [R, nq*d]")
    scratch = None
    counters = None
    if splits > 1:
        n = library().cib_paged_attention_decode_scratch_floats(R, num_q_heads, head_dim, splits)
        scratch = torch.empty(n, dtype=torch.float32, device=q.device)
        need = R * num_kv_heads
        counters = _decode_counters.get(q.device.index)
        if counters is None or counters.numel() < need:
            if torch.cuda.is_current_stream_capturing():
                raise KernelError("paged_attention_decode: the split counters must exist before a graph capture "
                                  "(run the step once eagerly first)")
            if counters is not None:
                _retired.append(counters)      # a captured graph may still point at the old buffer
            counters = torch.zeros(max(need, 4096), dtype=torch.int32, device=q.device)
            _decode_counters[q.device.index] = counters
    rc = library().cib_paged_attention_decode(
        _cuda(q, "q", contiguous=False), q.stride(0), _cuda(out, "out", contiguous=False), out.stride(0),
        _cuda(cache, "cache"), cache.shape[0], cache.shape[3], _cuda(block_table, "block_table", torch.int32),
        block_table.stride(0), _cuda(seq_lens, "seq_lens", torch.int32), R, num_q_heads, num_kv_heads, head_dim,
        float(scale), int(window), int(splits), scratch.data_ptr() if scratch is not None else None,
        counters.data_ptr() if counters is not None else None, 1 if use_pdl else 0,
        _error_flag(q.device).data_ptr() if decode_tma and tma is not False else None,
        warm.data_ptr() if warm is not None else None, warm.numel() * warm.element_size() if warm is not None else 0,
        _stream())
    _check(rc, "paged_attention_decode")
    note_flagged_launch()
    _count()


def paged_attention_prefill_supports(head_dim: int, num_q_heads: int, num_kv_heads: int) -> bool:
    return bool(library().cib_paged_attention_prefill_supports(head_dim, num_q_heads, num_kv_heads))


def paged_attention_prefill(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                            query_start_loc: torch.Tensor, seq_lens: torch.Tensor, query_lens_host, num_q_heads: int,
                            num_kv_heads: int, head_dim: int, scale: float, window: int = 0) -> None:
    """bfloat16 tensor-core attention for any mix of prompt portions and decoded tokens.
    ``query_lens_host``: tokens each request brings in this step (host ints), to size the grid."""
    T = q.shape[0]
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("paged_attention_prefill: bfloat16 only")
    if q.stride(1) != 1 or out.stride(1) != 1 or out.shape != (T, num_q_heads * head_dim):
        raise KernelError("paged_attention_prefill: q/out rows must be dense and out [T, nq*d]")
    g = num_q_heads // num_kv_heads
    # CTAs take 64-row tiles one by one, or in pairs (tile p with tile t-1-p: equal work under the causal mask)
    # when the pairs alone still fill the GPU
    paired = sum(((n * g + 63) // 64 + 1) // 2 for n in query_lens_host)
    pair = 1 if paired * num_kv_heads >= 200 else 0
    tiles = paired if pair else sum((n * g + 63) // 64 for n in query_lens_host)
    rc = library().cib_paged_attention_prefill(
        _cuda(q, "q", contiguous=False), q.stride(0), _cuda(out, "out", contiguous=False), out.stride(0),
        _cuda(cache, "cache"), cache.shape[0], cache.shape[3], _cuda(block_table, "block_table", torch.int32),
        block_table.stride(0), _cuda(query_start_loc, "query_start_loc", torch.int32),
        _cuda(seq_lens, "seq_lens", torch.int32), len(query_lens_host), tiles, num_q_heads, num_kv_heads, head_dim,
        float(scale), int(window), pair, _stream())
    _check(rc, "paged_attention_prefill")
    _count()


# ---- matrix product ----------------------------------------------------------------------------------

def gemm_generic(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T with 32-bit FMA accumulation, any sizes."""
    M, K = a.shape
    N, K2 = w.shape
    if K != K2 or out.shape != (M, N) or a.dtype != w.dtype:
        raise KernelError(f"gemm: a {list(a.shape)} {a.dtype}, w {list(w.shape)} {w.dtype}, out {list(out.shape)} do not fit")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm: rows must be dense")
    rc = library().cib_gemm_generic(
        _cuda(a, "a", contiguous=False), a.stride(0), _cuda(w, "w", contiguous=False), w.stride(0), _code(a, "a"),
        _cuda(out, "out", contiguous=False), out.stride(0), _code(out, "out"), M, N, K, _stream())
    _check(rc, "gemm_generic")
    _count()


# Programmatic dependent launch for the kernels that support it: such a kernel may start, and prefetch its
# weights, while the kernel before it in the stream is still running; it reads that kernel's results only after
# `griddepcontrol.wait`.  CUINFER_B200_PDL=0 switches it off.
use_pdl = os.environ.get("CUINFER_B200_PDL", "1") != "0"

EPILOGUE_BF16, EPILOGUE_F32, EPILOGUE_SILU_PAIR = 0, 1, 2


def gemm_skinny_supports(M: int, N: int, K: int, with_norm: bool = False) -> bool:
    return bool(library().cib_gemm_skinny_supports(M, N, K, 1 if with_norm else 0))


def gemm_skinny(w: torch.Tensor, out: torch.Tensor, *, act: torch.Tensor | None = None,
                residual: torch.Tensor | None = None, pending: torch.Tensor | None = None,
                norm_weight: torch.Tensor | None = None, eps: float = 0.0, residual_out: torch.Tensor | None = None,
                silu_pair: bool = False, warm: torch.Tensor | None = None) -> None:
    """out = act @ w^T for at most 16 rows, bfloat16 weights.  ``warm``: a tensor that the kernel after this one
    reads first (its weights); the kernel asks for it to be fetched into the L2 while it runs.

    Either ``act`` [M, K] is given, or ``residual`` (float32 [M, K]) with optional ``pending``: then the rows are
    RMSNorm(residual + pending) * norm_weight, computed in the kernel, and ``residual_out`` (another buffer)
    receives residual + pending.  ``silu_pair``: ``w`` is [2I, K] = gates then ups and out [M, I] = silu(g) * u.
    ``out`` float32 selects the 32-bit store."""
    N, K = w.shape
    M = out.shape[0]
    warm = _l2_hint(warm)
    if w.dtype != torch.bfloat16 or w.stride(1) != 1:
        raise KernelError("gemm_skinny: weights must be bfloat16 with dense rows")
    if silu_pair:
        epi = EPILOGUE_SILU_PAIR
        if out.dtype != torch.bfloat16 or out.shape[1] * 2 != N:
            raise KernelError("gemm_skinny: a gate/up pair writes bfloat16 [M, N/2]")
    else:
        if out.shape[1] != N:
            raise KernelError(f"gemm_skinny: out must be [M, {N}]")
        epi = EPILOGUE_F32 if out.dtype == torch.float32 else EPILOGUE_BF16
        if out.dtype not in (torch.float32, torch.bfloat16):
            raise KernelError("gemm_skinny: out must be bfloat16 or float32")
    if out.stride(1) != 1:
        raise KernelError("gemm_skinny: out rows must be dense")
    if act is not None:
        if act.dtype != torch.bfloat16 or act.shape != (M, K) or act.stride(1) != 1:
            raise KernelError("gemm_skinny: act must be bfloat16 [M, K] with dense rows")
    else:
        if residual is None or residual.dtype != torch.float32 or residual.shape != (M, K) or not residual.is_contiguous():
            raise KernelError("gemm_skinny: residual must be contiguous float32 [M, K]")
        if pending is not None and (pending.shape != (M, K) or not pending.is_contiguous()):
            raise KernelError("gemm_skinny: pending must be contiguous [M, K]")
        if norm_weight is None or norm_weight.numel() != K:
            raise KernelError("gemm_skinny: the norm needs K weights")
        if residual_out is not None and (residual_out.shape != (M, K) or residual_out.dtype != torch.float32
                                         or residual_out.data_ptr() == residual.data_ptr()):
            raise KernelError("gemm_skinny: residual_out must be another float32 [M, K] buffer")
    rc = library().cib_gemm_skinny(
        _cuda(w, "w", contiguous=False), w.stride(0), N, K,
        _cuda(act, "act", contiguous=False) if act is not None else None, act.stride(0) if act is not None else 0,
        _cuda(residual, "residual") if residual is not None else None,
        _cuda(pending, "pending") if pending is not None else None, _code(pending, "pending") if pending is not None else 0,
        _cuda(norm_weight, "norm_weight") if norm_weight is not None else None,
        _code(norm_weight, "norm_weight") if norm_weight is not None else 0, float(eps),
        _cuda(residual_out, "residual_out") if residual_out is not None else None,
        _cuda(out, "out", contiguous=False), out.stride(0), M, epi, N // 2 if silu_pair else 0, 1 if use_pdl else 0,
        warm.data_ptr() if warm is not None else None, warm.numel() * warm.element_size() if warm is not None else 0,
        _stream())
    _check(rc, "gemm_skinny")
    _count()


_error_flags: dict = {}


def _error_flag(device: torch.device) -> torch.Tensor:
    """One int per device that kernels with bounded waits raise instead of hanging."""
    flag = _error_flags.get(device.index)
    if flag is None:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the device error flag must exist before a graph capture (run the step once eagerly first)")
        flag = torch.zeros(1, dtype=torch.int32, device=device)
        _error_flags[device.index] = flag
    return flag


_flagged_launches = 0
_unchecked_steps = 0
CHECK_EVERY = 32          # a captured step that is replayed is looked at this often, not after every replay


def note_flagged_launch(replayed: bool = False) -> None:
    """Record that a kernel with bounded waits has run.  ``replayed``: it ran as part of a replayed CUDA graph, which
    happens every decode step; the flag is then read only every ``CHECK_EVERY`` steps (and whenever ``force`` is given),
    so that a step does not pay a device-to-host read for it."""
    global _flagged_launches, _unchecked_steps
    if replayed:
        _unchecked_steps += 1
    else:
        _flagged_launches += 1


def check_error_flags(force: bool = False) -> None:
    """Raise if a kernel gave up on a bounded wait since the last check.  Reads one int per device (which
    synchronises), but only if such a kernel was launched since the last check."""
    global _flagged_launches, _unchecked_steps
    if _flagged_launches == 0 and not (_unchecked_steps >= CHECK_EVERY or (force and _unchecked_steps)):
        return
    _flagged_launches = 0
    _unchecked_steps = 0
    for index, flag in _error_flags.items():
        code = int(flag.item())
        if code:
            flag.zero_()
            raise KernelError(f"a kernel on cuda:{index} gave up waiting on a barrier (code {code}); its results are invalid")


def selftest_bounded_wait(limit_cycles: int = 1_000_000, device: torch.device | str = "cuda:0",
                          gave_up: torch.Tensor | None = None) -> None:
    """Run the kernels' bounded mbarrier wait on a barrier that never completes (it gives up after ``limit_cycles``
    and raises the device's error word); the next ``check_error_flags`` must then raise.  For tests of the failure
    path: a healthy kernel never takes it."""
    device = torch.device(device)
    rc = library().cib_selftest_bounded_wait(int(limit_cycles), _error_flag(device).data_ptr(),
                                             _cuda(gave_up, "gave_up", torch.int32) if gave_up is not None else None, _stream())
    _check(rc, "selftest_bounded_wait")
    note_flagged_launch()
    _count()


def attention_tcgen05_supports(head_dim: int, num_q_heads: int, num_kv_heads: int, page_size: int) -> bool:
    return bool(library().cib_attention_tcgen05_supports(head_dim, num_q_heads, num_kv_heads, page_size))


def attention_tcgen05(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                      query_start_loc: torch.Tensor, seq_lens: torch.Tensor, query_lens_host, num_q_heads: int,
                      num_kv_heads: int, head_dim: int, scale: float, window: int = 0) -> None:
    """bfloat16 attention for prompt portions on tcgen05 tensor cores (head size 128, pages of 8, 16, 32, ...
    slots): scores and output accumulate in tensor memory, keys and values come page by page through TMA."""
    T = q.shape[0]
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("attention_tcgen05: bfloat16 only")
    if q.stride(1) != 1 or out.stride(1) != 1 or out.shape != (T, num_q_heads * head_dim) or not cache.is_contiguous():
        raise KernelError("attention_tcgen05: q/out rows must be dense, out [T, nq*d], cache contiguous")
    g = num_q_heads // num_kv_heads
    tiles = sum((n * g + 127) // 128 for n in query_lens_host)
    rc = library().cib_attention_tcgen05(
        _cuda(q, "q", contiguous=False), q.stride(0), _cuda(out, "out", contiguous=False), out.stride(0),
        _cuda(cache, "cache"), cache.shape[0], cache.shape[3], _cuda(block_table, "block_table", torch.int32),
        block_table.stride(0), _cuda(query_start_loc, "query_start_loc", torch.int32),
        _cuda(seq_lens, "seq_lens", torch.int32), len(query_lens_host), tiles, num_q_heads, num_kv_heads, head_dim,
        float(scale), int(window), _error_flag(q.device).data_ptr(), _stream())
    _check(rc, "attention_tcgen05")
    note_flagged_launch()
    _count()


def gemm_wstream_supports(M: int, N: int, K: int) -> bool:
    return bool(library().cib_gemm_wstream_supports(M, N, K))


def gemm_wstream(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, silu_pair: bool = False) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T for up to 128 rows on tcgen05 tensor cores with the weights as the streamed
    128-row operand (bfloat16 in, bfloat16 or float32 out).  ``silu_pair``: w holds N/2 gate rows then N/2 up rows and
    out[M, N/2] = silu(gate) * up (bfloat16)."""
    M, K = a.shape
    N, K2 = w.shape
    out_cols = N // 2 if silu_pair else N
    if K != K2 or out.shape != (M, out_cols) or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_wstream: a {list(a.shape)} {a.dtype}, w {list(w.shape)} {w.dtype}, out {list(out.shape)} do not fit")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1 or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("gemm_wstream: rows must be dense and out bfloat16 or float32")
    if silu_pair and (N % 2 or out.dtype != torch.bfloat16):
        raise KernelError("gemm_wstream: the gated epilogue needs an even N and a bfloat16 result")
    epilogue = 2 if silu_pair else (1 if out.dtype == torch.float32 else 0)
    rc = library().cib_gemm_wstream(
        _cuda(a, "a", contiguous=False), a.stride(0), _cuda(w, "w", contiguous=False), w.stride(0),
        _cuda(out, "out", contiguous=False), out.stride(0), epilogue, M, N, K, 1 if use_pdl else 0,
        _error_flag(a.device).data_ptr(), _stream())
    _check(rc, "gemm_wstream")
    note_flagged_launch()
    _count()


def gemm_tcgen05_supports(M: int, N: int, K: int) -> bool:
    return bool(library().cib_gemm_tcgen05_supports(M, N, K))


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, silu_pair: bool = False) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T on tcgen05 tensor cores (bfloat16 in, bfloat16 or float32 out).
    ``silu_pair``: w holds N/2 gate rows then N/2 up rows and out[M, N/2] = silu(gate) * up (bfloat16)."""
    M, K = a.shape
    N, K2 = w.shape
    out_cols = N // 2 if silu_pair else N
    if K != K2 or out.shape != (M, out_cols) or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_tcgen05: a {list(a.shape)} {a.dtype}, w {list(w.shape)} {w.dtype}, out {list(out.shape)} do not fit")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1 or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("gemm_tcgen05: rows must be dense and out bfloat16 or float32")
    if silu_pair and (N % 2 or out.dtype != torch.bfloat16 or out.stride(0) % 8 or out.data_ptr() % 16):
        raise KernelError("gemm_tcgen05: the gated epilogue needs an even N and 16-byte aligned bfloat16 rows")
    rc = library().cib_gemm_tcgen05(
        _cuda(a, "a", contiguous=False), a.stride(0), _cuda(w, "w", contiguous=False), w.stride(0),
        _cuda(out, "out", contiguous=False), out.stride(0), 1 if out.dtype == torch.float32 else 0,
        1 if silu_pair else 0, M, N, K, _error_flag(a.device).data_ptr(), _stream())
    _check(rc, "gemm_tcgen05")
    note_flagged_launch()
    _count()


# ---- random weights ------------------------------------------------------------------------------------

def fill_random(out: torch.Tensor, key: int, mean: float, std: float, factor: float = 1.0, via_bf16: bool = False) -> None:
    """out.flat[i] = factor * (mean + std * z(key, i)), z approximately standard normal and a function of (key, i)
    alone (``cuinfer_b200.weights.random_init.counter_normal`` computes the same values on the host)."""
    rc = library().cib_fill_random(_cuda(out, "out"), _code(out, "out"), out.numel(), int(key) & 0xFFFFFFFFFFFFFFFF,
                                   float(mean), float(std), float(factor), 1 if via_bf16 else 0, _stream())
    _check(rc, "fill_random")
    _count()


# ---- sampling ----------------------------------------------------------------------------------------

def argmax_rows(logits: torch.Tensor, out_ids: torch.Tensor) -> None:
    """out_ids[s] = index of the largest of logits[s] (float32), ties to the lowest index: greedy sampling of every row."""
    S, V = logits.shape
    if logits.stride(1) != 1 or out_ids.numel() < S:
        raise KernelError("argmax_rows: logits rows must be dense and out_ids hold a row each")
    rc = library().cib_argmax_rows(_cuda(logits, "logits", torch.float32, contiguous=False), logits.stride(0), S, V,
                                   _cuda(out_ids, "out_ids", torch.int32), _stream())
    _check(rc, "argmax_rows")
    _count()


def sample(logits: torch.Tensor, params: torch.Tensor, out_ids: torch.Tensor) -> None:
    """out_ids[s] = token drawn from logits[s]; params[s] = (temperature, top_k as int bits, top_p, u)."""
    S, V = logits.shape
    if logits.stride(1) != 1:
        raise KernelError("sample: logits rows must be dense")
    if params.numel() * params.element_size() < S * 16:
        raise KernelError("sample: params must hold 16 bytes per row")
    rc = library().cib_sample(_cuda(logits, "logits", torch.float32, contiguous=False), logits.stride(0), S, V,
                              _cuda(params, "params"), _cuda(out_ids, "out_ids", torch.int32), _stream())
    _check(rc, "sample")
    _count()
