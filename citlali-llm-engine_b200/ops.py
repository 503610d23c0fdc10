"""Python face of the kernel library: one function per kernel, taking torch tensors.

Each function checks dtypes, shapes and contiguity, then calls the C entry point on the
current CUDA stream.  There is no CPU implementation and no library implementation behind
these functions: if the kernel library cannot be built or loaded, or a tensor is not on a
CUDA device, they raise.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .errors import CitlaliError, require

_F32, _BF16 = 0, 1
_lib = None


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _F32
    if t.dtype == torch.bfloat16:
        return _BF16
    raise CitlaliError(f"kernels take float32 or bfloat16 tensors, not {t.dtype}")


def lib():
    global _lib
    if _lib is None:
        from .csrc.build import load
        l = load()
        l.citlali_last_error.restype = ctypes.c_char_p
        _lib = l
    return _lib


def _ptr(t: Optional[torch.Tensor]):
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current CUDA stream's handle.  Asked for at every launch, so by the quick route where torch has one
    (a step launches a few hundred kernels and the host must not be what a short prompt waits for)."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


_launches = 0
_KERNELS_PER_CALL = {"attention_decode_merged": 2, "argmax_rows_wide": 2}


def launch_count() -> int:
    """Kernels of this library launched so far through this module (a split-K product counts
    its reduction, split-context attention its merge)."""
    return _launches


def _check(code: int, what: str):
    global _launches
    if code == 0:
        _launches += _KERNELS_PER_CALL.get(what, 1)
        return
    if code < 0:
        raise CitlaliError(f"{what} refused: {lib().citlali_last_error().decode()}")
    raise CitlaliError(f"{what}: CUDA error {code} at launch")


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not (t.is_cuda and t.is_contiguous()):
            require(t.is_cuda, "kernels run on a CUDA device only; a tensor on the CPU was given")
            require(False, "kernels take contiguous tensors")


_i = ctypes.c_int
_f = ctypes.c_float


def embed_rows(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, error_flag: torch.Tensor,
               scale: float = 1.0):
    _need_cuda(table, tokens, out, error_flag)
    require(tokens.dtype == torch.int32 and out.dtype == torch.float32, "embed_rows: tokens int32, out float32")
    rows, hidden = out.shape
    require(table.shape[1] == hidden and tokens.numel() == rows, "embed_rows: shapes do not fit")
    _check(lib().citlali_embed_rows(_ptr(table), _i(_dtype_code(table)), _ptr(tokens), _ptr(out), _i(rows),
                                    _i(hidden), _i(table.shape[0]), _f(scale), _ptr(error_flag), _stream()), "embed_rows")


def embed_rows_streams(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, error_flag: torch.Tensor,
                       scale: float = 1.0):
    """``out[s] = table[tokens] * scale`` for every stream s of ``out`` [streams, rows, hidden], in one launch."""
    _need_cuda(table, tokens, out, error_flag)
    require(tokens.dtype == torch.int32 and out.dtype == torch.float32 and out.dim() == 3,
            "embed_rows_streams: tokens int32, out float32 [streams, rows, hidden]")
    streams, rows, hidden = out.shape
    require(table.shape[1] == hidden and tokens.numel() == rows, "embed_rows_streams: shapes do not fit")
    _check(lib().citlali_embed_rows_copies(_ptr(table), _i(_dtype_code(table)), _ptr(tokens), _ptr(out), _i(rows),
                                           _i(hidden), _i(table.shape[0]), _f(scale), _ptr(error_flag), _i(streams),
                                           ctypes.c_size_t(rows * hidden), _stream()), "embed_rows")


def scale_(x: torch.Tensor, scale: float):
    """x *= scale in place (float32)."""
    _need_cuda(x)
    require(x.dtype == torch.float32, "scale_: float32 only")
    _check(lib().citlali_scale(_ptr(x), ctypes.c_size_t(x.numel()), _f(scale), _stream()), "scale")


def soft_cap_(x: torch.Tensor, cap: float):
    """x = cap tanh(x / cap) in place (float32)."""
    _need_cuda(x)
    require(x.dtype == torch.float32 and cap > 0.0, "soft_cap_: float32 only, with a positive cap")
    _check(lib().citlali_soft_cap(_ptr(x), ctypes.c_size_t(x.numel()), _f(cap), _stream()), "soft_cap")


def concat_rows(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor):
    """``out[r] = [a[r] | b[r]]`` for two float32 matrices of one shape, rounded once to ``out``'s dtype."""
    _need_cuda(a, b, out)
    rows, width = a.shape
    require(a.dtype == torch.float32 and b.dtype == torch.float32 and b.shape == a.shape and out.shape == (rows, 2 * width),
            "concat_rows: two float32 matrices of one shape and an output twice as wide")
    _check(lib().citlali_concat_rows(_ptr(a), _ptr(b), _ptr(out), _i(_dtype_code(out)), _i(rows), _i(width), _stream()),
           "concat_rows")


def rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor,
             row_index: Optional[torch.Tensor] = None):
    _need_cuda(x, gain, out, row_index)
    require(x.dtype == torch.float32, "rms_norm: the input rows are float32")
    rows, hidden = out.shape
    require(x.shape[1] == hidden and gain.numel() == hidden, "rms_norm: shapes do not fit")
    if row_index is not None:
        require(row_index.dtype == torch.int32 and row_index.numel() == rows, "rms_norm: bad row index")
    else:
        require(x.shape[0] == rows, "rms_norm: shapes do not fit")
    _check(lib().citlali_rms_norm(_ptr(x), _ptr(gain), _i(_dtype_code(gain)), _ptr(row_index), _ptr(out),
                                  _i(_dtype_code(out)), _i(rows), _i(hidden), _f(eps), _stream()), "rms_norm")


def swiglu(gate_up: torch.Tensor, act: torch.Tensor, run: int):
    _need_cuda(gate_up, act)
    rows, inter = act.shape
    require(gate_up.shape == (rows, 2 * inter) and gate_up.dtype == act.dtype, "swiglu: shapes or dtypes do not fit")
    _check(lib().citlali_swiglu(_ptr(gate_up), _ptr(act), _i(_dtype_code(act)), _i(rows), _i(inter), _i(run),
                                _stream()), "swiglu")


def gemm_simt(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, accumulate: bool = False):
    _need_cuda(x, w, y)
    M, K = x.shape
    N = w.shape[0]
    require(w.shape[1] == K and y.shape == (M, N), "gemm_simt: shapes do not fit")
    _check(lib().citlali_gemm_simt(_ptr(x), _i(_dtype_code(x)), _ptr(w), _i(_dtype_code(w)), _ptr(y),
                                   _i(_dtype_code(y)), _i(M), _i(N), _i(K), _i(1 if accumulate else 0), _stream()),
           "gemm_simt")


def qk_norm_rope_cache(qkv, q_gain, k_gain, inv_freq, rotary_dim, row_slot, row_pos, page_table,
                       k_pool, v_pool, page_size, nq, nkv, head_dim, eps, write_cache=True):
    """Head RMSNorm of q and k (``q_gain``/``k_gain`` None: none), rotation of the first ``rotary_dim`` elements
    of each q and k head in pairs (i, i + rotary_dim/2), and the cache write, in one pass over the projection's
    rows.  ``write_cache``: True keys and values go to the cache; False nothing does; ``"keys_in_place"`` the
    normed, rotated keys go back into the row and the values stay, for a position encoding that works on the
    row before a second call stores it."""
    _need_cuda(qkv, q_gain, k_gain, inv_freq, row_slot, row_pos, page_table, k_pool, v_pool)
    rows = qkv.shape[0]
    require(qkv.shape[1] == (nq + 2 * nkv) * head_dim, "qk_norm_rope_cache: the projection's width does not fit")
    require(inv_freq.dtype == torch.float32 and inv_freq.numel() == rotary_dim // 2,
            "qk_norm_rope_cache: bad frequency table")
    require(row_slot.dtype == torch.int32 and row_pos.dtype == torch.int32 and page_table.dtype == torch.int32,
            "qk_norm_rope_cache: index tensors are int32")
    gain_code = _dtype_code(q_gain) if q_gain is not None else _F32
    if q_gain is not None and k_gain is not None:
        require(q_gain.dtype == k_gain.dtype, "qk_norm_rope_cache: q and k gains differ in dtype")
    cache_code = _dtype_code(k_pool) if k_pool is not None else _dtype_code(qkv)
    _check(lib().citlali_qk_norm_rope_cache(
        _ptr(qkv), _i(_dtype_code(qkv)), _ptr(q_gain), _ptr(k_gain), _i(gain_code), _ptr(inv_freq), _i(rotary_dim),
        _ptr(row_slot), _ptr(row_pos), _ptr(page_table), _i(page_table.shape[1]), _ptr(k_pool), _ptr(v_pool),
        _i(cache_code), _i(page_size), _i(rows), _i(nq), _i(nkv), _i(head_dim), _f(eps),
        _i(2 if write_cache == "keys_in_place" else (1 if write_cache else 0)), _stream()), "qk_norm_rope_cache")


def attention_rows(q, q_stride, k_pool, v_pool, page_table, row_slot, row_pos, out, nq, nkv, head_dim,
                   page_size, window, max_keys, scale):
    _need_cuda(k_pool, v_pool, page_table, row_slot, row_pos, out)
    require(q.is_cuda, "kernels run on a CUDA device only")
    rows = out.shape[0]
    _check(lib().citlali_attention_rows(
        _ptr(q), _i(q_stride), _i(_dtype_code(q)), _ptr(k_pool), _ptr(v_pool), _i(_dtype_code(k_pool)),
        _ptr(page_table), _i(page_table.shape[1]), _ptr(row_slot), _ptr(row_pos), _ptr(out), _i(out.shape[1]),
        _i(rows), _i(nq), _i(nkv), _i(head_dim), _i(page_size), _i(window or 0), _i(max_keys), _f(scale),
        _stream()), "attention_rows")


def argmax_rows(logits: torch.Tensor, tokens: torch.Tensor):
    _need_cuda(logits, tokens)
    require(logits.dtype == torch.float32 and tokens.dtype == torch.int32, "argmax_rows: float32 in, int32 out")
    rows, vocab = logits.shape
    if vocab >= 8192:
        scratch = _scratch(logits.device, "argmax segments", rows * 128 * 4)
        _check(lib().citlali_argmax_rows_wide(_ptr(logits), _ptr(tokens), _ptr(scratch), _i(rows), _i(vocab), _stream()),
               "argmax_rows_wide")
        return
    _check(lib().citlali_argmax_rows(_ptr(logits), _ptr(tokens), _i(rows), _i(vocab), _stream()), "argmax_rows")


def sample_rows(logits, temperature, uniform, tokens):
    _need_cuda(logits, temperature, uniform, tokens)
    require(logits.dtype == torch.float32 and tokens.dtype == torch.int32 and temperature.dtype == torch.float32
            and uniform.dtype == torch.float32, "sample_rows: float32 in, int32 out")
    rows, vocab = logits.shape
    require(temperature.numel() >= rows and uniform.numel() >= rows and tokens.numel() >= rows,
            "sample_rows: per-row tensors are too short")
    _check(lib().citlali_sample_rows(_ptr(logits), _ptr(temperature), _ptr(uniform), _ptr(tokens), _i(rows),
                                     _i(vocab), _stream()), "sample_rows")


# ---- choices between kernels ---------------------------------------------------------------

def attention_steps_from_device(dtype, head_dim: int) -> bool:
    """Whether a step of single tokens in this dtype and head size runs the split-context kernel, whose
    launch depends on no host-side length (the condition :func:`attention` tests first)."""
    return dtype == torch.bfloat16 and head_dim % 8 == 0 and head_dim <= 256


def attention(q, q_stride, cache_view, batch, out, nq, nkv, head_dim, window, scale):
    """Attention of every row of the step over its slot's cache.  ``q`` holds the rotated
    queries with ``q_stride`` elements between rows.  bfloat16 steps in which every sequence
    brings one token run the split-context kernel, whose launch does not depend on the
    sequences' lengths; everything else runs the generic kernel."""
    if batch.is_decode and attention_steps_from_device(q.dtype, head_dim):
        attention_decode(q, q_stride, cache_view.keys, cache_view.values, cache_view.page_table, batch.row_slot,
                         batch.row_pos, out, nq, nkv, head_dim, cache_view.page_size, window,
                         cache_view.page_table.shape[1] * cache_view.page_size, scale)
        return
    require(not torch.cuda.is_current_stream_capturing(),
            "attention: this dtype and head size run a kernel whose launch is sized from the host's lists of lengths, "
            "which a captured step would freeze; such a model steps without CUDA graphs")
    if (q.dtype == torch.bfloat16 and q_stride % 8 == 0 and out.shape[1] % 8 == 0 and batch.max_new >= 48
            and lib().citlali_attention_prefill_tc_supports(_i(head_dim), _i(cache_view.page_size))):
        attention_prefill_tc(q, q_stride, cache_view.keys, cache_view.values, cache_view.page_table, batch.seq_start,
                             batch.seq_slot, batch.seq_past, out, batch.sequences, batch.max_new, nq, nkv, head_dim,
                             cache_view.page_size, window, scale)
        return
    if (q.dtype == torch.bfloat16 and q_stride % 8 == 0
            and lib().citlali_attention_prefill_supports(_i(head_dim), _i(cache_view.page_size))):
        attention_prefill(q, q_stride, cache_view.keys, cache_view.values, cache_view.page_table, batch.seq_start,
                          batch.seq_slot, batch.seq_past, out, batch.sequences, batch.max_new, nq, nkv, head_dim,
                          cache_view.page_size, window, scale)
        return
    attention_rows(q, q_stride, cache_view.keys, cache_view.values, cache_view.page_table,
                   batch.row_slot, batch.row_pos, out, nq, nkv, head_dim, cache_view.page_size,
                   window, batch.max_keys, scale)


def attention_prefill(q, q_stride, k_pool, v_pool, page_table, seq_start, seq_slot, seq_past, out, sequences, max_new,
                      nq, nkv, head_dim, page_size, window, scale, keep_first=0, softcap=0.0, gate=None):
    """``softcap`` c > 0: scaled scores become c tanh(s / c).  ``gate``: float32 [rows, heads * head size] (rows may be
    further apart than they are long), the output is multiplied by its sigmoids."""
    _need_cuda(k_pool, v_pool, page_table, seq_start, seq_slot, seq_past, out)
    require(q.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
            "attention_prefill: bfloat16 only")
    require(gate is None or (gate.is_cuda and gate.dtype == torch.float32 and gate.stride(1) == 1
                             and gate.shape == (out.shape[0], nq * head_dim)), "attention_prefill: the gate does not fit")
    _check(lib().citlali_attention_prefill(
        _ptr(q), _i(q_stride), _ptr(k_pool), _ptr(v_pool), _ptr(page_table), _i(page_table.shape[1]),
        _ptr(seq_start), _ptr(seq_slot), _ptr(seq_past), _ptr(out), _i(out.shape[1]), _i(sequences), _i(max_new),
        _i(nq), _i(nkv), _i(head_dim), _i(page_size), _i(window or 0), _i(keep_first or 0), _f(scale),
        _f(float(softcap or 0.0)), _ptr(gate), _sz(gate.stride(0) if gate is not None else 0), _stream()),
        "attention_prefill")


def attention_prefill_tc(q, q_stride, k_pool, v_pool, page_table, seq_start, seq_slot, seq_past, out, sequences, max_new,
                         nq, nkv, head_dim, page_size, window, scale, error_flag=None):
    """Prompt attention on tcgen05 (head size 128, pages of 64)."""
    _need_cuda(k_pool, v_pool, page_table, seq_start, seq_slot, seq_past, out, error_flag)
    require(q.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
            "attention_prefill_tc: bfloat16 only")
    _check(lib().citlali_attention_prefill_tc(
        _ptr(q), _i(q_stride), _i(q.shape[0]), _ptr(k_pool), _ptr(v_pool), _i(k_pool.shape[0]), _ptr(page_table),
        _i(page_table.shape[1]), _ptr(seq_start), _ptr(seq_slot), _ptr(seq_past), _ptr(out), _i(out.shape[1]),
        _i(sequences), _i(max_new), _i(nq), _i(nkv), _i(head_dim), _i(page_size), _i(window or 0), _f(scale),
        _ptr(error_flag), _stream()), "attention_prefill_tc")


def attention_decode(q, q_stride, k_pool, v_pool, page_table, row_slot, row_pos, out, nq, nkv, head_dim,
                     page_size, window, max_positions, scale):
    _need_cuda(k_pool, v_pool, page_table, row_slot, row_pos, out)
    require(q.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
            "attention_decode: bfloat16 only")
    rows = out.shape[0]
    l = lib()
    l.citlali_attention_decode_scratch_floats.restype = ctypes.c_size_t
    need = l.citlali_attention_decode_scratch_floats(_i(rows), _i(nq), _i(head_dim), _i(page_size), _i(max_positions))
    ws = _scratch(q.device, "attention_decode", need * 4)
    counters = _scratch(q.device, "attention_decode counters", rows * nq * 4, zeroed=True)
    _check(l.citlali_attention_decode(
        _ptr(q), _i(q_stride), _ptr(k_pool), _ptr(v_pool), _ptr(page_table), _i(page_table.shape[1]),
        _ptr(row_slot), _ptr(row_pos), _ptr(out), _i(out.shape[1]), _ptr(ws), ctypes.c_size_t(ws.numel() // 4),
        _ptr(counters), ctypes.c_size_t(counters.numel() // 4),
        _i(rows), _i(nq), _i(nkv), _i(head_dim), _i(page_size), _i(window or 0), _i(max_positions), _f(scale),
        _stream()),
        # one kernel whose blocks merge through distributed shared memory, or a partial and a merge kernel
        "attention_decode" if (page_size == 64 and q_stride % 8 == 0 and q.data_ptr() % 16 == 0
                               and head_dim in (16, 32, 48, 64, 80, 96, 112, 128, 256)) else "attention_decode_merged")


_sm_count = {}
_workspace = {}
_retired = []


def sm_count(device) -> int:
    idx = (device.index if isinstance(device, torch.device) else torch.device(device).index) or 0
    n = _sm_count.get(idx)
    if n is None:
        n = _sm_count[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return n


def gemm_tc_plan(M: int, N: int, K: int, device, force_splits: int = 0) -> dict:
    """How the tensor-core product of this shape runs."""
    swapped, bn, splits = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    lib().citlali_gemm_tc_plan(_i(M), _i(N), _i(K), _i(sm_count(device)), _i(force_splits), ctypes.byref(swapped),
                               ctypes.byref(bn), ctypes.byref(splits))
    return {"swapped": bool(swapped.value), "bn": bn.value, "splits": splits.value}


def wait_selftest(error_flag: torch.Tensor, limit_ms: float = 2.0):
    """Run the tensor-core kernels' bounded wait on a barrier nothing arrives on; it gives up after
    ``limit_ms``.  Returns (the wait's return value, the block's abort word); ``error_flag[1..2]`` hold
    code 900 and the block."""
    _need_cuda(error_flag)
    result = torch.full((2,), -1, dtype=torch.int32, device=error_flag.device)
    _check(lib().citlali_wait_selftest(_ptr(error_flag), _ptr(result), ctypes.c_longlong(int(limit_ms * 1e6)), _stream()),
           "wait_selftest")
    ok, abort = result.tolist()
    return ok, abort


def gemm_tc_pair_plan(M: int, N: int, K: int) -> dict:
    """The pair kernel's tile width for this shape and how many clusters of two the device runs at once."""
    bn, pairs = ctypes.c_int(), ctypes.c_int()
    lib().citlali_gemm_tc_pair_plan(_i(M), _i(N), _i(K), ctypes.byref(bn), ctypes.byref(pairs))
    return {"bn": bn.value, "pairs": pairs.value}


def gemm_tc_set_pair_rows(rows: int) -> int:
    """From ``rows`` rows of ``x`` on, ``gemm_tc`` runs on pairs of SMs where their waves cost less
    (0: never). Returns the number that stood before."""
    return int(lib().citlali_gemm_tc_set_pair_rows(_i(rows)))


def gemm_tc_runs_on_pairs(M: int, N: int, K: int, device, swiglu: bool = False) -> bool:
    """Whether ``gemm_tc`` gives a product of this shape to the pair kernel."""
    return bool(lib().citlali_gemm_tc_runs_on_pairs(_i(M), _i(N), _i(K), _i(sm_count(device)), _i(1 if swiglu else 0)))


def gemm_tc_pair(x, w, y, accumulate=False, error_flag=None, swiglu=False):
    """``gemm_tc`` on pairs of SMs (tcgen05.mma with cta_group::2), whatever the number of rows."""
    _need_cuda(x, w, y, error_flag)
    M, K = x.shape
    N = w.shape[0]
    require(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0 and w.shape[1] == K
            and x.is_contiguous() and w.is_contiguous(),
            "gemm_tc_pair: operands must be contiguous bfloat16 with an inner size that is a multiple of 8")
    require(y.shape == (M, N // 2 if swiglu else N), "gemm_tc_pair: the output's shape does not fit")
    mode = (1 if accumulate else 0) | (2 if swiglu else 0)
    _check(lib().citlali_gemm_tc_pair(_ptr(x), _ptr(w), _ptr(y), _i(_dtype_code(y)), _i(M), _i(N), _i(K), _i(mode),
                                      _ptr(error_flag), _stream()), "gemm_tc_pair")


_zeroed_purposes = set()


def zero_counters() -> None:
    """Put the scratch buffers that hold counters back to zero, in place (captured graphs keep their addresses).  For
    after a kernel reported a fault: a step that gave up half-way may have left counters standing."""
    for (index, purpose), ws in _workspace.items():
        if purpose in _zeroed_purposes:
            ws.zero_()
    for purpose, ws in _retired:
        if purpose in _zeroed_purposes:
            ws.zero_()


def _scratch(device, purpose: str, nbytes: int, zeroed: bool = False) -> torch.Tensor:
    """One scratch buffer per device and purpose (split-context attention partials, argmax segments);
    it only grows.  Kernels on one stream use it one after another.  ``zeroed``: filled with zeros when it
    is made (for counters that every kernel leaves at zero)."""
    key = (torch.device(device).index or 0, purpose)
    ws = _workspace.get(key)
    if ws is None or ws.numel() < nbytes:
        require(not torch.cuda.is_current_stream_capturing(),
                f"the {purpose} scratch buffer would have to grow during graph capture; run the step once before capturing")
        if ws is not None:
            _retired.append((purpose, ws))          # a captured graph may still hold its address: it is kept, not freed
        ws = (torch.zeros if zeroed else torch.empty)(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspace[key] = ws
        if zeroed:
            _zeroed_purposes.add(purpose)
    return ws


def gemm_tc_accepts(x, w, y) -> bool:
    """The tensor-core product's shape rules: bfloat16 operands, an inner size that is a
    multiple of 8 (TMA needs rows of 16-byte multiples), 16-byte aligned starts."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and y.dtype in (torch.float32, torch.bfloat16)
            and x.shape[1] % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and x.is_contiguous() and w.is_contiguous() and y.is_contiguous())


def norm_inputs(x: torch.Tensor, rows_out: torch.Tensor, sumsq: torch.Tensor):
    """``rows_out = bfloat16(x)`` and ``sumsq[r, g]`` = the sum of squares of x[r]'s g-th group of 32 features."""
    _need_cuda(x, rows_out, sumsq)
    rows, hidden = x.shape
    require(x.dtype == torch.float32 and rows_out.dtype == torch.bfloat16 and sumsq.dtype == torch.float32
            and rows_out.shape == x.shape and sumsq.shape == (rows, hidden // 32), "norm_inputs: shapes or dtypes do not fit")
    _check(lib().citlali_norm_inputs(_ptr(x), _ptr(rows_out), _ptr(sumsq), _i(rows), _i(hidden), _stream()), "norm_inputs")


def gemm_tc_is_small_form(M: int, N: int, K: int, device) -> bool:
    """Whether the product of this shape runs the form for few rows of x, whose epilogue can do a norm's work."""
    return gemm_tc_plan(M, N, K, device)["swapped"]


def gemm_tc(x, w, y, accumulate=False, error_flag=None, swiglu=False, force_splits=0, emit=None, row_scale=None):
    """``y = x . w^T`` on the tensor cores.  ``accumulate``: ``y`` (float32) ``+=``.  ``swiglu``: ``w``'s
    rows alternate gate/up in runs of 16 and ``y`` is bfloat16 ``[M, N/2] = silu(gate) * up``.
    Few rows of x only: ``emit = (rows_bf16 [M, N], sumsq [M, N/32])`` (with ``accumulate``) also writes the updated
    rows as bfloat16 and the sums of their squares over groups of 32 features; ``row_scale = (sumsq [M, groups], dim,
    eps)`` multiplies result row m by ``rsqrt(sum(sumsq[m]) / dim + eps)``."""
    _need_cuda(x, w, y, error_flag)
    M, K = x.shape
    N = w.shape[0]
    require(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0 and w.shape[1] == K
            and x.is_contiguous() and w.is_contiguous(),
            "gemm_tc: operands must be contiguous bfloat16 with an inner size that is a multiple of 8")
    require(y.shape == (M, N // 2 if swiglu else N), "gemm_tc: the output's shape does not fit")
    mode = (1 if accumulate else 0) | (2 if swiglu else 0)
    if emit is None and row_scale is None:
        _check(lib().citlali_gemm_tc(_ptr(x), _ptr(w), _ptr(y), _i(_dtype_code(y)), _i(M), _i(N), _i(K), _i(mode),
                                     _i(force_splits), _ptr(error_flag), _i(sm_count(x.device)), _stream()), "gemm_tc")
        return
    emit_rows = emit_sumsq = scale_sumsq = None
    groups = dim = 0
    eps = 0.0
    if emit is not None:
        emit_rows, emit_sumsq = emit
        _need_cuda(emit_rows, emit_sumsq)
        require(emit_rows.dtype == torch.bfloat16 and emit_rows.shape == (M, N) and emit_sumsq.dtype == torch.float32
                and emit_sumsq.shape == (M, N // 32), "gemm_tc: the emitted rows or their sums have the wrong shape or dtype")
    if row_scale is not None:
        scale_sumsq, dim, eps = row_scale
        _need_cuda(scale_sumsq)
        require(scale_sumsq.dtype == torch.float32 and scale_sumsq.dim() == 2 and scale_sumsq.shape[0] == M,
                "gemm_tc: the sums of squares to scale by have the wrong shape or dtype")
        groups = scale_sumsq.shape[1]
    _check(lib().citlali_gemm_tc_normed(_ptr(x), _ptr(w), _ptr(y), _i(_dtype_code(y)), _i(M), _i(N), _i(K), _i(mode),
                                        _i(force_splits), _ptr(error_flag), _i(sm_count(x.device)), _ptr(emit_rows),
                                        _ptr(emit_sumsq), _ptr(scale_sumsq), _i(groups), _i(int(dim)), _f(float(eps)), _stream()),
           "gemm_tc")


# ---- residual streams --------------------------------------------------------------------------

_sz = ctypes.c_size_t


def hyper_read_norm(X: torch.Tensor, w_in: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor):
    """``out = rms_norm(sum_s w_in[s] X[s]) * gain``; X float32 [streams, rows, width], gain float32."""
    _need_cuda(X, w_in, gain, out)
    S, rows, width = X.shape
    require(X.dtype == torch.float32 and w_in.dtype == torch.float32 and gain.dtype == torch.float32
            and w_in.numel() == S and gain.numel() == width and out.shape == (rows, width),
            "hyper_read_norm: shapes or dtypes do not fit")
    _check(lib().citlali_hyper_read_norm(_ptr(X), _sz(rows * width), _i(S), _ptr(w_in), _ptr(gain), _ptr(out),
                                         _i(_dtype_code(out)), _i(rows), _i(width), _f(eps), _stream()), "hyper_read_norm")


def hyper_write(X: torch.Tensor, y: torch.Tensor, w_mix: torch.Tensor, w_out: torch.Tensor):
    """``X[t] <- sum_s w_mix[s, t] X[s] + w_out[t] y`` in place, every stream from the old ones."""
    _need_cuda(X, y, w_mix, w_out)
    S, rows, width = X.shape
    require(X.dtype == torch.float32 and y.dtype == torch.float32 and y.shape == (rows, width)
            and w_mix.dtype == torch.float32 and w_mix.shape == (S, S) and w_out.dtype == torch.float32
            and w_out.numel() == S, "hyper_write: shapes or dtypes do not fit")
    _check(lib().citlali_hyper_write(_ptr(X), _sz(rows * width), _i(S), _ptr(y), _ptr(w_mix), _ptr(w_out),
                                     _sz(rows * width), _stream()), "hyper_write")


def hyper_write_read_norm(X, y, w_mix, w_out, w_in, gain, eps, out):
    """:func:`hyper_write` of one sub-layer and :func:`hyper_read_norm` of the next in one pass over the streams."""
    _need_cuda(X, y, w_mix, w_out, w_in, gain, out)
    S, rows, width = X.shape
    require(X.dtype == torch.float32 and y.dtype == torch.float32 and y.shape == (rows, width)
            and w_mix.dtype == torch.float32 and w_mix.shape == (S, S) and w_out.dtype == torch.float32 and w_out.numel() == S
            and w_in.dtype == torch.float32 and w_in.numel() == S and gain.dtype == torch.float32 and gain.numel() == width
            and out.shape == (rows, width), "hyper_write_read_norm: shapes or dtypes do not fit")
    _check(lib().citlali_hyper_write_read_norm(_ptr(X), _sz(rows * width), _i(S), _ptr(y), _ptr(w_mix), _ptr(w_out),
                                               _ptr(w_in), _ptr(gain), _ptr(out), _i(_dtype_code(out)), _i(rows),
                                               _i(width), _f(eps), _stream()), "hyper_write_read_norm")


def stream_sum(X: torch.Tensor, out: torch.Tensor, row_index: Optional[torch.Tensor] = None):
    """``out[i] = sum_s X[s, row_index[i]]``."""
    _need_cuda(X, out, row_index)
    S, rows, width = X.shape
    require(X.dtype == torch.float32 and out.dtype == torch.float32 and out.shape[1] == width
            and (row_index is None or (row_index.dtype == torch.int32 and row_index.numel() == out.shape[0])),
            "stream_sum: shapes or dtypes do not fit")
    _check(lib().citlali_stream_sum(_ptr(X), _sz(rows * width), _i(S), _ptr(row_index), _ptr(out), _i(out.shape[0]),
                                    _i(width), _stream()), "stream_sum")


def relu_squared(x: torch.Tensor, y: torch.Tensor):
    _need_cuda(x, y)
    require(x.dtype == y.dtype and x.shape == y.shape, "relu_squared: shapes or dtypes do not fit")
    _check(lib().citlali_relu_squared(_ptr(x), _ptr(y), _i(_dtype_code(x)), _sz(x.numel()), _stream()), "relu_squared")


# ---- the gated delta rule ------------------------------------------------------------------------

def delta_prepare(proj, taps_w, state, conv_off, row_slot, seq_start, seq_slot, sequences, a_log, dt_bias, prep,
                  H, KH, D, V, unit_eps, block_a_segment=False, beta_col=None, decay_col=None, decay_in=None,
                  channel_decay=False):
    """See ``citlali_delta_prepare`` (csrc/api.h).  ``state`` [slots, n] float32; two launches unless taps == 1.
    ``beta_col`` / ``decay_col``: the columns of b and a in a row of ``proj`` (default: behind q, k, v and a gate of H V
    columns).  ``decay_in``: the decays' inputs in a tensor of their own (a view whose rows may be further apart than its
    width).  ``channel_decay``: a decay per head and key channel, ``prep`` is then [rows, C + H + H D]."""
    _need_cuda(proj, taps_w, state, row_slot, seq_start, seq_slot, a_log, dt_bias, prep)
    rows = proj.shape[0]
    C = 2 * KH * D + H * V
    taps = taps_w.shape[1]
    GD = D if channel_decay else 1
    beta_col = C + H * V if beta_col is None else int(beta_col)
    decay_col = beta_col + H if decay_col is None else int(decay_col)
    require(proj.dtype == torch.float32 and prep.dtype == torch.float32 and state.dtype == torch.float32
            and taps_w.dtype == torch.float32 and a_log.dtype == torch.float32 and dt_bias.dtype == torch.float32,
            "delta_prepare: float32 tensors only")
    require(proj.shape[1] >= beta_col + H and (decay_in is not None or proj.shape[1] >= decay_col + H)
            and prep.shape == (rows, C + H + H * GD) and taps_w.shape[0] == C and dt_bias.numel() == H * GD
            and state.dim() == 2 and state.shape[1] >= conv_off + (taps - 1) * C, "delta_prepare: shapes do not fit")
    require(not channel_decay or decay_in is not None, "delta_prepare: a decay per channel needs decay_in")
    decay_stride = 0
    if decay_in is not None:
        require(decay_in.is_cuda and decay_in.dtype == torch.float32 and decay_in.shape == (rows, H * GD)
                and decay_in.stride(1) == 1, "delta_prepare: the decays' inputs do not fit")
        decay_stride = decay_in.stride(0)
    _check(lib().citlali_delta_prepare(_ptr(proj), _i(proj.shape[1]), _ptr(taps_w), _i(taps), _ptr(state),
                                       _sz(state.shape[1]), _sz(conv_off), _ptr(row_slot), _ptr(seq_start), _ptr(seq_slot),
                                       _i(sequences), _ptr(a_log), _ptr(dt_bias), _ptr(prep), _i(rows), _i(H), _i(KH),
                                       _i(D), _i(V), _f(unit_eps), _i(1 if block_a_segment else 0), _i(beta_col),
                                       _i(decay_col), _ptr(decay_in), _i(decay_stride), _i(1 if channel_decay else 0),
                                       _stream()),
           "delta_prepare" if taps == 1 else "delta_prepare_kept")


_KERNELS_PER_CALL["delta_prepare_kept"] = 2

DELTA_HEAD_DECAY, DELTA_CHANNEL_DECAY, DELTA_NO_CORRECTION = 0, 1, 2


def delta_rule(prep, state, seq_start, seq_slot, sequences, H, KH, D, V, out, pairs=False, mode=DELTA_HEAD_DECAY):
    """``mode``: one decay a head; a decay a key channel; or no correction term (u = beta v: a state-space recurrence)."""
    _need_cuda(prep, state, seq_start, seq_slot, out)
    require(prep.dtype == torch.float32 and state.dtype == torch.float32 and out.dtype == torch.float32
            and out.shape == (prep.shape[0], H * V) and state.shape[1] >= H * D * V, "delta_rule: shapes or dtypes do not fit")
    require(prep.shape[1] == 2 * KH * D + H * V + H + H * (D if mode == DELTA_CHANNEL_DECAY else 1),
            "delta_rule: the prepared rows' width does not fit the form")
    _check(lib().citlali_delta_rule(_ptr(prep), _i(prep.shape[1]), _ptr(state), _sz(state.shape[1]), _ptr(seq_start),
                                    _ptr(seq_slot), _i(sequences), _i(H), _i(KH), _i(D), _i(V), _ptr(out),
                                    _i(1 if pairs else 0), _i(mode), _stream()), "delta_rule")


def delta_output(o, gate, gate_stride, weight, y, H, V, eps, gate_act="silu"):
    """``gate``: a view into rows that starts at the gate's first column; ``gate_act``: "silu" or "sigmoid"."""
    _need_cuda(o, weight, y)
    require(gate.is_cuda and o.dtype == torch.float32 and gate.dtype == torch.float32 and weight.dtype == torch.float32
            and weight.numel() == V and y.shape == o.shape and gate_act in ("silu", "sigmoid"),
            "delta_output: shapes or dtypes do not fit")
    _check(lib().citlali_delta_output(_ptr(o), _ptr(gate), _i(gate_stride), _ptr(weight), _ptr(y), _i(_dtype_code(y)),
                                      _i(o.shape[0]), _i(H), _i(V), _f(eps), _i(1 if gate_act == "sigmoid" else 0), _stream()),
           "delta_output")


# ---- a norm on a sub-layer's output ---------------------------------------------------------------------

def layer_norm_add(y, gain, eps, x, emit=None):
    """``x += layer_norm(y) * gain`` (float32); ``emit`` receives the updated rows in its own dtype."""
    _need_cuda(y, gain, x, emit)
    rows, hidden = x.shape
    require(y.dtype == torch.float32 and x.dtype == torch.float32 and y.shape == x.shape and gain.numel() == hidden
            and (emit is None or emit.shape == x.shape), "layer_norm_add: shapes or dtypes do not fit")
    _check(lib().citlali_layer_norm_add(_ptr(y), _ptr(gain), _i(_dtype_code(gain)), _ptr(x), _ptr(emit),
                                        _i(_dtype_code(emit) if emit is not None else _F32), _i(rows), _i(hidden), _f(eps),
                                        _stream()), "layer_norm_add")


def layer_norm_rows(x, gain, eps, out, row_index=None, bias=None):
    """``out = layer_norm(x[row_index]) * gain + bias`` (``bias``, of the gain's dtype, may be None)."""
    _need_cuda(x, gain, out, row_index, bias)
    rows, hidden = out.shape
    require(x.dtype == torch.float32 and x.shape[1] == hidden and gain.numel() == hidden
            and (row_index is not None or x.shape[0] == rows)
            and (row_index is None or (row_index.dtype == torch.int32 and row_index.numel() == rows))
            and (bias is None or (bias.numel() == hidden and bias.dtype == gain.dtype)),
            "layer_norm_rows: shapes or dtypes do not fit")
    _check(lib().citlali_layer_norm_rows(_ptr(x), _ptr(gain), _ptr(bias), _i(_dtype_code(gain)), _ptr(row_index), _ptr(out),
                                         _i(_dtype_code(out)), _i(rows), _i(hidden), _f(eps), _stream()), "layer_norm_rows")


def layer_norm_chain(y, x, gain, bias, eps, in_bias=None, emit=None, next_gain=None, next_bias=None, next_eps=0.0,
                     next_out=None):
    """``x += layer_norm(y + in_bias) * gain + bias``; ``emit`` receives the updated rows; with ``next_gain`` also
    ``next_out = layer_norm(x) * next_gain + next_bias``.  y, x and all gains and biases are float32; ``emit`` and
    ``next_out`` share a dtype."""
    _need_cuda(y, x, gain, bias, in_bias, emit, next_gain, next_bias, next_out)
    rows, hidden = x.shape
    vectors = [v for v in (gain, bias, in_bias, next_gain, next_bias) if v is not None]
    outs = [o for o in (emit, next_out) if o is not None]
    require(y.dtype == torch.float32 and x.dtype == torch.float32 and y.shape == x.shape
            and all(v.dtype == torch.float32 and v.numel() == hidden for v in vectors)
            and all(o.shape == x.shape and o.dtype == outs[0].dtype for o in outs)
            and (next_gain is None) == (next_out is None), "layer_norm_chain: shapes or dtypes do not fit")
    _check(lib().citlali_layer_norm_chain(_ptr(y), _ptr(in_bias), _ptr(gain), _ptr(bias), _ptr(x), _ptr(emit), _ptr(next_gain),
                                          _ptr(next_bias), _ptr(next_out), _i(_dtype_code(outs[0]) if outs else _F32),
                                          _i(rows), _i(hidden), _f(eps), _f(next_eps), _stream()), "layer_norm_chain")


def cast_rows(x, out):
    _need_cuda(x, out)
    require(x.dtype == torch.float32 and x.shape == out.shape, "cast_rows: a float32 tensor and one of its shape")
    _check(lib().citlali_cast_rows(_ptr(x), _ptr(out), _i(_dtype_code(out)), _sz(x.numel()), _stream()), "cast_rows")


def scaled_sum(a, left, b, right, out):
    """``out = a * left + b * right`` (float32; ``out`` may be one of them)."""
    _need_cuda(left, right, out)
    require(left.dtype == torch.float32 and right.dtype == torch.float32 and out.dtype == torch.float32
            and left.shape == right.shape == out.shape, "scaled_sum: three float32 tensors of one shape")
    _check(lib().citlali_scaled_sum(_f(a), _ptr(left), _f(b), _ptr(right), _ptr(out), _sz(out.numel()), _stream()), "scaled_sum")


# ---- mixers with a state per sequence -----------------------------------------------------------------------

def causal_conv(x, in_stride, taps_w, state, conv_off, batch, out, in_bias=None, bias=None, act=None, keep=True):
    """A causal convolution over time of the first C columns of ``x`` (a view whose rows are ``in_stride`` floats apart),
    C = ``taps_w.shape[0]``; see ``citlali_causal_conv``.  ``act``: None or "silu"."""
    _need_cuda(taps_w, state, out, in_bias, bias)
    C, taps = taps_w.shape
    rows = out.shape[0]
    require(x.is_cuda and x.dtype == torch.float32 and out.dtype == torch.float32 and taps_w.dtype == torch.float32
            and out.shape[1] >= C and state.dtype == torch.float32 and state.shape[1] >= conv_off + (taps - 1) * C
            and act in (None, "silu"), "causal_conv: shapes or dtypes do not fit")
    _check(lib().citlali_causal_conv(_ptr(x), _i(in_stride), _ptr(in_bias), _ptr(taps_w), _i(taps), _ptr(bias),
                                     _i(1 if act == "silu" else 0), _ptr(state), _sz(state.shape[1]), _sz(conv_off),
                                     _ptr(batch.row_slot), _ptr(batch.seq_start), _ptr(batch.seq_slot), _i(batch.sequences),
                                     _ptr(out), _i(out.shape[1]), _i(rows), _i(C), _i(1 if keep else 0), _stream()),
           "causal_conv_kept" if (keep and taps > 1) else "causal_conv")


_KERNELS_PER_CALL["causal_conv_kept"] = 2
_KERNELS_PER_CALL["ssm_prepare_kept"] = 2


def conv_keep(x, in_stride, taps, C, state, conv_off, batch, in_bias=None):
    _need_cuda(state, in_bias)
    if taps <= 1:
        return
    require(x.is_cuda and x.dtype == torch.float32 and state.shape[1] >= conv_off + (taps - 1) * C, "conv_keep: shapes do not fit")
    _check(lib().citlali_conv_keep(_ptr(x), _i(in_stride), _ptr(in_bias), _i(taps), _ptr(state), _sz(state.shape[1]),
                                   _sz(conv_off), _ptr(batch.seq_start), _ptr(batch.seq_slot), _i(batch.sequences), _i(C),
                                   _stream()), "conv_keep")


def ssm_prepare(proj, taps_w, conv_bias, state, conv_off, batch, a_log, dt_bias, prep, H, P, G, N):
    _need_cuda(proj, taps_w, conv_bias, state, a_log, dt_bias, prep)
    rows = proj.shape[0]
    Cc = H * P + 2 * G * N
    taps = taps_w.shape[1]
    require(proj.dtype == torch.float32 and prep.dtype == torch.float32 and proj.shape[1] == H * P + Cc + H
            and prep.shape == (rows, Cc + 2 * H) and taps_w.shape[0] == Cc and taps_w.dtype == torch.float32
            and (conv_bias is None or conv_bias.numel() == Cc) and a_log.numel() == H and dt_bias.numel() == H
            and state.shape[1] >= conv_off + (taps - 1) * Cc, "ssm_prepare: shapes or dtypes do not fit")
    _check(lib().citlali_ssm_prepare(_ptr(proj), _i(proj.shape[1]), _ptr(taps_w), _i(taps), _ptr(conv_bias), _ptr(state),
                                     _sz(state.shape[1]), _sz(conv_off), _ptr(batch.row_slot), _ptr(batch.seq_start),
                                     _ptr(batch.seq_slot), _i(batch.sequences), _ptr(a_log), _ptr(dt_bias), _ptr(prep),
                                     _i(rows), _i(H), _i(P), _i(G), _i(N), _stream()),
           "ssm_prepare" if taps == 1 else "ssm_prepare_kept")


def ssm_output(o, prep, x_col, proj, skip, weight, y, H, P, groups, eps):
    _need_cuda(o, prep, proj, skip, weight, y)
    require(o.dtype == torch.float32 and o.shape == (prep.shape[0], H * P) and y.shape == o.shape and skip.numel() == H
            and weight.numel() == H * P and skip.dtype == torch.float32 and weight.dtype == torch.float32,
            "ssm_output: shapes or dtypes do not fit")
    _check(lib().citlali_ssm_output(_ptr(o), _ptr(prep), _i(prep.shape[1]), _i(x_col), _ptr(proj), _i(proj.shape[1]),
                                    _ptr(skip), _ptr(weight), _ptr(y), _i(_dtype_code(y)), _i(o.shape[0]), _i(H), _i(P),
                                    _i(groups), _f(eps), _stream()), "ssm_output")


def lru_gates(u, wa_t, ba, wi_t, bi, lam, a_out, coef_out, blocks):
    _need_cuda(u, wa_t, ba, wi_t, bi, lam, a_out, coef_out)
    rows, width = u.shape
    bw = width // max(blocks, 1)
    require(all(t.dtype == torch.float32 for t in (u, wa_t, ba, wi_t, bi, lam, a_out, coef_out))
            and wa_t.shape == (blocks, bw, bw) and wi_t.shape == (blocks, bw, bw) and ba.numel() == width
            and bi.numel() == width and lam.numel() == width and a_out.shape == u.shape and coef_out.shape == u.shape,
            "lru_gates: shapes or dtypes do not fit")
    _check(lib().citlali_lru_gates(_ptr(u), _ptr(wa_t), _ptr(ba), _ptr(wi_t), _ptr(bi), _ptr(lam), _ptr(a_out),
                                   _ptr(coef_out), _i(rows), _i(width), _i(blocks), _stream()), "lru_gates")


def gated_scan(a, coef, side, side_stride, side_bias, state, state_off, batch, out):
    _need_cuda(a, coef, side_bias, state, out)
    rows, width = a.shape
    require(a.dtype == torch.float32 and coef.shape == a.shape and side.is_cuda and side.dtype == torch.float32
            and out.shape == a.shape and state.shape[1] >= state_off + width, "gated_scan: shapes or dtypes do not fit")
    _check(lib().citlali_gated_scan(_ptr(a), _ptr(coef), _ptr(side), _i(side_stride), _ptr(side_bias), _ptr(state),
                                    _sz(state.shape[1]), _sz(state_off), _ptr(batch.seq_start), _ptr(batch.seq_slot),
                                    _i(batch.sequences), _ptr(out), _i(_dtype_code(out)), _i(width), _stream()), "gated_scan")


# ---- attention over a window that keeps the first tokens -------------------------------------------------------

def conv_heads_prepare(proj, taps_w, state, conv_off, q_gain, k_gain, inv_freq, rot_dims, batch, kv, q_out, nq, nkv, d, vd,
                       eps, write_cache=True, bias=None):
    """``kv``: the cache view (keys [page, nkv, page_size, d], values [..., vd], page table).  ``proj`` may be wider than
    q | k | v (what follows is not looked at).  ``bias``: float32, a number a channel, added ahead of the head norm."""
    _need_cuda(proj, taps_w, state, q_gain, k_gain, inv_freq, kv.keys, kv.values, kv.page_table, q_out, bias)
    rows = proj.shape[0]
    C = (nq + nkv) * d + nkv * vd
    require(bias is None or (bias.dtype == torch.float32 and bias.numel() == C), "conv_heads_prepare: the bias does not fit")
    require(proj.dtype == torch.float32 and proj.shape[1] >= C and taps_w.shape[0] == C and taps_w.dtype == torch.float32
            and q_out.shape == (rows, nq * d) and kv.keys.shape[-1] == d and kv.values.shape[-1] == vd
            and kv.keys.dtype == kv.values.dtype and (rot_dims == 0 or inv_freq.numel() == rot_dims // 2),
            "conv_heads_prepare: shapes or dtypes do not fit")
    _check(lib().citlali_conv_heads_prepare(
        _ptr(proj), _i(proj.shape[1]), _ptr(taps_w), _i(taps_w.shape[1]), _ptr(state), _sz(state.shape[1] if state is not None else 0),
        _sz(conv_off), _ptr(q_gain), _ptr(k_gain), _ptr(inv_freq), _i(rot_dims), _ptr(batch.row_slot), _ptr(batch.row_pos),
        _ptr(kv.page_table), _i(kv.page_table.shape[1]), _ptr(kv.keys), _ptr(kv.values), _i(_dtype_code(kv.keys)),
        _i(kv.page_size), _ptr(q_out), _i(_dtype_code(q_out)), _i(rows), _i(nq), _i(nkv), _i(d), _i(vd), _f(eps),
        _i(1 if write_cache else 0), _ptr(bias), _stream()), "conv_heads_prepare")


def attention_window(q, kv, batch, out, nq, nkv, d, vd, window, keep_first, scale, softcap=0.0, gate=None):
    """Attention of every row over its slot's cache, through a window that keeps the first tokens.  bfloat16 steps that
    bring runs of tokens, with keys and values of one size the tensor-core kernel has, run that kernel; steps of single
    tokens, the 32-bit path and other sizes run the kernel whose launch depends on the row count alone.  ``softcap`` c > 0:
    the scaled scores become c tanh(s / c).  ``gate``: float32 columns of a matrix (a view whose rows may be further apart
    than they are long), the output is multiplied by their sigmoids element by element."""
    _need_cuda(q, kv.keys, kv.values, kv.page_table, out)
    rows = q.shape[0]
    require(q.shape == (rows, nq * d) and out.shape == (rows, nq * vd) and q.dtype == out.dtype,
            "attention_window: shapes or dtypes do not fit")
    gate_stride = 0
    if gate is not None:
        require(gate.is_cuda and gate.dtype == torch.float32 and gate.shape == (rows, nq * vd) and gate.stride(1) == 1,
                "attention_window: the gate is float32 [rows, heads * value size] with unit column stride")
        gate_stride = gate.stride(0)
    softcap = float(softcap or 0.0)
    if (q.dtype == torch.bfloat16 and kv.keys.dtype == torch.bfloat16 and d == vd and not batch.is_decode
            and (nq * d) % 8 == 0 and not torch.cuda.is_current_stream_capturing()
            and (gate is None or (gate_stride % 2 == 0 and gate.data_ptr() % 8 == 0))
            and lib().citlali_attention_prefill_supports(_i(d), _i(kv.page_size))):
        attention_prefill(q, nq * d, kv.keys, kv.values, kv.page_table, batch.seq_start, batch.seq_slot, batch.seq_past, out,
                          batch.sequences, batch.max_new, nq, nkv, d, kv.page_size, window, scale, keep_first=keep_first,
                          softcap=softcap, gate=gate)
        return
    longest = kv.page_table.shape[1] * kv.page_size          # a bound that no step's lengths change
    max_keys = min(longest, window + keep_first) if window else longest
    _check(lib().citlali_attention_window(
        _ptr(q), _i(_dtype_code(q)), _ptr(kv.keys), _ptr(kv.values), _i(_dtype_code(kv.keys)), _ptr(kv.page_table),
        _i(kv.page_table.shape[1]), _ptr(batch.row_slot), _ptr(batch.row_pos), _ptr(out), _i(rows), _i(nq), _i(nkv), _i(d),
        _i(vd), _i(kv.page_size), _i(int(window or 0)), _i(int(keep_first or 0)), _i(max_keys), _f(scale), _f(softcap),
        _ptr(gate), _sz(gate_stride), _stream()), "attention_window")


# ---- routed experts -----------------------------------------------------------------------------------------------

ROUTER_SCORES = {"softmax": 0, "sigmoid": 1}


def moe_route(logits, weights, groups, keep, top, chosen=None, weight_scale=1.0, score="softmax"):
    _need_cuda(logits, weights, chosen)
    require(score in ROUTER_SCORES, f"moe_route: unknown score '{score}'; known: {', '.join(ROUTER_SCORES)}")
    rows, E = logits.shape
    require(logits.dtype == torch.float32 and weights.dtype == torch.float32 and weights.shape == logits.shape
            and (chosen is None or (chosen.dtype == torch.int32 and chosen.shape == (rows, top))),
            "moe_route: shapes or dtypes do not fit")
    _check(lib().citlali_moe_route(_ptr(logits), _ptr(weights), _ptr(chosen), _i(rows), _i(E), _i(int(groups or 0)),
                                   _i(int(keep or 0)), _i(top), _f(weight_scale), _i(ROUTER_SCORES[score]), _stream()),
           "moe_route")


def moe_scale(act, weights, ff):
    _need_cuda(act, weights)
    rows, E = weights.shape
    require(act.shape == (rows, E * ff) and weights.dtype == torch.float32, "moe_scale: shapes or dtypes do not fit")
    _check(lib().citlali_moe_scale(_ptr(act), _i(_dtype_code(act)), _ptr(weights), _i(rows), _i(E), _i(ff), _stream()),
           "moe_scale")


EXPERT_ACTIVATIONS = {"silu": 0, "clamped_swish": 1, "gelu_tanh": 2}


def expert_gate(gate_up, weights, act, E, ff, run, kind, limit=0.0, alpha=1.0, tail_ff=0, tail_run=1, tail_limit=0.0,
                bias=None, weight_input=False):
    """The gated activation of ``E`` routed experts (times the row's weight for each) and of a last expert that every row
    uses, from one product ``gate_up`` [rows, 2 (E ff + tail_ff)] into ``act`` [rows, E ff + tail_ff].  ``bias``: float32,
    a number a column of ``gate_up``, added first.  ``weight_input``: the row's weight multiplies gate and up ahead of
    the activation (the expert applied to the weighted input) instead of the activation's result."""
    _need_cuda(gate_up, weights, act, bias)
    require(bias is None or (bias.dtype == torch.float32 and bias.numel() == gate_up.shape[1]), "expert_gate: the bias does not fit")
    rows = act.shape[0]
    n = E * ff + tail_ff
    require(kind in EXPERT_ACTIVATIONS and act.shape == (rows, n) and gate_up.shape == (rows, 2 * n)
            and (E == 0 or (weights is not None and weights.dtype == torch.float32 and weights.shape == (rows, E))),
            "expert_gate: shapes or dtypes do not fit")
    _check(lib().citlali_expert_gate(_ptr(gate_up), _i(_dtype_code(gate_up)), _ptr(weights), _ptr(act), _i(_dtype_code(act)),
                                     _i(rows), _i(E), _i(ff), _i(run), _i(EXPERT_ACTIVATIONS[kind]), _f(limit), _f(alpha),
                                     _i(tail_ff), _i(tail_run), _f(tail_limit), _ptr(bias), _i(1 if weight_input else 0),
                                     _stream()), "expert_gate")


def bias_xielu(z, bias, ap, an, out):
    """``out = xielu(z + bias)``: u > 0: ap u^2 + u / 2; else an (exp(u) - 1 - u) + u / 2.  ``bias`` float32 or None."""
    _need_cuda(z, bias, out)
    rows, n = z.shape
    require(out.shape == z.shape and (bias is None or (bias.dtype == torch.float32 and bias.numel() == n)),
            "bias_xielu: shapes or dtypes do not fit")
    _check(lib().citlali_bias_xielu(_ptr(z), _i(_dtype_code(z)), _ptr(bias), _f(ap), _f(an), _ptr(out), _i(_dtype_code(out)),
                                    _i(rows), _i(n), _stream()), "bias_xielu")


def add_row_bias(y, bias):
    """``y[r] += bias`` over float32 rows."""
    _need_cuda(y, bias)
    require(y.dtype == torch.float32 and bias.dtype == torch.float32 and bias.numel() == y.shape[1],
            "add_row_bias: a float32 matrix and a float32 vector of its row length")
    _check(lib().citlali_add_row_bias(_ptr(y), _ptr(bias), _i(y.shape[0]), _i(y.shape[1]), _stream()), "add_row_bias")


# ---- attention with sigmoid weights --------------------------------------------------------------------------------

def biased_heads_prepare(proj, bias, batch, kv, q_out, gate_out, H, G, D, V, has_kv, temp_coef, temp_every):
    """Bias, query temperature, cache write and the gate's sigmoid for ``proj`` = q | k | v | gate (float32)."""
    _need_cuda(proj, bias, kv.keys, kv.values, kv.page_table, q_out, gate_out)
    rows = proj.shape[0]
    C = H * D + (G * (D + V) if has_kv else 0) + (H if gate_out is not None else 0)
    require(proj.dtype == torch.float32 and proj.shape == (rows, C) and q_out.shape == (rows, H * D)
            and (bias is None or (bias.dtype == torch.float32 and bias.numel() == C))
            and (gate_out is None or (gate_out.dtype == torch.float32 and gate_out.shape == (rows, H)))
            and kv.keys.shape[-1] == D and kv.values.shape[-1] == V and kv.keys.shape[-3] == G
            and kv.keys.dtype == kv.values.dtype, "biased_heads_prepare: shapes or dtypes do not fit")
    _check(lib().citlali_biased_heads_prepare(
        _ptr(proj), _ptr(bias), _ptr(batch.row_slot), _ptr(batch.row_pos), _ptr(kv.page_table), _i(kv.page_table.shape[1]),
        _ptr(kv.keys), _ptr(kv.values), _i(_dtype_code(kv.keys)), _i(kv.page_size), _ptr(q_out), _i(_dtype_code(q_out)),
        _ptr(gate_out), _i(rows), _i(H), _i(G), _i(D), _i(V), _i(1 if has_kv else 0), _i(1 if gate_out is not None else 0),
        _f(temp_coef), _i(int(temp_every or 0)), _stream()), "biased_heads_prepare")


def sigmoid_attention_run_keys() -> int:
    return int(lib().citlali_sigmoid_attention_run_keys())


def sigmoid_attention(q, kv, batch, talk, head_bias, gate, out, H, G, D, V, window, scale, slope_exp, runs=1):
    """Every row over its slot's cache with sigmoid weights on scores mixed over the heads.  ``runs`` > 1: the keys of a row
    are dealt to that many blocks (it must cover the longest row) and a second kernel adds their sums; same bits."""
    _need_cuda(q, kv.keys, kv.values, kv.page_table, talk, head_bias, gate, out)
    rows = q.shape[0]
    require(q.shape == (rows, H * D) and out.shape == (rows, H * V) and q.dtype == out.dtype
            and (talk is None or (talk.dtype == torch.float32 and talk.shape == (H, H)))
            and (head_bias is None or (head_bias.dtype == torch.float32 and head_bias.numel() == H))
            and (gate is None or (gate.dtype == torch.float32 and gate.shape == (rows, H))),
            "sigmoid_attention: shapes or dtypes do not fit")
    partial = None
    if runs > 1:
        partial = torch.empty((rows, runs, H * V), dtype=torch.float32, device=q.device)
    _check(lib().citlali_sigmoid_attention(
        _ptr(q), _i(_dtype_code(q)), _ptr(kv.keys), _ptr(kv.values), _i(_dtype_code(kv.keys)), _ptr(kv.page_table),
        _i(kv.page_table.shape[1]), _ptr(batch.row_slot), _ptr(batch.row_pos), _ptr(talk), _ptr(head_bias), _ptr(gate),
        _ptr(out), _ptr(partial), _i(runs), _i(rows), _i(H), _i(G), _i(D), _i(V), _i(kv.page_size), _i(int(window or 0)),
        _f(scale), _f(slope_exp), _stream()), "sigmoid_attention")


def sigmoid_attention_mma_supports(H, G, D, V, page_size) -> bool:
    return bool(lib().citlali_sigmoid_attention_mma_supports(_i(H), _i(G), _i(D), _i(V), _i(page_size)))


def sigmoid_attention_mma_scratch_bytes(rows, sequences, max_keys, H, window) -> int:
    """Bytes of the weights that ``sigmoid_attention_mma`` keeps between its two kernels."""
    l = lib()
    columns = int(l.citlali_sigmoid_attention_mma_columns(_i(int(window or 0)), _i(max_keys)))
    groups = int(l.citlali_sigmoid_attention_mma_groups(_i(rows), _i(sequences)))
    return H * groups * columns * 8 * 2


def sigmoid_attention_mma(q, kv, batch, talk, head_bias, gate, out, H, G, D, V, window, scale, slope_exp):
    """``sigmoid_attention`` for runs of new tokens on the tensor cores (bfloat16): every head's weights go to a scratch
    buffer, a second kernel multiplies them with the values."""
    _need_cuda(q, kv.keys, kv.values, kv.page_table, talk, head_bias, gate, out)
    rows = q.shape[0]
    require(q.dtype == torch.bfloat16 and kv.keys.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
            and q.shape == (rows, H * D) and out.shape == (rows, H * V) and q.is_contiguous() and out.is_contiguous()
            and (talk is None or (talk.dtype == torch.float32 and talk.shape == (H, H)))
            and (head_bias is None or (head_bias.dtype == torch.float32 and head_bias.numel() == H))
            and (gate is None or (gate.dtype == torch.float32 and gate.shape == (rows, H))),
            "sigmoid_attention_mma: shapes or dtypes do not fit")
    l = lib()
    sequences = len(batch.slots)
    columns = int(l.citlali_sigmoid_attention_mma_columns(_i(int(window or 0)), _i(max(batch.max_keys, 1))))
    groups = int(l.citlali_sigmoid_attention_mma_groups(_i(rows), _i(sequences)))
    weights = _scratch(q.device, "sigmoid attention weights", H * groups * columns * 8 * 2)
    _check(l.citlali_sigmoid_attention_mma(
        _ptr(q), _ptr(kv.keys), _ptr(kv.values), _ptr(kv.page_table), _i(kv.page_table.shape[1]), _ptr(batch.seq_start),
        _ptr(batch.seq_slot), _ptr(batch.seq_past), _ptr(talk), _ptr(head_bias), _ptr(gate), _ptr(out), _ptr(weights),
        _i(columns), _i(groups), _i(sequences), _i(max(batch.n_new)), _i(H), _i(G), _i(D), _i(V), _i(kv.page_size),
        _i(int(window or 0)), _f(scale), _f(slope_exp), _stream()), "sigmoid_attention_mma")


# ---- attention through a shared latent -------------------------------------------------------------

def latent_prepare(proj, RQ, R, P, has_kv, q_weight, c_weight, inv_freq, rot_dims, row_slot, row_pos, page_table, pool,
                   page_size, cq, eps, rot_halves=False):
    _need_cuda(proj, q_weight, c_weight, inv_freq, row_slot, row_pos, page_table, pool, cq)
    rows = proj.shape[0]
    require(proj.dtype == torch.float32 and q_weight.dtype == torch.float32 and cq.shape == (rows, RQ)
            and proj.shape[1] >= RQ + (R + P if has_kv else 0), "latent_prepare: shapes or dtypes do not fit")
    if has_kv:
        require(pool is not None and pool.shape[-1] == R + P and c_weight.dtype == torch.float32
                and (rot_dims == 0 or (inv_freq is not None and inv_freq.numel() == rot_dims // 2)),
                "latent_prepare: the cache or the rotation's table does not fit")
    _check(lib().citlali_latent_prepare(
        _ptr(proj), _i(proj.shape[1]), _i(RQ), _i(R), _i(P), _i(1 if has_kv else 0), _ptr(q_weight), _ptr(c_weight),
        _ptr(inv_freq), _i(rot_dims), _ptr(row_slot), _ptr(row_pos), _ptr(page_table), _i(page_table.shape[1]), _ptr(pool),
        _i(_dtype_code(pool) if pool is not None else _F32), _i(page_size), _ptr(cq), _i(_dtype_code(cq)), _i(rows),
        _f(eps), _i(1 if rot_halves else 0), _stream()), "latent_prepare")


def heads_product(x, x_row, x_head, M, m_head, m_k, m_n, y, y_row, y_head, rows, heads, K, N, tail=0, inv_freq=None,
                  rot_dims=0, row_pos=None, gate=None, gate_stride=0, rot_halves=False, gate_per_head=False):
    """``y[r, h, :N] = x[r, h, :K] . M_h`` with a matrix per head given by strides; see ``citlali_heads_product``."""
    _need_cuda(M, y, inv_freq, row_pos)
    require(x.is_cuda and (gate is None or (gate.is_cuda and gate.dtype == torch.float32)), "heads_product: bad operands")
    _check(lib().citlali_heads_product(
        _ptr(x), _i(_dtype_code(x)), _sz(x_row), _i(x_head), _ptr(M), _i(_dtype_code(M)), _sz(m_head), _i(m_k), _i(m_n),
        _ptr(y), _i(_dtype_code(y)), _sz(y_row), _i(y_head), _i(rows), _i(heads), _i(K), _i(N), _i(tail), _ptr(inv_freq),
        _i(rot_dims), _ptr(row_pos), _ptr(gate), _sz(gate_stride), _i(1 if rot_halves else 0),
        _i(1 if gate_per_head else 0), _stream()), "heads_product")


_KERNELS_PER_CALL["latent_attention_mma_runs"] = 2


def latent_attention(q, pool, page_table, row_slot, row_pos, sink, out, H, R, E, page_size, window, scale,
                     tensor_cores=None, splits=None):
    """The walk over a latent cache.  A bfloat16 cache whose sizes the tensor-core kernel takes runs that kernel
    (``tensor_cores`` False: never), everything else the one on CUDA cores, which is exact in 32-bit."""
    _need_cuda(q, pool, page_table, row_slot, row_pos, sink, out)
    rows = q.shape[0]
    require(q.dtype == torch.float32 and out.dtype == torch.float32 and q.shape == (rows, H * E)
            and out.shape == (rows, H * R) and pool.shape[-1] == E and (sink is None or (sink.dtype == torch.float32
            and sink.numel() == H)), "latent_attention: shapes or dtypes do not fit")
    if (tensor_cores is not False and pool.dtype == torch.bfloat16
            and lib().citlali_latent_attention_mma_supports(_i(R), _i(E))):
        # few rows (decoding): a unit's key tiles go to several blocks, so that the device is busy; the number of runs
        # follows the number of rows alone and never exceeds the tiles a window (or the longest sequence) has
        units = rows * ((H + 15) // 16)
        longest = int(window) if window else page_table.shape[1] * page_size
        splits = max(1, min(sm_count(q.device) * 2 // units, (longest + 63) // 64, 32)) if splits is None else int(splits)
        partial = None
        if splits > 1:
            partial = _scratch(q.device, "latent_attention runs", units * splits * 16 * (R + 2) * 4)
        _check(lib().citlali_latent_attention_mma(_ptr(q), _ptr(pool), _ptr(page_table), _i(page_table.shape[1]),
                                                  _ptr(row_slot), _ptr(row_pos), _ptr(sink), _ptr(out), _i(rows), _i(H),
                                                  _i(R), _i(E), _i(page_size), _i(int(window or 0)), _f(scale), _i(splits),
                                                  _ptr(partial), _sz(partial.numel() // 4 if partial is not None else 0),
                                                  _stream()),
               "latent_attention_mma" if splits == 1 else "latent_attention_mma_runs")
        return
    require(tensor_cores is not True, "latent_attention: the tensor-core kernel does not take this cache")
    _check(lib().citlali_latent_attention(_ptr(q), _ptr(pool), _i(_dtype_code(pool)), _ptr(page_table),
                                          _i(page_table.shape[1]), _ptr(row_slot), _ptr(row_pos), _ptr(sink), _ptr(out),
                                          _i(rows), _i(H), _i(R), _i(E), _i(page_size), _i(int(window or 0)), _f(scale),
                                          _stream()), "latent_attention")
