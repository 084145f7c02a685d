"""Python face of the hand-written CUDA kernels (``csrc/*.cu``) and of the library matrix
product.  Every function here works on CUDA tensors on the current stream and has no
other implementation: if the kernel library cannot be built or loaded, the first call
raises ``KernelLibraryError``.

The matrix product (``linear``, ``linear_swiglu``) has two kernels of this package for
bfloat16, chosen by the number of rows: up to 8 the weight-streaming mma.sync product
(``gemm_skinny``), from 256 on, where the tiles fill the GPU, the TMA + tcgen05 product
(``gemm_tcgen05``).  Everything else is the library's (cuBLAS through ``torch.mm``), as in the reference, which calls
``cublasHgemm`` for every projection with more than one row
(kernels/src/matmul_kernel_cuda.cu:83-91); in float32 mode it runs with the
reduced-precision matrix modes switched off.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..csrc import build as _build

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

# flags of qk_norm_rope_store (csrc/qk_rope_store.cu)
QK_NORM, QK_ROPE, QK_STORE, QK_QOUT, QK_KVOUT = 1, 2, 4, 8, 16


class KernelLibraryError(RuntimeError):
    pass


class KernelError(RuntimeError):
    pass


_lib = None


def lib():
    """The loaded kernel library (built on first use)."""
    global _lib
    if _lib is not None:
        return _lib
    try:
        path = _build.library_path()
    except Exception as exc:  # BuildError and anything the toolchain throws
        raise KernelLibraryError(f"the CUDA kernel library is not available: {exc}") from exc
    try:
        handle = ctypes.CDLL(str(path))
    except OSError as exc:
        raise KernelLibraryError(f"cannot load {path}: {exc}") from exc
    _declare(handle)
    _lib = handle
    return handle


def _declare(h) -> None:
    vp, i32, f32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
    h.tllm_last_error.restype = ctypes.c_char_p
    h.tllm_last_error.argtypes = []
    sigs = {
        "tllm_embedding": [vp, vp, i32, vp, i32, i32, i32, vp],
        "tllm_add_rmsnorm": [vp, vp, vp, i32, f32, vp, i32, vp, i32, i32, vp],
        "tllm_swiglu": [vp, vp, i32, i32, i32, i32, vp],
        "tllm_cast": [vp, i32, vp, i32, i64, vp],
        "tllm_feed_tokens": [vp, vp, vp, vp, i32, vp],
        "tllm_qk_norm_rope_store": [vp, vp, vp, i32, f32, vp, i32, vp, vp, vp, i32, vp, i32, vp,
                                    i32, i32, i32, i32, i32, i32, vp, vp],
        "tllm_rope_table": [vp, vp, i32, i32, vp, vp],
        "tllm_paged_attention_general": [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32,
                                         i32, f32, vp, vp],
        "tllm_sample": [vp, i32, i32, i64, vp, vp, vp, vp],
        "tllm_sample_split": [vp, i32, i32, i64, vp, vp, vp, vp, i32, vp, vp],
        "tllm_gemm_skinny": [vp, vp, vp, i32, i32, i32, i32, vp],
        "tllm_gemm_plain": [vp, i32, vp, i32, vp, i32, i32, i32, i32, vp],
        "tllm_gemm_tcgen05": [vp, vp, vp, i32, i32, i32, i32, vp, vp],
        "tllm_gemm_skinny_swiglu": [vp, vp, vp, i32, i32, i32, vp],
        "tllm_paged_attention_decode": [vp, vp, vp, vp, vp, i32, vp, i32, i32, i32, i32, i32, i32, f32,
                                        i32, vp, vp, vp, vp],
        "tllm_paged_attention_prefill": [vp, vp, vp, vp, i32, vp, i32, i32, i32, i32, i32, i32, f32, vp, vp],
        "tllm_paged_attention_prefill_tc": [vp, i32, vp, i32, vp, vp, i32, vp, i32, i32, i32, i32, i32, i32, f32,
                                            vp, i32, vp, vp, vp, vp],
    }
    for name, args in sigs.items():
        fn = getattr(h, name)
        fn.argtypes = args
        fn.restype = i32
    h.tllm_paged_attention_prefill_tc_rows.argtypes = [i32, i32]
    h.tllm_paged_attention_prefill_tc_rows.restype = i32
    h.tllm_sample_nucleus_scratch_bytes.argtypes = [i32]
    h.tllm_sample_nucleus_scratch_bytes.restype = i64
    h.tllm_uniform_of.argtypes = [ctypes.c_ulonglong, i32]
    h.tllm_uniform_of.restype = f32


launches = 0      # kernels of csrc/ launched so far (graph replays are added by the runner)


def _check(code: int, what: str, kernels: int = 1) -> None:
    global launches
    launches += kernels
    if code != 0:
        raise KernelError(f"{what}: {lib().tllm_last_error().decode(errors='replace')} (code {code})")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """Handle of the current CUDA stream of the current device (the raw getter costs a fraction
    of a microsecond, the Stream object several)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise KernelError("kernels take contiguous CUDA tensors")


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"unsupported dtype {t.dtype}") from None


# --------------------------------------------------------------------------- ops
def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] = table[ids[t]] as float32; rows with a negative id become zero."""
    _cuda(ids, table, out)
    assert ids.dtype == torch.int32 and out.dtype == torch.float32
    vocab, hidden = table.shape
    _check(lib().tllm_embedding(_p(ids), _p(table), _dt(table), _p(out), ids.numel(), hidden, vocab,
                                _stream()), "embedding")
    return out


def add_rmsnorm(h: torch.Tensor, delta: Optional[torch.Tensor], gain: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """h += delta (float32 sum, written back) and out = gain * h / sqrt(mean(h^2) + eps).
    With ``rows`` only those rows are normed, into out[0..len(rows)), and h is not written."""
    _cuda(h, delta, gain, out, rows)
    assert h.dtype == torch.float32
    if delta is not None:
        assert delta.dtype == out.dtype and delta.shape == h.shape
    n_out = out.shape[0] if rows is None else rows.numel()
    _check(lib().tllm_add_rmsnorm(_p(h), _p(delta), _p(gain), _dt(gain), float(eps), _p(out), _dt(out),
                                  _p(rows), n_out, h.shape[-1], _stream()), "add_rmsnorm")
    return out


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[2 I, K] with the rows of ``gate`` and ``up`` ([I, K], I a multiple of 8) interleaved by
    eight: eight gate rows, the eight up rows that belong to them, and so on.  A block of the
    weight-streaming product and a tile of the tcgen05 product then read neighbouring rows and
    find a gate and its up in one accumulator, so SwiGLU fits their epilogues."""
    inter, k = gate.shape
    assert up.shape == gate.shape and inter % 8 == 0
    return torch.stack([gate.reshape(inter // 8, 8, k), up.reshape(inter // 8, 8, k)], dim=1).reshape(2 * inter, k)


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> torch.Tensor:
    """out[t, i] = silu(gate) * up with gate = gate_up[t, i], up = gate_up[t, I + i], or, for columns
    interleaved by eight, gate = gate_up[t, 16 (i // 8) + i % 8] and up eight columns further."""
    _cuda(gate_up, out)
    tokens, two_i = gate_up.shape
    assert out.shape == (tokens, two_i // 2) and out.dtype == gate_up.dtype
    _check(lib().tllm_swiglu(_p(gate_up), _p(out), _dt(out), tokens, two_i // 2, int(interleaved), _stream()),
           "swiglu")
    return out


def cast(src: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    _cuda(src)
    if src.dtype == dtype:
        return src
    dst = torch.empty_like(src, dtype=dtype)
    _check(lib().tllm_cast(_p(src), _dt(src), _p(dst), _dt(dst), src.numel(), _stream()), "cast")
    return dst


def feed_tokens(ids: torch.Tensor, places: torch.Tensor, rows: torch.Tensor, sampled: torch.Tensor) -> None:
    """ids[places[i]] = sampled[rows[i]] (all int32, on the device): the tokens that the step before
    is still sampling go into this step's token ids without passing through the host."""
    _cuda(ids, places, rows, sampled)
    assert ids.dtype == places.dtype == rows.dtype == sampled.dtype == torch.int32 and places.numel() == rows.numel()
    _check(lib().tllm_feed_tokens(_p(ids), _p(places), _p(rows), _p(sampled), places.numel(), _stream()), "feed_tokens")


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """[tokens, 2, half] float32: cosines and sines of position * inv_freq (the float32 product), made
    once per step and read by every layer's ``qk_norm_rope_store``."""
    _cuda(positions, inv_freq)
    assert positions.dtype == torch.int32 and inv_freq.dtype == torch.float32
    tokens, half = positions.numel(), inv_freq.numel()
    table = torch.empty((tokens, 2, half), dtype=torch.float32, device=positions.device)
    _check(lib().tllm_rope_table(_p(positions), _p(inv_freq), half, tokens, _p(table), _stream()), "rope_table")
    return table


def qk_norm_rope_store(qkv: torch.Tensor, q_gain, k_gain, eps: float, inv_freq, rotary_dim: int,
                       positions: torch.Tensor, token_slot: torch.Tensor, block_table, cache,
                       page_size: int, q_out, q_heads: int, kv_heads: int, head_dim: int,
                       flags: int, table: Optional[torch.Tensor] = None) -> None:
    """One pass over the fused q|k|v rows [T, (q_heads + 2 kv_heads) * head_dim]: per-head
    RMSNorm of q and k (QK_NORM), rotate-half rotation (QK_ROPE), write of k and v into
    their page (QK_STORE), write of q to ``q_out`` (QK_QOUT), write of the processed k back
    in place (QK_KVOUT).  Rows whose token_slot is negative are skipped.  ``table``: the step's
    ``rope_table`` for these positions and frequencies (same values, no sincosf per layer)."""
    _cuda(qkv, q_gain, k_gain, inv_freq, positions, token_slot, block_table, cache, q_out, table)
    if table is not None:
        assert table.dtype == torch.float32 and tuple(table.shape) == (qkv.shape[0], 2, rotary_dim // 2)
    tokens = qkv.shape[0]
    assert qkv.shape[1] == (q_heads + 2 * kv_heads) * head_dim
    gain_dt = _dt(q_gain) if q_gain is not None else F32
    max_pages = block_table.shape[1] if block_table is not None else 0
    if cache is not None:
        assert cache.dtype == qkv.dtype and tuple(cache.shape[1:]) == (2, kv_heads, page_size, head_dim)
    _check(lib().tllm_qk_norm_rope_store(
        _p(qkv), _p(q_gain), _p(k_gain), gain_dt, float(eps), _p(inv_freq), rotary_dim,
        _p(positions), _p(token_slot), _p(block_table), max_pages, _p(cache), page_size, _p(q_out),
        _dt(qkv), tokens, q_heads, kv_heads, head_dim, flags, _p(table), _stream()), "qk_norm_rope_store")


_workspaces = {}


WORKSPACE_FLOATS = 16 << 20


def workspace(device, floats: int) -> torch.Tensor:
    """Float32 scratch for one call.  Up to WORKSPACE_FLOATS it is one buffer per device
    that lives as long as the process and never moves (captured CUDA graphs keep its
    address); a larger request gets a tensor of its own."""
    if floats > WORKSPACE_FLOATS:
        return torch.empty(floats, dtype=torch.float32, device=device)
    key = str(device)
    buf = _workspaces.get(key)
    if buf is None:
        buf = torch.empty(WORKSPACE_FLOATS, dtype=torch.float32, device=device)
        _workspaces[key] = buf
    return buf


SM_COUNT = 148


def decode_splits(rows: int, kv_heads: int, max_context: int) -> int:
    """How many blocks share the keys of one (row, key/value head): enough blocks for
    about four per multiprocessor, each with at least 128 keys."""
    by_length = -(-max_context // 1024)                       # about a thousand keys per block
    by_count = -(-128 // max(rows * kv_heads, 1))             # but at least 128 blocks in all
    return max(1, min(max(by_length, by_count), -(-max_context // 128), 64))


def fast_attention_ok(dtype, page_size: int, q_heads: int, kv_heads: int, head_dim: int) -> bool:
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and page_size % 16 == 0
            and q_heads % kv_heads == 0 and q_heads // kv_heads <= 16)


def paged_attention_decode(q, cache, positions, token_slot, rows, n_rows, block_table, page_size,
                           q_heads, kv_heads, head_dim, window, scale, out, max_context, splits=None):
    """Attention of one-token rows (``rows``: their indices, None for all), keys split over
    ``splits`` blocks per (row, key/value head); the splits' partial results go through scratch
    in global memory to a second small kernel that combines them in the order of the splits."""
    _cuda(q, cache, positions, token_slot, rows, block_table, out)
    if splits is None:
        splits = decode_splits(n_rows, kv_heads, max_context)
    part_o = part_ml = None
    if splits > 1:
        n = n_rows * q_heads * splits
        ws = workspace(q.device, n * (head_dim + 2))
        part_o, part_ml = ws[:n * head_dim], ws[n * head_dim:n * (head_dim + 2)]
    _check(lib().tllm_paged_attention_decode(
        _p(q), _p(cache), _p(positions), _p(token_slot), _p(rows), n_rows, _p(block_table),
        block_table.shape[1], page_size, q_heads, kv_heads, head_dim, int(window or 0), float(scale),
        splits, _p(part_o), _p(part_ml), _p(out), _stream()), "paged_attention_decode",
        kernels=2 if splits > 1 else 1)
    return out


def paged_attention_prefill(q, cache, seg_info, tiles, n_tiles, block_table, page_size, q_heads,
                            kv_heads, head_dim, window, scale, out):
    """Attention of the segments' query blocks listed in ``tiles`` ([n, 2] = segment, offset)."""
    _cuda(q, cache, seg_info, tiles, block_table, out)
    _check(lib().tllm_paged_attention_prefill(
        _p(q), _p(cache), _p(seg_info), _p(tiles), n_tiles, _p(block_table), block_table.shape[1],
        page_size, q_heads, kv_heads, head_dim, int(window or 0), float(scale), _p(out), _stream()),
        "paged_attention_prefill")
    return out


PREFILL_TCGEN05 = True     # head width 128 takes the tcgen05 kernel; False keeps the mma.sync one


def prefill_tcgen05_block_rows(q_heads: int, kv_heads: int) -> int:
    """Query rows per entry of the tile list that ``paged_attention_prefill_tcgen05`` wants: 128
    where two heads of one key/value head share a thread block (an even group), else 256."""
    return int(lib().tllm_paged_attention_prefill_tc_rows(q_heads, kv_heads))


def prefill_splits(blocks: int, max_context: int) -> int:
    """Runs of keys per block of query rows in ``paged_attention_prefill_tcgen05``: 1, 2, 4 or 8.
    A step with few query rows (a short portion of a prompt) has few blocks, each walking all keys
    of its request; cutting the keys fills the GPU (148 SMs, one block each), as long as a run
    keeps eight tiles of 64 keys, below which a block's start and end outweigh its work."""
    fit = min(SM_COUNT // max(blocks, 1), -(-max_context // 64) // 8)
    splits = 1
    while splits * 2 <= min(fit, 8):
        splits *= 2
    return splits



def paged_attention_prefill_tcgen05(q, cache, seg_info, tiles, n_tiles, block_table, page_size, q_heads,
                                    kv_heads, head_dim, window, scale, out, splits=1):
    """As ``paged_attention_prefill`` on tcgen05 tensor cores with TMA loads: bfloat16, head width
    128, ``tiles`` at multiples of ``prefill_tcgen05_block_rows`` rows.  With ``splits`` > 1 every
    block's keys are shared by that many blocks and a second kernel combines what they leave.
    The kernel's waits are bounded; what they report is read by ``check_error_word``."""
    _cuda(q, cache, seg_info, tiles, block_table, out)
    assert q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert q.shape[1] == q_heads * head_dim and tuple(out.shape) == tuple(q.shape)
    global tcgen05_calls
    tcgen05_calls += 1
    part_o = part_ml = None
    if splits > 1:
        n = q.shape[0] * q_heads * splits
        ws = workspace(q.device, n * (head_dim + 2))
        part_o, part_ml = ws[:n * head_dim], ws[n * head_dim:n * (head_dim + 2)]
    _check(lib().tllm_paged_attention_prefill_tc(
        _p(q), q.shape[0], _p(cache), cache.shape[0], _p(seg_info), _p(tiles), n_tiles, _p(block_table),
        block_table.shape[1], page_size, q_heads, kv_heads, head_dim, int(window or 0), float(scale),
        _p(out), splits, _p(part_o), _p(part_ml), _p(error_word(q.device)), _stream()), "paged_attention_prefill_tc",
        kernels=2 if splits > 1 else 1)
    return out


def paged_attention(q: torch.Tensor, cache: torch.Tensor, positions, token_slot, block_table,
                    page_size: int, q_heads: int, kv_heads: int, head_dim: int,
                    window: Optional[int], scale: float, out: torch.Tensor, ctx=None) -> torch.Tensor:
    """Attention of every row of ``q`` over the keys of its own request in the paged cache:
    positions max(0, pos - window + 1) .. pos.  With the step's context and a shape the
    tensor-core kernels take (bfloat16, head width 64 or 128, pages of a multiple of 16),
    one-token rows go to the split-key decode kernel and longer segments to the tiled
    prefill kernel; everything else runs the general kernel."""
    _cuda(q, cache, positions, token_slot, block_table, out)
    tokens = q.shape[0]
    assert tuple(cache.shape[1:]) == (2, kv_heads, page_size, head_dim) and cache.dtype == q.dtype
    if ctx is not None and ctx.pf_tiles is not None and ctx.tokens == tokens \
            and fast_attention_ok(q.dtype, page_size, q_heads, kv_heads, head_dim):
        if ctx.n_dec:
            paged_attention_decode(q, cache, positions, token_slot, ctx.dec_rows, ctx.n_dec, block_table,
                                   page_size, q_heads, kv_heads, head_dim, window, scale, out,
                                   ctx.max_context)
        if ctx.n_tiles:
            if PREFILL_TCGEN05 and head_dim == 128 and getattr(ctx, "n_tiles256", 0):
                pairs = prefill_tcgen05_block_rows(q_heads, kv_heads) == 128
                blocks = ctx.n_tiles128 if pairs else ctx.n_tiles256
                keys = ctx.max_context if not window else min(ctx.max_context, window + 256)
                splits = prefill_splits(blocks * (q_heads // 2 if pairs else q_heads), keys)
                paged_attention_prefill_tcgen05(q, cache, ctx.seg_info, ctx.pf_tiles, blocks,
                                                block_table, page_size, q_heads, kv_heads, head_dim,
                                                window, scale, out, splits)
            else:
                paged_attention_prefill(q, cache, ctx.seg_info, ctx.pf_tiles, ctx.n_tiles, block_table,
                                        page_size, q_heads, kv_heads, head_dim, window, scale, out)
        return out
    _check(lib().tllm_paged_attention_general(
        _p(q), _p(cache), _p(positions), _p(token_slot), _p(block_table), block_table.shape[1],
        page_size, _dt(q), tokens, q_heads, kv_heads, head_dim, int(window or 0), float(scale),
        _p(out), _stream()), "paged_attention")
    return out


SAMPLE_BLOCKS = 1024     # blocks over all rows beyond which a row's vocabulary is cut less finely


def sample(logits: torch.Tensor, params: torch.Tensor, seeds: torch.Tensor,
           out: torch.Tensor, any_nucleus: Optional[bool] = None) -> torch.Tensor:
    """Token per row of float32 ``logits`` [S, V]: params[s] = (temperature, top_p), seeds[s]
    an int64 key.  temperature <= 1e-6 is argmax (lowest id on ties).  ``any_nucleus`` says
    whether some row samples with top_p < 1 (None: not known, assume so)."""
    _cuda(logits, params, seeds, out)
    assert logits.dtype == torch.float32 and params.dtype == torch.float32
    assert seeds.dtype == torch.int64 and out.dtype == torch.int32
    rows, vocab = logits.shape
    if vocab >= 4096 and rows > 0:
        # a row's vocabulary shared by several blocks; rows with top-p take four more passes
        blocks = min(64, -(-vocab // 2048), max(8, SAMPLE_BLOCKS // rows))
        partial = torch.empty((rows, blocks, 2), dtype=torch.float32, device=logits.device)
        scratch = None
        if any_nucleus is None or any_nucleus:
            size = lib().tllm_sample_nucleus_scratch_bytes(rows)
            scratch = torch.empty(size // 8, dtype=torch.int64, device=logits.device)
        _check(lib().tllm_sample_split(_p(logits), rows, vocab, logits.stride(0), _p(params), _p(seeds),
                                       _p(out), _p(partial), blocks, _p(scratch), _stream()), "sample",
               kernels=2 if scratch is None else 7)
        return out
    _check(lib().tllm_sample(_p(logits), rows, vocab, logits.stride(0), _p(params), _p(seeds),
                             _p(out), _stream()), "sample")
    return out


def uniform_of(seed: int, token: int) -> float:
    """The uniform number the sampler draws for (seed, token); for host-side checks."""
    return float(lib().tllm_uniform_of(seed & 0xFFFFFFFFFFFFFFFF, token))


SKINNY_MAX_ROWS = 8       # up to this many rows the weight-streaming product beats the library


def gemm_skinny(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """y = x . weight^T for at most 32 bfloat16 rows: every weight is read once, straight from
    HBM into tensor-core fragments (csrc/gemm_skinny.cu)."""
    _cuda(x, weight)
    rows, k = x.shape
    n = weight.shape[0]
    assert weight.shape[1] == k and x.dtype == weight.dtype == torch.bfloat16
    y = torch.empty((rows, n), dtype=out_dtype, device=x.device)
    _check(lib().tllm_gemm_skinny(_p(x), _p(weight), _p(y), _DT[out_dtype], rows, n, k, _stream()),
           "gemm_skinny")
    return y


def gemm_plain(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """y = x . weight^T by the plain kernel (csrc/gemm_plain.cu): one thread per output, the sum over
    k in order in float32, any sizes, bfloat16 or float32 operands.  Slow; it is what the fast products
    are checked against at sizes too large for the host."""
    _cuda(x, weight)
    rows, k = x.shape
    n = weight.shape[0]
    assert weight.shape[1] == k
    y = torch.empty((rows, n), dtype=out_dtype, device=x.device)
    _check(lib().tllm_gemm_plain(_p(x), _dt(x), _p(weight), _dt(weight), _p(y), _dt(y), rows, n, k, _stream()), "gemm_plain")
    return y


_error_words = {}


def error_word(device) -> torch.Tensor:
    """Device int32 that kernels with bounded waits (the tcgen05 product) set to a non-zero
    code when a wait ran out.  ``check_error_word`` reads it (a synchronisation)."""
    key = str(device)
    if key not in _error_words:
        _error_words[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_words[key]


def check_error_word(device) -> None:
    code = int(error_word(device).item())
    if code:
        error_word(device).zero_()
        raise KernelError(f"a bounded wait ran out inside a kernel (code {code}); its result is invalid")


tcgen05_calls = 0          # products issued on the tcgen05 path (their bounded waits report to error_word)


def tcgen05_pays(rows: int, out_cols: int, k: int, dtype, col_tile: int = 256) -> bool:
    """Whether the hand-written tcgen05 product is used instead of the library's: bfloat16, at
    least 256 rows, and a tile count that fills the SMs' last round to 85% (blocks of 256 rows;
    with fewer tiles per round the library's 2-CTA kernels are faster)."""
    if dtype != torch.bfloat16 or rows < 256 or k % 8 or out_cols % 8:
        return False
    tiles = -(-rows // 256) * -(-out_cols // col_tile)
    rounds = -(-tiles // SM_COUNT)
    return tiles / (rounds * SM_COUNT) >= 0.85


def gemm_tcgen05(x: torch.Tensor, weight: torch.Tensor, swiglu: bool = False, short_tiles: bool = False,
                 interleaved: bool = False) -> torch.Tensor:
    """y = x . weight^T on tcgen05 tensor cores fed by TMA (csrc/gemm_tcgen05.cu), bfloat16 in
    and out, float32 accumulation in tensor memory.  With ``swiglu`` the weight is [gate; up]
    (or, ``interleaved``, gate and up rows interleaved by eight) and the result is
    silu(x . gate^T) * (x . up^T), [rows, weight rows / 2].  ``short_tiles`` keeps blocks of 128
    rows even when there are more (for measurements)."""
    _cuda(x, weight)
    rows, k = x.shape
    n = weight.shape[0]
    assert weight.shape[1] == k and x.dtype == weight.dtype == torch.bfloat16
    y = torch.empty((rows, n // 2 if swiglu else n), dtype=torch.bfloat16, device=x.device)
    if rows == 0:
        return y
    global tcgen05_calls
    tcgen05_calls += 1
    _check(lib().tllm_gemm_tcgen05(_p(x), _p(weight), _p(y), rows, n, k, int(swiglu) | (2 if short_tiles else 0) | (4 if interleaved else 0),
                                   _p(error_word(x.device)), _stream()), "gemm_tcgen05")
    return y


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """y[T, N] = x[T, K] . weight[N, K]^T with float32 accumulation.  A weight kept in
    float32 is multiplied in float32 whatever the activations are stored in."""
    if not x.is_cuda:
        raise KernelError("linear takes CUDA tensors")
    want = out_dtype or x.dtype
    if weight.dtype == torch.float32:
        if torch.backends.cuda.matmul.allow_tf32 or torch.get_float32_matmul_precision() != "highest":
            raise KernelError("float32 products need the reduced-precision matrix modes off")
        y = torch.mm(cast(x, torch.float32), weight.t())
        return y if want == torch.float32 else cast(y, want)
    if x.dtype != weight.dtype:
        x = cast(x, weight.dtype)
    rows, k = x.shape
    if weight.dtype == torch.bfloat16 and 0 < rows <= SKINNY_MAX_ROWS and k % 8 == 0 \
            and x.is_contiguous() and weight.is_contiguous() and want in _DT:
        return gemm_skinny(x, weight, want)
    if want == torch.bfloat16 and tcgen05_pays(rows, weight.shape[0], k, weight.dtype) \
            and x.is_contiguous() and weight.is_contiguous():
        return gemm_tcgen05(x, weight)
    if want == weight.dtype:
        return torch.mm(x, weight.t())
    return torch.mm(x, weight.t(), out_dtype=want)


def gemm_skinny_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """silu(x . Wg^T) * (x . Wu^T) for at most 16 bfloat16 rows as one weight-streaming kernel;
    ``w_gate_up`` holds the rows of Wg and Wu interleaved by eight (``interleave_gate_up``)."""
    _cuda(x, w_gate_up)
    rows, k = x.shape
    inter = w_gate_up.shape[0] // 2
    act = torch.empty((rows, inter), dtype=torch.bfloat16, device=x.device)
    _check(lib().tllm_gemm_skinny_swiglu(_p(x), _p(w_gate_up), _p(act), rows, inter, k, _stream()), "gemm_skinny_swiglu")
    return act


def linear_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, out_dtype: torch.dtype,
                  interleaved: bool = False) -> torch.Tensor:
    """silu(x . Wg^T) * (x . Wu^T) for w_gate_up = [Wg; Wu], or with the rows of Wg and Wu
    interleaved by eight (``interleave_gate_up``).  With enough bfloat16 rows the product and the
    activation are one tcgen05 kernel, with few rows and interleaved weights one weight-streaming
    kernel; otherwise the product is followed by the SwiGLU kernel."""
    rows, k = x.shape
    inter = w_gate_up.shape[0] // 2
    plain = x.dtype == w_gate_up.dtype == out_dtype == torch.bfloat16 and x.is_contiguous() \
        and w_gate_up.is_contiguous()
    if plain and tcgen05_pays(rows, inter, k, w_gate_up.dtype, col_tile=128):
        return gemm_tcgen05(x, w_gate_up, swiglu=True, interleaved=interleaved)
    if plain and interleaved and 0 < rows <= SKINNY_MAX_ROWS and k % 8 == 0:
        return gemm_skinny_swiglu(x, w_gate_up)
    gate_up = linear(x, w_gate_up, out_dtype=out_dtype)
    act = torch.empty((rows, inter), dtype=out_dtype, device=x.device)
    return swiglu(gate_up, act, interleaved)
