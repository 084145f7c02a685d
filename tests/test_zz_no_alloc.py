"""The entry point for callers that cannot allocate device memory
(``tllm_paged_attention_decode_noalloc``, declared in csrc/tllm_noalloc.h): an embedding
program whose device memory was fixed at start-up, a plug-in inside a process that owns
all of it, a real-time loop.  It is called here the way such a caller would, through the
symbol the shared library exports, with raw pointers, and must give what the ordinary
entry point gives with scratch brought by the caller, to the bit (the same kernels add the
same partial results in the same order); twice in a row, the second time with sizes that use
less of the library's one scratch array than the first, so that it runs among the first
call's leftovers.

This file is named so that pytest collects it last.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

SCRATCH_FLOATS = 4 * 1024 * 1024


@pytest.fixture(scope="module")
def library():
    from tiny_llm_infer_b200 import ops
    h = ops.lib()
    vp, i32, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn = h.tllm_paged_attention_decode_noalloc
    fn.argtypes = [vp, vp, vp, vp, vp, i32, vp, i32, i32, i32, i32, i32, i32, f32, i32, vp, vp]
    fn.restype = i32
    h.tllm_noalloc_scratch_needed.argtypes = [i32, i32, i32, i32]
    h.tllm_noalloc_scratch_needed.restype = ctypes.c_longlong
    return h, ops


def make_case(seed, rows, nh, nkv, hd, ps, ctx_max):
    """Random queries and a filled paged cache for `rows` single-token rows."""
    g = torch.Generator().manual_seed(seed)
    max_pages = -(-ctx_max // ps)
    num_pages = rows * max_pages + 3
    table = torch.randperm(num_pages, generator=g)[:rows * max_pages].view(rows, max_pages).to(torch.int32)
    cache = (torch.randn((num_pages, 2, nkv, ps, hd), generator=g) * 0.7).to(torch.bfloat16)
    q = torch.randn((rows + 1, nh * hd), generator=g).to(torch.bfloat16)
    pos = torch.randint(0, ctx_max, (rows + 1,), generator=g).to(torch.int32)
    pos[0] = ctx_max - 1
    slot = torch.arange(rows + 1, dtype=torch.int32)
    slot[rows] = -1                                           # a padding row
    return [t.cuda().contiguous() for t in (q, cache, pos, slot, table)]


@pytest.mark.parametrize("first,second", [
    (dict(rows=8, nh=32, nkv=8, hd=128, ps=16, ctx=900, splits=7, window=0),
     dict(rows=3, nh=6, nkv=2, hd=64, ps=32, ctx=300, splits=4, window=50)),
])
def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row(library, first, second):
    h, ops = library
    stream = torch.cuda.current_stream().cuda_stream
    for call, c in enumerate((first, second)):
        q, cache, pos, slot, table = make_case(40 + call, c["rows"], c["nh"], c["nkv"], c["hd"], c["ps"], c["ctx"])
        n_rows = c["rows"] + 1
        scale = 1.0 / math.sqrt(c["hd"])
        want = torch.full_like(q, 7.0)
        ops.paged_attention_decode(q, cache, pos, slot, None, n_rows, table, c["ps"], c["nh"], c["nkv"], c["hd"],
                                   c["window"], scale, want, c["ctx"], splits=c["splits"])
        need = h.tllm_noalloc_scratch_needed(n_rows, c["nh"], c["hd"], c["splits"])
        assert 0 < need <= SCRATCH_FLOATS
        got = torch.full_like(q, -7.0)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = h.tllm_paged_attention_decode_noalloc(
            q.data_ptr(), cache.data_ptr(), pos.data_ptr(), slot.data_ptr(), None, n_rows, table.data_ptr(),
            table.shape[1], c["ps"], c["nh"], c["nkv"], c["hd"], c["window"], scale, c["splits"],
            got.data_ptr(), stream)
        assert rc == 0, h.tllm_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before          # nothing was taken from torch's allocator either
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, want), (call, (got.float() - want.float()).abs().max().item())
        if call == 1:
            assert need < first_need                            # inside what the first call left behind
        first_need = need
        assert (got[-1] == 0).all()                             # the padding row


def test_no_alloc_entry_point_refuses_what_does_not_fit(library):
    h, _ = library
    q, cache, pos, slot, table = make_case(50, 4, 8, 2, 128, 16, 64)
    out = torch.zeros_like(q)
    stream = torch.cuda.current_stream().cuda_stream
    assert h.tllm_noalloc_scratch_needed(512, 64, 128, 64) > SCRATCH_FLOATS
    rc = h.tllm_paged_attention_decode_noalloc(
        q.data_ptr(), cache.data_ptr(), pos.data_ptr(), slot.data_ptr(), None, 512, table.data_ptr(),
        table.shape[1], 16, 64, 8, 128, 0, 1.0, 64, out.data_ptr(), stream)
    assert rc == -1
    text = h.tllm_last_error().decode()
    assert "exceed" in text and "scratch" in text
    torch.cuda.synchronize()
    assert (out == 0).all()                                     # nothing ran
