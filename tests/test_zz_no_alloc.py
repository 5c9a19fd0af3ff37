"""kvb_flash_decode_static, the decode-attention entry point that brings its own scratch.

It exists for callers that cannot allocate device memory - a process that has given every free
byte to its key/value pool, or a host program whose memory plan belongs to someone else - and so
it is called here the way such a caller would: through its exported C symbol, with nothing but
pointers to inputs and outputs.  Its result must equal the regular entry point's (which is handed
scratch by the caller) on two calls in a row, the second of which finds the first call's leftovers
in the shared array.  The file sorts last on purpose: if it fails, every other test has already run.
"""
import ctypes

import pytest
import torch

from helpers import assert_close, batch_to, clone_kv, paged_scenario
from torch_kernels import TorchKernels

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ERR_STATIC_SCRATCH = -5


def _library(head_dim):
    from kvcache_b200.kernels import build
    lib = build.load_module("attention_flash", f"d{head_dim}", [f"-DKVB_HEAD_DIM={head_dim}"])
    p, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.kvb_flash_decode_static.argtypes = [p, p, p, p, p, i, p, i, p, p, p, i, i, i, i, i, f, p]
    lib.kvb_flash_decode_static.restype = i
    lib.kvb_flash_decode.argtypes = [p, p, p, p, p, i, p, i, p, p, p, p, p, i, i, i, i, i, f, p]
    lib.kvb_flash_decode.restype = i
    return lib


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("head_dim", [64, 128])
def test_static_scratch_entry_point_matches_the_regular_one(head_dim):
    lib = _library(head_dim)
    Hq, Hkv, page = 8, 2, 16
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # The second call has fewer items and fewer splits than the first: its partial results and tickets lie over what
    # the first call left behind in another layout.
    for call, segments in enumerate([[(3000, 1), (700, 1), (64, 1), (0, 1)], [(1500, 1), (2999, 1), (5, 1)]]):
        nsplit = 8 if call == 0 else 4
        batch, kv = paged_scenario(segments, num_kv_heads=Hkv, head_dim=head_dim, page_size=page, dtype=torch.bfloat16,
                                   device="cpu", seed=30 + call)
        q = torch.randn(batch.num_tokens, Hq * head_dim, generator=torch.Generator().manual_seed(40 + call)).to(torch.bfloat16)
        want = torch.empty_like(q)
        TorchKernels(wide=True).paged_attention(q, batch, kv, want, Hq, head_dim ** -0.5)
        b, c, qd = batch_to(batch, DEV), clone_kv(kv, DEV), q.to(DEV)
        n = batch.num_segments
        common_head = [_ptr(c.k_pages), _ptr(c.v_pages), _ptr(c.block_table), c.block_table.shape[1], _ptr(b.plans["paged_attention"].arrays["decode_items"]), n,
                       _ptr(b.seg_q_start), _ptr(b.seg_q_len), _ptr(b.seg_kv_len)]
        common_tail = [Hq, Hkv, page, 0, nsplit, head_dim ** -0.5, stream]
        regular = torch.full_like(qd, float("nan"))
        scratch = torch.empty(n * Hkv * nsplit * 16 * (head_dim + 2), dtype=torch.float32, device=DEV)
        tickets = torch.zeros(n * Hkv, dtype=torch.int32, device=DEV)
        assert lib.kvb_flash_decode(_ptr(qd), _ptr(regular), *common_head, _ptr(scratch), _ptr(tickets), *common_tail) == 0
        static = torch.full_like(qd, float("nan"))
        assert lib.kvb_flash_decode_static(_ptr(qd), _ptr(static), *common_head, *common_tail) == 0
        torch.cuda.synchronize()
        assert torch.equal(static, regular), f"call {call}: the two entry points disagree"
        assert_close(static, want, 1e-2, f"call {call}")


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    lib = _library(64)
    null = ctypes.c_void_p(0)
    # 4000 items x 8 kv heads x 32 splits would need gigabytes of partial results: refused before any launch.
    code = lib.kvb_flash_decode_static(null, null, null, null, null, 1, null, 4000, null, null, null, 64, 8, 16, 0, 32,
                                       ctypes.c_float(0.125), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert code == ERR_STATIC_SCRATCH
    torch.cuda.synchronize()
