"""The allocation-free decode entry point against the regular one.

pkv_decode_attn_noalloc serves hosts that may not allocate device memory (they are handed inputs and
outputs only), so the split partials live in a fixed array inside the library. This test calls it
through the C ABI and compares with pkv_decode_attn + pkv_merge on caller-owned scratch, twice in a
row with different queries and split counts, so that whatever the first call left in the built-in
array would show up in the second. It is collected last on purpose: a failure here must not hide
the result of any other test.
"""
import ctypes

import pytest
import torch

from phasorkv_b200 import _lib

from helpers import Scenario, rel

pytestmark = pytest.mark.gpu


def _noalloc(sc, ws, n_split, out):
    L = sc.pk._layer()
    return _lib.load().pkv_decode_attn_noalloc(ctypes.byref(L), ctypes.byref(sc.cache.c), _lib.ptr(ws.qop),
                                               _lib.ptr(sc.cache.page_table), sc.cache.max_pages,
                                               _lib.ptr(sc.cache.seqlens), sc.B, n_split, _lib.ptr(out),
                                               _lib.ptr(ws.status), _lib.current_stream())


def test_noalloc_matches_regular_entry_point_twice():
    sc = Scenario("cfg2", seqlens=(900, 0, 257, 128), gain=64.0, pos0=20000)
    gen = torch.Generator().manual_seed(77)
    for call, n_split in enumerate((3, 5)):
        q = torch.randn(sc.q.shape, generator=gen).cuda()
        ws = sc.pk.workspace(sc.B, n_split)
        sc.pk.absorb_step(q, sc.qpos.cuda(), ws, operand=True)
        sc.pk.attend_step(sc.cache, ws, simt=False)
        sc.pk.merge_step(ws)
        want = ws.out.clone()
        out = torch.full_like(want, float("nan"))
        _lib.check(_noalloc(sc, ws, n_split, out), "pkv_decode_attn_noalloc")
        torch.cuda.synchronize()
        assert int(ws.status.abs().sum()) == 0
        assert torch.isfinite(out).all(), f"call {call}"
        assert rel(out.cpu(), want.cpu()) < 2e-3, f"call {call}"
        assert float(out[1].abs().max()) == 0.0           # the empty sequence attends to nothing


def test_noalloc_rejects_requests_beyond_its_scratch():
    sc = Scenario("cfg2", seqlens=(130,))
    ws = sc.pk.workspace(sc.B, 1)
    sc.pk.absorb_step(sc.q.cuda(), sc.qpos.cuda(), ws, operand=True)
    out = torch.zeros((1, 32, 128), device="cuda")
    assert _noalloc(sc, ws, _lib.NOALLOC_MAX_PARTS + 1, out) == -2
    assert float(out.abs().max()) == 0.0
