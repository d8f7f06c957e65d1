"""Quantised V pages (per-token low-bit tiers, phasorkv/kernels/nvfp4.py:58-67): the CUDA quantiser is bit-exact
against the reference's vectors, and decode attention over such pages meets the oracle on the dequantised
values within the tolerance of the attention output (2e-3 relative)."""
import os

import numpy as np
import pytest
import torch

from oracle import phasor_oracle as po
from phasorkv_b200 import _lib
from phasorkv_b200.latent import PagedLatentCache

from conftest import GOLDEN
from helpers import Scenario, rel

pytestmark = pytest.mark.gpu

OUT_TOL = 2e-3


@pytest.mark.parametrize("bits", [3, 2])
def test_vq_quantiser_matches_reference_golden_vectors(bits):
    g = np.load(os.path.join(GOLDEN, "v_tiers.npz"))
    x = torch.from_numpy(g["x"])                                        # [n, 128], bf16-exact values
    n = x.shape[0]
    cache = PagedLatentCache(256, 1, 128, 1, n, "cuda", v_bits=bits)
    order = torch.randperm(n, generator=torch.Generator().manual_seed(1)).to(torch.int32).cuda()     # scattered rows of the page
    slots = cache.slots(torch.zeros_like(order), order)
    cache.write_v(x.view(n, 1, 128), slots)
    rows, codes, scales = cache.read_vq(slots)
    assert np.array_equal(codes[:, 0].cpu().numpy(), g[f"codes{bits}"])
    assert np.array_equal(scales[:, 0].cpu().view(torch.int16).numpy(), g[f"scale{bits}"])
    assert np.array_equal(rows[:, 0].cpu().numpy(), g[f"xhat{bits}"])


@pytest.mark.parametrize("config,bits,seqlens,n_split,n_kv", [
    ("cfg2", 3, (1, 15, 129, 300), 2, None), ("cfg2", 2, (513, 0, 77), 3, None), ("cfg3", 3, (260, 128), 1, None),
    ("cfg5", 3, (300, 127), 2, None), ("cfg2", 3, (1400,), 4, None),
    ("cfg2", 3, (300, 127, 1), 2, 4), ("cfg2", 2, (1400,), 3, 4)])            # the last two: 8 query heads per kv head
def test_vq_decode_against_oracle(config, bits, seqlens, n_split, n_kv):
    sc = Scenario(config, seqlens=seqlens, gain=16.0, pos0=9000, v_bits=bits, n_kv=n_kv)
    ws = sc.pk.workspace(sc.B, n_split)
    sc.pk.absorb_step(sc.q.cuda(), sc.qpos.cuda(), ws)
    sc.pk.attend_step(sc.cache, ws, out=ws.out, after_absorb=True)
    torch.cuda.synchronize()
    assert int(ws.status.abs().sum()) == 0
    for b, T in enumerate(sc.seqlens):
        if T == 0:
            assert float(ws.out[b].abs().max()) == 0.0
            continue
        # what the pages hold is exactly the reference's quantisation of the bf16 value rows
        rows, codes, scales = sc.cache.read_vq(sc.slots_of(b))
        c_ref, s_ref, hat_ref = po.quantize_per_token(sc.v[b].to(torch.bfloat16).float(), bits)
        assert torch.equal(codes.cpu(), c_ref) and torch.equal(scales.cpu(), s_ref) and torch.equal(rows.cpu(), hat_ref)
        _, _, O_ref = sc.oracle_scores_and_output(b, sc.dequantised(b), V=hat_ref)
        assert rel(ws.out[b].cpu(), O_ref) < OUT_TOL, (b, T)


def test_vq_cache_refuses_the_cuda_core_kernel():
    sc = Scenario("cfg2", seqlens=(130,), v_bits=3)
    ws = sc.pk.workspace(sc.B, 1)
    sc.pk.absorb_step(sc.q.cuda(), sc.qpos.cuda(), ws, operand=False)
    with pytest.raises(_lib.PhasorKVError, match="unsupported"):
        sc.pk.attend_step(sc.cache, ws, simt=True)


def test_vq_logits_dump_and_packed_triples():
    """With quantised V the attention still dumps its logits (the softmax reads the scores from tensor memory in
    chunks there) and hands out merged (o, m, l) triples for token sharding: both against the oracle."""
    sc = Scenario("cfg2", seqlens=(700, 129), gain=16.0, pos0=5000, v_bits=3)
    ws = sc.pk.workspace(sc.B, 3)
    S = torch.zeros((sc.B, sc.spec.n_q, max(sc.seqlens)), device="cuda")
    sc.pk.absorb_step(sc.q.cuda(), sc.qpos.cuda(), ws)
    sc.pk.attend_step(sc.cache, ws, scores_out=S, packed_out=ws.packed, after_absorb=True)
    out = torch.empty_like(ws.out)
    sc.pk.merge_gathered(ws.packed[None].contiguous(), out)
    torch.cuda.synchronize()
    assert int(ws.status.abs().sum()) == 0
    for b, T in enumerate(sc.seqlens):
        rows, _, _ = sc.cache.read_vq(sc.slots_of(b))
        _, S_ref, O_ref = sc.oracle_scores_and_output(b, sc.dequantised(b), V=rows.cpu())
        assert rel(S[b, :, :T].cpu(), S_ref) < 1e-3, (b, T)
        assert rel(out[b].cpu(), O_ref) < OUT_TOL, (b, T)


@pytest.mark.parametrize("config,bits", [("cfg2", 3), ("cfg5", 2), ("cfg3", 3)])
def test_prologue_quantises_the_value_rows_like_the_writer(config, bits):
    """The step prologue stores the newest tokens' value rows into quantised V pages itself: same codes and
    scales as the stand-alone writer (cfg3, R = 120, goes through the entry point's separate launches)."""
    sc = Scenario(config, seqlens=(5,), pos0=700, v_bits=bits)
    pk, n = sc.pk, 5
    x, v = sc.x[0].cuda(), sc.v[0].cuda()
    wpos = sc.pos[0].to(torch.int32).cuda()
    slots = sc.slots_of(0)
    q = torch.randn((n, sc.spec.n_q, sc.spec.head_dim), generator=torch.Generator().manual_seed(3)).cuda()
    caches = []
    for fused in (False, True):
        cache = pk.new_cache(1, n, v_bits=bits)
        ws = pk.workspace(n, 1)
        if fused:
            pk.prologue_step(cache, x, wpos, slots, q, (wpos + 1).contiguous(), ws, v=v)
        else:
            pk.write_paged(cache, x, wpos, slots, v=v, scratch=ws.wscratch)
        torch.cuda.synchronize()
        caches.append(cache)
    a, b = caches[0].read_vq(slots), caches[1].read_vq(slots)
    assert float(a[0].abs().max()) > 0
    for u, w in zip(a, b):
        assert torch.equal(u, w)
    assert torch.equal(caches[0].vq, caches[1].vq)
