"""Parity of the CUDA path (through the C ABI) with the CPU oracle and the reference's golden vectors.

Tolerances (from the task statement): NVFP4 codes and scales bit-exact when fed the reference's fp32
latent; logits within 1e-3 and attention outputs within 2e-3 relative (Frobenius norm, per
sequence) of fp32 scoring on the dequantised cache.
"""
import os

import numpy as np
import pytest
import torch

from oracle import c_oracle
from oracle import phasor_oracle as po
from phasorkv_b200 import synth
from phasorkv_b200.latent import PagedLatentCache, PhasorKey

from conftest import GOLDEN
from helpers import Scenario, fac_from_golden, rel

pytestmark = pytest.mark.gpu

LOGIT_TOL = 1e-3
OUT_TOL = 2e-3


def _golden(name):
    return np.load(os.path.join(GOLDEN, name))


# ------------------------------------------------------------------------------------------------
# NVFP4 quantiser: bit-exact
# ------------------------------------------------------------------------------------------------

def _quantise_and_read(rows, second, order=None):
    n, W = rows.shape
    cache = PagedLatentCache(W, 8, 128, 1, max(n, 1), "cuda", with_v=False)
    lp = torch.arange(n, dtype=torch.int32, device="cuda") if order is None else order.cuda()
    slots = cache.slots(torch.zeros_like(lp), lp)
    cache.quantize_rows(rows.cuda(), slots, second)
    xhat, codes, scales = cache.read(slots, second)
    return xhat.cpu(), codes.cpu(), scales.cpu()


def test_quantiser_matches_reference_golden_vectors():
    g = _golden("nvfp4_cases.npz")
    x = torch.from_numpy(g["x"])
    xhat, codes, scales = _quantise_and_read(x, float(g["second"][0]))
    assert np.array_equal(codes.numpy(), g["packed"])
    assert np.array_equal(scales.numpy(), g["scales"])
    assert np.array_equal(xhat.numpy(), g["xhat"])


@pytest.mark.parametrize("config,T", [("cfg2", 700), ("cfg3", 300), ("cfg5", 260)])
def test_quantiser_bit_exact_on_oracle_latent(config, T):
    spec = synth.make_layer(config, 1)
    opk = po.PhasorKeyOracle.from_spec(spec)
    gen = torch.Generator().manual_seed(21)
    x = synth.make_hidden(gen, T)
    rows = opk.write(x, po.rope_phasors(spec.inv_freq, torch.arange(T) + 32000))
    second = po.nv_static_second(rows.var(0))
    ref_codes, ref_scales, ref_hat = po.nvfp4_quantize(rows, second)
    order = torch.randperm(T, generator=gen).to(torch.int32)            # scattered slots, page boundaries
    xhat, codes, scales = _quantise_and_read(rows, float(second), order)
    assert torch.equal(codes, po.pack_nibbles(ref_codes))
    assert torch.equal(scales, ref_scales)
    assert torch.equal(xhat, ref_hat)
    c_codes, c_scales, _ = c_oracle.nvfp4_quantize(rows.numpy(), float(second))
    assert np.array_equal(c_codes, ref_codes.numpy()) and np.array_equal(c_scales, ref_scales.numpy())


def test_quantiser_scale_round_up_matches_reference_golden_vectors():
    """The reference's PHASORKV_SCALE_UP=1 mode (block scales rounded up): bit-exact against vectors it
    produced with that switch, through the quantiser entry point and through the fused write kernels."""
    from phasorkv_b200 import _lib
    g = _golden("nvfp4_cases_scale_up.npz")
    x = torch.from_numpy(g["x"])
    lib = _lib.load()
    try:
        _lib.check(lib.pkv_set_scale_round_up(1), "pkv_set_scale_round_up")
        xhat, codes, scales = _quantise_and_read(x, float(g["second"][0]))
        assert np.array_equal(codes.numpy(), g["packed"])
        assert np.array_equal(scales.numpy(), g["scales"])
        assert np.array_equal(xhat.numpy(), g["xhat"])
        # the write kernels (CUDA-core, tensor-core, decode-time, one-launch prologue) round their scales the same way:
        # each stores what the quantiser entry point stores for the rows the kernel itself reports
        sc = Scenario("cfg2", seqlens=(200,), pos0=100)
        for dt, n in ((torch.float32, 200), (torch.bfloat16, 200), (torch.bfloat16, 16)):
            xs = sc.x[0][:n].cuda().to(dt)
            pos = sc.pos[0][:n].to(torch.int32).cuda()
            slots = sc.slots_of(0)[:n]
            rows = torch.empty((n, sc.spec.cache_width), device="cuda")
            c1, c2 = sc.pk.new_cache(1, 200), sc.pk.new_cache(1, 200)
            sc.pk.write_paged(c1, xs, pos, slots, latent_out=rows, scratch=sc.pk.write_scratch(n) if n <= 64 else None)
            c2.quantize_rows(rows, slots, sc.second)
            assert torch.equal(c1.latent, c2.latent), (dt, n)
        ws = sc.pk.workspace(16, 1)
        c1, c2 = sc.pk.new_cache(1, 200), sc.pk.new_cache(1, 200)
        sc.pk.prologue_step(c1, xs, pos, slots, None, None, ws, latent_out=rows)
        c2.quantize_rows(rows, slots, sc.second)
        assert torch.equal(c1.latent, c2.latent)
        up = c2.latent.clone()
    finally:
        _lib.check(lib.pkv_set_scale_round_up(0), "pkv_set_scale_round_up")
    c3 = sc.pk.new_cache(1, 200)
    c3.quantize_rows(rows, slots, sc.second)
    assert not torch.equal(c3.latent, up)                      # the default (round to nearest) stores other scales


@pytest.mark.parametrize("second", [1e-3, 1.0, 37.5])
def test_quantiser_bit_exact_over_wide_magnitudes(second):
    """Blocks whose magnitudes span 2^-24 .. 2^14 around the tensor scale (scale saturation at 448,
    subnormal and zero block scales), blocks of exact zeros, and values that sit exactly on the E2M1
    rounding boundaries of their block: codes, scales and dequantised values equal the oracle's bits."""
    g = torch.Generator().manual_seed(int(second * 1000) + 3)
    n, W = 768, 256
    mag = torch.exp2(torch.rand((n, W // 16, 1), generator=g) * 38.0 - 24.0) * second
    x = (torch.randn((n, W // 16, 16), generator=g) * mag).reshape(n, W)
    x[::7, 32:48] = 0.0                                                   # zero blocks
    # boundary rows: block maximum 6 * s with s a power of two, the other entries on the midpoints .25 .75 1.25 ... 5
    mids = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
    for r in range(0, 64):
        s_blk = second * 2.0 ** (r % 12 - 6)
        x[r, 64:80] = mids * s_blk
    ref_codes, ref_scales, ref_hat = po.nvfp4_quantize(x, torch.tensor([second]))
    xhat, codes, scales = _quantise_and_read(x, float(second))
    assert torch.equal(codes, po.pack_nibbles(ref_codes))
    assert torch.equal(scales, ref_scales)
    assert torch.equal(xhat, ref_hat)
    c_codes, c_scales, _ = c_oracle.nvfp4_quantize(x.numpy(), float(second))
    assert np.array_equal(c_codes, ref_codes.numpy()) and np.array_equal(c_scales, ref_scales.numpy())


def test_quantiser_with_one_scale_per_tier_matches_reference():
    """Tiers: every 16-aligned span of the row has its own static tensor scale (phasorkv/quant.py:119-124 applied per
    span, as phasorkv/kernels/latent_attn.py:255-262 writes its cache). Bit-exact against the reference's
    span-by-span quantisation, and the tiered read-back returns its x_hat."""
    g = _golden("nvfp4_tiers.npz")
    x = torch.from_numpy(g["x"])
    n, W = x.shape
    sb = torch.zeros(W // 16)
    for (lo, hi), sec in zip(g["spans"].tolist(), g["seconds"].tolist()):
        sb[lo // 16:hi // 16] = sec
    cache = PagedLatentCache(W, 8, 128, 1, n, "cuda", with_v=False)
    lp = torch.arange(n, dtype=torch.int32, device="cuda")
    slots = cache.slots(torch.zeros_like(lp), lp)
    cache.quantize_rows(x.cuda(), slots, sb)
    xhat, codes, scales = cache.read(slots, sb)
    assert np.array_equal(codes.cpu().numpy(), g["packed"]) and np.array_equal(scales.cpu().numpy(), g["scales"])
    assert np.array_equal(xhat.cpu().numpy(), g["xhat"])


@pytest.mark.parametrize("x_dtype", [torch.float32, torch.bfloat16])
def test_tiered_tensor_scales_through_write_and_decode(x_dtype):
    """A layer whose energy-sorted latent falls by orders of magnitude along the row, with one static scale per
    64-column span: every write kernel stores the reference quantiser's bits of its own rows under the span's
    scale, and the decode (the query carries second_tier / second per block) meets fp32 scoring on the
    dequantised cache. With the single scale of the widest channel the last span's blocks underflow to zero."""
    spec = synth.make_layer("cfg2", 2)
    decay = torch.exp(-torch.arange(spec.R, dtype=torch.float32) / 10.0)           # complex dim k shrinks like e^{-k/10}
    pk = PhasorKey.from_factors(spec.A, spec.B * decay[:, None], spec.freq, spec.n_q, spec.n_kv, spec.head_dim, spec.inv_freq)
    opk = po.PhasorKeyOracle(spec.A, spec.B * decay[:, None], spec.freq, spec.n_q, spec.n_kv, spec.head_dim)
    g = torch.Generator().manual_seed(12)
    T, pos0 = 333, 2000
    x = synth.make_hidden(g, T, 4096).to(x_dtype)
    v = synth.make_values(g, T, spec.n_kv, spec.head_dim)
    q = synth.make_query(g, 1, spec.n_q, spec.head_dim)
    pos = torch.arange(T) + pos0
    rows_ref = opk.write(x.float(), po.rope_phasors(spec.inv_freq, pos))
    pk.calibrate_second(rows_ref, span=64)
    sb = pk.second_arg()
    assert torch.is_tensor(sb) and float(sb.max() / sb.min()) > 100.0
    cache = pk.new_cache(1, T)
    lp = torch.arange(T, dtype=torch.int32, device="cuda")
    slots = cache.slots(torch.zeros_like(lp), lp)
    out = torch.empty((T, 256), device="cuda")
    pk.write_paged(cache, x.cuda(), pos.to(torch.int32).cuda(), slots, v=v.cuda(), latent_out=out)       # chunk write kernels
    assert rel(out.cpu(), rows_ref) < (5e-6 if x_dtype == torch.float32 else 3e-5)
    hat, codes, scales = cache.read(slots, sb)
    o_codes, o_scales, o_hat = po.nvfp4_quantize(out.cpu(), sb)
    assert torch.equal(codes.cpu(), po.pack_nibbles(o_codes)) and torch.equal(scales.cpu(), o_scales) and torch.equal(hat.cpu(), o_hat)
    assert float(hat[:, 112:128].abs().max()) > 0                                   # the weakest span survives with its own scale
    _, _, flat = po.nvfp4_quantize(out.cpu(), torch.tensor([pk.second]))
    assert float(flat[:, 112:128].abs().max()) == 0.0                               # ... and would not with the row's one scale
    # newest token through the prologue (small-batch and general path use the same per-block scales)
    cache.seqlens.fill_(T)
    ws = pk.workspace(1, 2)
    qpos = torch.tensor([T + pos0], dtype=torch.int32, device="cuda")
    x_new = synth.make_hidden(g, 1, 4096).to(x_dtype).cuda()
    row_new = torch.empty((1, 256), device="cuda")
    pk.prologue_step(cache, x_new, qpos - 1, slots[-1:], q.cuda(), qpos, ws, v=v[-1:].cuda(), latent_out=row_new)
    hat1, c1, s1 = cache.read(slots[-1:], sb)
    n_codes, n_scales, _ = po.nvfp4_quantize(row_new.cpu(), sb)
    assert torch.equal(c1.cpu(), po.pack_nibbles(n_codes)) and torch.equal(s1.cpu(), n_scales)
    Sd = torch.zeros((1, spec.n_q, T), device="cuda")
    pk.attend_step(cache, ws, scores_out=Sd, out=ws.out, after_prologue=True)
    torch.cuda.synchronize()
    hat, _, _ = cache.read(slots, sb)
    qa = opk.absorb(q[0][:, None, :], po.rope_phasors(spec.inv_freq, torch.tensor([T + pos0])))[:, 0]
    S_ref = opk.scores(qa, hat.cpu())
    assert rel(Sd[0].cpu(), S_ref) < LOGIT_TOL
    assert rel(ws.out[0].cpu(), po.attend(S_ref, v, spec.n_kv, spec.head_dim)) < OUT_TOL
    # the reference-surface absorb stays the reference's (no tier ratio inside)
    assert rel(pk.absorb(q[0][:, None, :], po.rope_phasors(spec.inv_freq, torch.tensor([T + pos0])))[:, 0].cpu(), qa) < 2e-6


def test_quantiser_empty_and_bad_slots():
    cache = PagedLatentCache(256, 8, 128, 1, 128, "cuda", with_v=False)
    cache.quantize_rows(torch.zeros(0, 256), torch.zeros(0, dtype=torch.int32, device="cuda"), 1.0)
    before = cache.latent.clone()
    bad = torch.tensor([-1, 128, 99999], dtype=torch.int32, device="cuda")       # all outside the pool
    cache.quantize_rows(torch.ones(3, 256), bad, 1.0)
    torch.cuda.synchronize()
    assert torch.equal(before, cache.latent)


# ------------------------------------------------------------------------------------------------
# write / absorb / scores behind the reference's PhasorKey interface
# ------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("tag", ["freq", "band"])
def test_phasorkey_interface_against_reference_vectors(tag):
    g = _golden("phasorkey_injected.npz")
    D, n_q, n_kv, d = (int(v) for v in g["dims"])
    t = lambda k: torch.from_numpy(g[f"{tag}_{k}"]) if f"{tag}_{k}" in g else None
    pk = PhasorKey.from_factors(t("A"), t("B"), t("freq"), n_q, n_kv, d, torch.from_numpy(g["inv_freq"]),
                                t("A_s"), t("B_s"), t("slow"))
    rows = pk.write(t("x"), t("ph_k")).cpu()
    qabs = pk.absorb(t("q"), t("ph_q")).cpu()
    assert rows.shape == t("rows").shape and qabs.shape == t("qabs").shape
    assert rel(rows, t("rows")) < 2e-6
    assert rel(qabs, t("qabs")) < 2e-6
    assert pk.cache_width == t("rows").shape[1]
    # positions instead of phasors: the kernel forms the angle in double like rope.py:29-32
    n = t("x").shape[0]
    out = torch.empty((n, pk.cache_width), device="cuda")
    pk.write_paged(None, t("x").cuda(), t("pos_k").to(torch.int32).cuda(), None, latent_out=out)
    assert rel(out.cpu(), t("rows")) < 2e-6


@pytest.mark.parametrize("tag", ["freq", "band"])
def test_rebuilt_keys_identity(tag):
    """Scores from the CUDA write and absorb equal 'keys rebuilt from W_hat, rotated by HF rotary'
    (README.md:75-77 of the reference) within the logit tolerance."""
    g = _golden("phasorkey_factorized.npz")
    D, n_q, n_kv, d = (int(v) for v in g["dims"])
    t = lambda k: torch.from_numpy(g[f"{tag}_{k}"]) if f"{tag}_{k}" in g else None
    pk = PhasorKey.from_factors(t("A"), t("B"), t("freq"), n_q, n_kv, d, torch.from_numpy(g["inv_freq"]),
                                t("A_s"), t("B_s"), t("slow") if f"{tag}_A_s" in g else None)
    rows = pk.write(torch.from_numpy(g["x"]).float(), torch.from_numpy(g["ph_k"]))
    qabs = pk.absorb(torch.from_numpy(g["q"]).float(), torch.from_numpy(g["ph_q"]))
    S = PhasorKey.scores(qabs, rows).cpu()                          # the reference's static call, exact fp32 product
    assert S.dtype == torch.float32
    assert rel(S, t("scores_hf")) < LOGIT_TOL
    assert rel(S, t("scores")) < 1e-5


@pytest.mark.parametrize("tag", ["freq", "band"])
def test_reference_call_sequence_on_a_factorization(tag):
    """The reference's own sequence, unchanged: ``pk = PhasorKey(fac, ranks, n_q)`` (no inv_freq), then
    ``PhasorKey.scores(pk.absorb(q, ph), pk.write(x, ph))`` -- in fp64, which the reference keeps
    (phasorkv/latent.py:63-64), it meets the reference's scores and the rebuilt-keys identity of its
    README.md:75-77 to 1e-13; in fp32 to 1e-5."""
    from phasorkv_b200._lib import PhasorKVError
    g = _golden("phasorkey_factorized.npz")
    fac, n_q = fac_from_golden(g, tag)
    pk = PhasorKey(fac, g[f"{tag}_ranks"].tolist(), n_q)
    t = lambda k: torch.from_numpy(g[k])
    x, q, ph_k, ph_q = t("x"), t("q"), t("ph_k"), t("ph_q")
    rows, qabs = pk.write(x, ph_k), pk.absorb(q, ph_q)
    assert rows.dtype == torch.float64 and qabs.dtype == torch.float64
    assert rel(rows.cpu(), t(f"{tag}_rows")) < 1e-13 and rel(qabs.cpu(), t(f"{tag}_qabs")) < 1e-13
    S = PhasorKey.scores(qabs, rows)
    assert S.dtype == torch.float64
    assert rel(S.cpu(), t(f"{tag}_scores")) < 1e-13
    assert rel(S.cpu(), t(f"{tag}_scores_hf")) < 1e-13
    S32 = PhasorKey.scores(pk.absorb(q.float(), ph_q), pk.write(x.float(), ph_k))
    assert S32.dtype == torch.float32 and rel(S32.cpu(), t(f"{tag}_scores")) < 1e-5
    # the calls that form phasors from positions say what they miss instead of rotating by zero
    with pytest.raises(PhasorKVError, match="inv_freq"):
        pk.write_paged(None, x.float().cuda(), t("pos_k").to(torch.int32).cuda(), None,
                       latent_out=torch.empty((x.shape[0], pk.cache_width), device="cuda"))
    pk.set_inv_freq(t("inv_freq"))
    out = torch.empty((x.shape[0], pk.cache_width), device="cuda")
    pk.write_paged(None, x.float().cuda(), t("pos_k").to(torch.int32).cuda(), None, latent_out=out)
    assert rel(out.cpu(), t(f"{tag}_rows")) < 2e-6


@pytest.mark.parametrize("config", ["cfg2", "cfg3", "cfg5"])
@pytest.mark.parametrize("x_dtype", [torch.float32, torch.bfloat16])
def test_fused_write_against_oracle(config, x_dtype):
    sc = Scenario(config, seqlens=(129, 70), pos0=32700, x_dtype=x_dtype)
    for b in range(sc.B):
        ref_codes, ref_scales, ref_hat = po.nvfp4_quantize(sc.rows_ref[b], torch.tensor([sc.second]))
        xhat, codes, scales = sc.cache.read(sc.slots_of(b), sc.second)
        got = po.unpack_nibbles(codes.cpu())
        # the projection is summed in a different order than the CPU matmul, so a value sitting on a
        # rounding boundary may land one step away: almost all codes and scales agree, all rows are close
        assert (got != ref_codes).float().mean() < 2e-3
        assert (scales.cpu() != ref_scales).float().mean() < 2e-3
        assert rel(xhat.cpu(), ref_hat) < 5e-3
        # ... and where a code differs it is the neighbouring E2M1 level, never further (signed level index)
        level = lambda c: torch.where((c & 8) != 0, -(c & 7).to(torch.int32), (c & 7).to(torch.int32))
        assert int((level(got) - level(ref_codes)).abs().max()) <= 1
        sb, rb = scales.cpu().to(torch.int32), ref_scales.to(torch.int32)
        assert int((sb - rb).abs().max()) <= 1                               # neighbouring E4M3 bytes at most
        out = torch.empty((sc.seqlens[b], sc.spec.cache_width), device="cuda")
        sc.pk.write_paged(sc.cache, sc.x[b].cuda(), sc.pos[b].to(torch.int32).cuda(), sc.slots_of(b), latent_out=out)
        # fp32 x: CUDA-core FMA chain; bf16 x: tensor cores, factors as three bf16 terms, fp32 accumulation in TMEM
        assert rel(out.cpu(), sc.rows_ref[b]) < (5e-6 if x_dtype == torch.float32 else 3e-5)
        # The stored bits are exactly the reference quantiser's bits of the fp32 rows the kernel itself reports:
        # the bit-exact quantiser (checked against the reference's vectors) fed with them gives the same bytes,
        # and so does the oracle. What differs from the oracle's write is only the summation order of x . B^T.
        _, codes2, scales2 = sc.cache.read(sc.slots_of(b), sc.second)
        _, q_codes, q_scales = _quantise_and_read(out, sc.second)
        assert torch.equal(codes2.cpu(), q_codes) and torch.equal(scales2.cpu(), q_scales)
        o_codes, o_scales, _ = po.nvfp4_quantize(out.cpu(), torch.tensor([sc.second]))
        assert torch.equal(codes2.cpu(), po.pack_nibbles(o_codes)) and torch.equal(scales2.cpu(), o_scales)


def test_absorb_batch_against_oracle():
    for config in ("cfg2", "cfg3", "cfg5"):
        sc = Scenario(config, seqlens=(5, 9, 1), pos0=131000)
        ws = sc.pk.workspace(sc.B, 1)
        sc.pk.absorb_step(sc.q.cuda(), sc.qpos.cuda(), ws, operand=False)
        for b in range(sc.B):
            qa, _, _ = sc.oracle_scores_and_output(b, sc.rows_ref[b])
            assert rel(ws.qabs[b].cpu(), qa) < 2e-6


# ------------------------------------------------------------------------------------------------
# decode attention
# ------------------------------------------------------------------------------------------------

def _check_decode(sc, n_split, simt, scores_tol=LOGIT_TOL, out_tol=OUT_TOL):
    Tmax = max(sc.seqlens)
    ws = sc.pk.workspace(sc.B, n_split)
    S = torch.zeros((sc.B, sc.spec.n_q, Tmax), device="cuda")
    sc.pk.absorb_step(sc.q.cuda(), sc.qpos.cuda(), ws, operand=not simt)
    sc.pk.attend_step(sc.cache, ws, simt=simt, scores_out=S, out=ws.out, after_absorb=True)   # attention + merge, one call
    fused = ws.out.clone()
    sc.pk.merge_step(ws)                                                       # the separate merge kernel
    torch.cuda.synchronize()
    assert int(ws.status.abs().sum()) == 0
    assert rel(fused.cpu(), ws.out.cpu()) < 1e-6 or float(ws.out.abs().max()) == 0.0
    for b, T in enumerate(sc.seqlens):
        if T == 0:
            assert float(ws.out[b].abs().max()) == 0.0
            continue
        _, S_ref, O_ref = sc.oracle_scores_and_output(b, sc.dequantised(b))
        assert rel(S[b, :, :T].cpu(), S_ref) < scores_tol, (b, T)
        assert rel(ws.out[b].cpu(), O_ref) < out_tol, (b, T)
    return ws


@pytest.mark.parametrize("T", [1, 15, 16, 17, 127, 128, 129, 1000])
def test_simt_decode_lengths(T):
    _check_decode(Scenario("cfg2", seqlens=(T,), pos0=4000), n_split=3, simt=True)


@pytest.mark.parametrize("config,gain", [("cfg2", 1.0), ("cfg2", 256.0), ("cfg3", 1.0), ("cfg3", 256.0), ("cfg5", 1.0),
                                         ("cfg5", 256.0)])
def test_simt_decode_ragged_batch(config, gain):
    """Ragged batch including an empty sequence; gain 256 makes the softmax peaked so that the
    running-max rescaling is exercised."""
    _check_decode(Scenario(config, seqlens=(513, 0, 77, 300), gain=gain, pos0=100000), n_split=4, simt=True)


def test_scores_only_mode_gives_log_sum_exp():
    sc = Scenario("cfg2", seqlens=(400, 130), gain=64.0)
    ws = sc.pk.workspace(sc.B, 2)
    sc.pk.absorb_step(sc.q.cuda(), sc.qpos.cuda(), ws, operand=False)
    sc.pk.attend_step(sc.cache, ws, simt=True, scores_only=True)
    sc.pk.merge_step(ws, normalise=False, packed=True)
    for b, T in enumerate(sc.seqlens):
        _, S_ref, _ = sc.oracle_scores_and_output(b, sc.dequantised(b))
        s2 = S_ref.double() * (po.LOG2E * sc.spec.head_dim ** -0.5)
        lse = torch.log2(torch.exp2(s2 - s2.amax(-1, keepdim=True)).sum(-1)) + s2.amax(-1)
        got = ws.packed[b, :, -2].double().cpu() + torch.log2(ws.packed[b, :, -1].double().cpu())
        assert torch.allclose(got, lse, atol=2e-3)


def test_scores_on_the_quantised_rows():
    sc = Scenario("cfg2", seqlens=(200,))
    qa, _, _ = sc.oracle_scores_and_output(0, sc.rows_ref[0])
    S = sc.pk.scores_nvfp4(qa[:, None, :], sc.rows_ref[0]).cpu()     # [H, 1, Tk], on the NVFP4 of the given rows
    _, _, hat = po.nvfp4_quantize(sc.rows_ref[0], torch.tensor([sc.second]))
    assert rel(S[:, 0], sc.opk.scores(qa, hat)) < LOGIT_TOL


def test_token_sharded_merge_equals_unsharded():
    """Sequence sharding as on several GPUs, emulated on one: each shard holds a contiguous token
    range in its own cache, emits a packed (o, m, l) triple, and the merge of the gathered triples
    equals attention over the whole sequence."""
    T, G = 1024, 4
    full = Scenario("cfg2", seqlens=(T, T // 2), gain=64.0, pos0=50000)
    ws_full = _check_decode(full, n_split=2, simt=True)
    gathered = torch.zeros((G, full.B, full.spec.n_q, full.spec.head_dim + 2), device="cuda")
    for r in range(G):
        lens = []
        shard_cache = None
        for b, Tb in enumerate(full.seqlens):
            lo, hi = r * Tb // G, (r + 1) * Tb // G
            lens.append(hi - lo)
        shard_cache = full.pk.new_cache(full.B, max(lens))
        for b, Tb in enumerate(full.seqlens):
            lo, hi = r * Tb // G, (r + 1) * Tb // G
            n = hi - lo
            seq = torch.full((n,), b, dtype=torch.int32, device="cuda")
            slots = shard_cache.slots(seq, torch.arange(n, dtype=torch.int32, device="cuda"))
            full.pk.write_paged(shard_cache, full.x[b][lo:hi].cuda(), full.pos[b][lo:hi].to(torch.int32).cuda(), slots,
                                v=full.v[b][lo:hi].cuda())
        shard_cache.seqlens.copy_(torch.tensor(lens, dtype=torch.int32))
        ws = full.pk.workspace(full.B, 2)
        full.pk.absorb_step(full.q.cuda(), full.qpos.cuda(), ws, operand=False)
        full.pk.attend_step(shard_cache, ws, simt=True)
        full.pk.merge_step(ws, normalise=False, packed=True)
        gathered[r] = ws.packed
    out = torch.empty_like(ws_full.out)
    full.pk.merge_gathered(gathered, out)
    assert rel(out.cpu(), ws_full.out.cpu()) < 1e-5


@pytest.mark.parametrize("config,n", [("cfg2", 16), ("cfg3", 5), ("cfg5", 64)])
def test_decode_time_write_path(config, n):
    """The small-batch write (projection spread over the GPU, staged through caller scratch) stores
    the same cache content as the one-CTA-per-64-tokens kernel, up to summation order."""
    sc = Scenario(config, seqlens=(n,), pos0=32767)
    cache2 = sc.pk.new_cache(1, n)
    scratch = sc.pk.write_scratch(n)
    out = torch.empty((n, sc.spec.cache_width), device="cuda")
    slots = sc.slots_of(0)
    sc.pk.write_paged(cache2, sc.x[0].cuda(), sc.pos[0].to(torch.int32).cuda(), slots, v=sc.v[0].cuda(), latent_out=out,
                      scratch=scratch)
    assert torch.equal(cache2.v_rows(slots).cpu(), sc.v[0])
    assert rel(out.cpu(), sc.rows_ref[0]) < 5e-6
    a, ca, sa = sc.cache.read(slots, sc.second)
    b, cb, sb = cache2.read(slots, sc.second)
    assert (ca != cb).float().mean() < 2e-3 and (sa != sb).float().mean() < 2e-3
    assert rel(b.cpu(), a.cpu()) < 5e-3


@pytest.mark.parametrize("config,n", [("cfg2", 16), ("cfg2", 1), ("cfg2", 4), ("cfg2", 5), ("cfg2", 37), ("cfg5", 64), ("cfg5", 3),
                                      ("cfg3", 5)])
@pytest.mark.parametrize("x_dtype", [torch.float32, torch.bfloat16])
def test_decode_prologue_equals_separate_calls(config, n, x_dtype):
    """The one-launch step prologue (write of the newest tokens + absorb) leaves the bits of the two
    separate calls: cache codes and scales, V rows, unquantised rows, absorbed queries, operand.
    cfg3 (R = 120, not a multiple of 16) takes the entry point's two-launch route. The one-launch prologue
    projects with a register tile that adds the k slices in another order than the separate write: there the
    rows agree to fp32 rounding, and the stored bits are the reference quantiser's bits of the prologue's own rows."""
    sc = Scenario(config, seqlens=(n,), pos0=32767)
    pk, W = sc.pk, sc.spec.cache_width
    x = sc.x[0].cuda().to(x_dtype)
    wpos = sc.pos[0].to(torch.int32).cuda()
    slots = sc.slots_of(0)
    v = sc.v[0].cuda()
    g = torch.Generator().manual_seed(5)
    q = torch.randn((n, sc.spec.n_q, sc.spec.head_dim), generator=g).cuda()
    qpos = (wpos + 1).contiguous()
    caches, outs, wss = [], [], []
    for fused in (False, True):
        cache = pk.new_cache(1, n)
        ws = pk.workspace(n, 1)
        ws.qabs.zero_()
        ws.qop.zero_()
        out = torch.zeros((n, W), device="cuda")
        if fused:
            pk.prologue_step(cache, x, wpos, slots, q, qpos, ws, v=v, latent_out=out)
        else:
            pk.write_paged(cache, x, wpos, slots, v=v, latent_out=out, scratch=ws.wscratch)
            pk.absorb_step(q, qpos, ws)
        torch.cuda.synchronize()
        caches.append(cache), outs.append(out), wss.append(ws)
    assert float(outs[1].abs().max()) > 0
    tiled = config != "cfg3"                                 # the register-tiled projection of the one-launch prologue
    if tiled:
        assert rel(outs[1], outs[0]) < 2e-6
        if x_dtype == torch.float32:                           # rows_ref is the oracle's write of the fp32 hidden states
            assert rel(outs[1].cpu(), sc.rows_ref[0]) < 5e-6
        _, codes, scales = caches[1].read(slots, sc.second)
        _, q_codes, q_scales = _quantise_and_read(outs[1], sc.second)
        assert torch.equal(codes.cpu(), q_codes) and torch.equal(scales.cpu(), q_scales)
    else:
        assert torch.equal(outs[0], outs[1])
        assert torch.equal(caches[0].latent, caches[1].latent)
    assert torch.equal(caches[0].v, caches[1].v)
    assert torch.equal(caches[1].v_rows(slots).cpu(), sc.v[0])
    assert torch.equal(wss[0].qabs, wss[1].qabs) and float(wss[1].qabs.abs().max()) > 0
    assert torch.equal(wss[0].qop, wss[1].qop) and int(wss[1].qop.max()) > 0


@pytest.mark.parametrize("n_split", [1, 3])
def test_attention_behind_prologue_sees_the_newest_token(n_split):
    """Attention launched right behind the prologue streams pages early, except the page the prologue
    is writing: replacing the newest token of every sequence (latent row and V row) and attending at
    once gives what a fully ordered launch gives afterwards, and the oracle's result for the new rows."""
    sc = Scenario("cfg2", seqlens=(300, 129, 128, 1), pos0=5000)
    pk, B = sc.pk, sc.B
    g = torch.Generator().manual_seed(77)
    x_new = (synth.make_hidden(g, B, 4096) * 3.0).cuda()
    v_new = (synth.make_values(g, B, sc.spec.n_kv, sc.spec.head_dim) * 4.0)
    lens = torch.tensor(sc.seqlens, dtype=torch.int32, device="cuda")
    seq = torch.arange(B, dtype=torch.int32, device="cuda")
    slots = sc.cache.slots(seq, lens - 1)
    wpos = (lens - 1 + 5000).contiguous()
    ws = pk.workspace(B, n_split)
    out_early = torch.zeros((B, sc.spec.n_q, sc.spec.head_dim), device="cuda")
    for _ in range(3):                                      # repeated: the launch pair must be ordered every time
        pk.prologue_step(sc.cache, x_new, wpos, slots, sc.q.cuda(), sc.qpos.cuda(), ws, v=v_new.cuda())
        pk.attend_step(sc.cache, ws, out=out_early, after_prologue=True)
    torch.cuda.synchronize()
    assert int(ws.status.abs().sum()) == 0
    out_late = torch.zeros_like(out_early)
    pk.attend_step(sc.cache, ws, out=out_late)
    torch.cuda.synchronize()
    assert torch.equal(out_early, out_late)
    for b, T in enumerate(sc.seqlens):
        sc.v[b][T - 1] = v_new[b]
        _, _, O_ref = sc.oracle_scores_and_output(b, sc.dequantised(b))
        assert rel(out_early[b].cpu(), O_ref) < OUT_TOL


@pytest.mark.parametrize("producer", ["absorb", "prologue"])
def test_attention_polls_operand_ready_counters(producer):
    """pkv_decode_attn_sync: the attention polls the counters its producer raises per sequence instead of waiting for
    the whole launch before it. Same result as the plain, fully ordered launches, round after round (the counters
    are cleared by the attention itself), scores-only mode included."""
    sc = Scenario("cfg2", seqlens=(300, 129, 128, 1), pos0=5000)
    pk, B = sc.pk, sc.B
    g = torch.Generator().manual_seed(78)
    lens = torch.tensor(sc.seqlens, dtype=torch.int32, device="cuda")
    slots = sc.cache.slots(torch.arange(B, dtype=torch.int32, device="cuda"), lens - 1)
    wpos = (lens - 1 + 5000).contiguous()
    q, qpos = sc.q.cuda(), sc.qpos.cuda()
    ws = pk.workspace(B, 3)
    outs = torch.zeros((3, B, sc.spec.n_q, sc.spec.head_dim), device="cuda")
    refs = torch.zeros_like(outs)
    xs = [(synth.make_hidden(g, B, 4096) * (k + 1.0)).cuda() for k in range(3)]
    vs = [(synth.make_values(g, B, sc.spec.n_kv, sc.spec.head_dim) * (k + 1.0)).cuda() for k in range(3)]
    for k in range(3):
        if producer == "absorb":
            pk.absorb_step(q, qpos, ws, signal=True)
            pk.attend_step(sc.cache, ws, out=outs[k], after_absorb=True, polled=True)
        else:
            pk.prologue_step(sc.cache, xs[k], wpos, slots, q, qpos, ws, v=vs[k], signal=True)
            pk.attend_step(sc.cache, ws, out=outs[k], after_prologue=True, polled=True)
        pk.attend_step(sc.cache, ws, out=refs[k])                         # waits for everything before it
    torch.cuda.synchronize()
    assert int(ws.status.abs().sum()) == 0 and int(ws.qsync.abs().sum()) == 0
    for k in range(3):
        assert torch.equal(outs[k], refs[k]), k
    assert float(refs[0].abs().max()) > 0
    if producer == "prologue":
        assert not torch.equal(refs[0], refs[1])                          # the newest token really changed
    # K path
    pk.absorb_step(q, qpos, ws, signal=True)
    pk.attend_step(sc.cache, ws, scores_only=True, after_absorb=True, polled=True)
    pk.merge_step(ws, normalise=False, packed=True)
    a = ws.packed.clone()
    pk.attend_step(sc.cache, ws, scores_only=True)
    pk.merge_step(ws, normalise=False, packed=True)
    torch.cuda.synchronize()
    assert torch.equal(a[..., -2:], ws.packed[..., -2:]) and int(ws.qsync.abs().sum()) == 0


@pytest.mark.parametrize("v_bits,scores_only", [(0, False), (3, False), (0, True)])
def test_polling_attention_gives_up_when_nothing_signals(v_bits, scores_only):
    """A polled attention launch whose producer never raises the counters: the bounded poll runs out, status says
    so (1 = a wait gave up; where = 11: the operand poll, or 30 / 40: a role that waits for the operand), the outputs
    are zero (every CTA leaves the neutral partial), the counters are clean again, and the next, properly signalled
    round is right. Every instantiation of the kernel (bf16 V, quantised V, scores only) has its own set of roles."""
    sc = Scenario("cfg2", seqlens=(200, 64), v_bits=v_bits)
    pk = sc.pk
    ws = pk.workspace(sc.B, 2)
    q, qpos = sc.q.cuda(), sc.qpos.cuda()
    S = torch.zeros((sc.B, sc.spec.n_q, 200), device="cuda")
    kw = dict(scores_only=True, scores_out=S) if scores_only else {}
    pk.absorb_step(q, qpos, ws)                                           # no signal
    out = torch.ones((sc.B, sc.spec.n_q, sc.spec.head_dim), device="cuda")
    pk.attend_step(sc.cache, ws, out=out, after_absorb=True, polled=True, **kw)
    torch.cuda.synchronize()
    assert int(ws.status[0]) == 1 and int(ws.status[1]) in (11, 30, 40)  # the poll, or a role that waits for the operand it feeds
    assert float(out.abs().max()) == 0.0 and int(ws.qsync.abs().sum()) == 0
    ws.status.zero_()
    S.zero_()
    pk.absorb_step(q, qpos, ws, signal=True)
    pk.attend_step(sc.cache, ws, out=out, after_absorb=True, polled=True, **kw)
    got = S.clone()
    ref = torch.zeros_like(out)
    S.zero_()
    pk.attend_step(sc.cache, ws, out=ref, **kw)
    torch.cuda.synchronize()
    assert int(ws.status.abs().sum()) == 0 and torch.equal(out, ref)
    if scores_only:
        assert torch.equal(got, S) and float(S.abs().max()) > 0
    else:
        assert float(ref.abs().max()) > 0


def test_attention_behind_chunk_write_and_prologue():
    """The first decode step after a prefill, all on one stream with nothing in between: a chunk write
    of the cache (tensor-core kernel), the prologue of the newest token, the attention that streams pages
    early. The attention must see the chunk's rows: the prologue lets it start only after its own wait,
    i.e. after the chunk write has completed. Each round rewrites the chunk with other data and compares
    with a launch that waits for everything."""
    T, n = 1500, 1024
    sc = Scenario("cfg2", seqlens=(T, T), pos0=0, x_dtype=torch.bfloat16)
    pk, B = sc.pk, sc.B
    g = torch.Generator().manual_seed(5)
    chunks = [(synth.make_hidden(g, n, 4096) * (k + 2.0)).to(torch.bfloat16).cuda() for k in range(3)]
    vchunks = [(synth.make_values(g, n, sc.spec.n_kv, sc.spec.head_dim) * (k + 2.0)).cuda() for k in range(3)]
    lp = torch.arange(n, dtype=torch.int32, device="cuda")
    cslots = sc.cache.slots(torch.zeros_like(lp), lp)                   # rows 0 .. n-1 of sequence 0
    x_new = (synth.make_hidden(g, B, 4096) * 3.0).cuda()
    v_new = (synth.make_values(g, B, sc.spec.n_kv, sc.spec.head_dim) * 4.0).cuda()
    lens = torch.tensor(sc.seqlens, dtype=torch.int32, device="cuda")
    slots = sc.cache.slots(torch.arange(B, dtype=torch.int32, device="cuda"), lens - 1)
    wpos = (lens - 1).contiguous()
    q, qpos = sc.q.cuda(), sc.qpos.cuda()
    ws, ws2 = pk.workspace(B, 3), pk.workspace(B, 3)
    early = torch.zeros((3, B, sc.spec.n_q, sc.spec.head_dim), device="cuda")
    late = torch.zeros_like(early)
    torch.cuda.synchronize()
    for k in range(3):
        pk.write_paged(sc.cache, chunks[k], lp, cslots, v=vchunks[k])
        pk.prologue_step(sc.cache, x_new, wpos, slots, q, qpos, ws, v=v_new)
        pk.attend_step(sc.cache, ws, out=early[k], after_prologue=True)
        pk.absorb_step(q, qpos, ws2)
        pk.attend_step(sc.cache, ws2, out=late[k])                     # waits for every launch before it
    torch.cuda.synchronize()
    assert int(ws.status.abs().sum()) == 0 and int(ws2.status.abs().sum()) == 0
    for k in range(3):
        assert torch.equal(early[k], late[k]), k
    assert not torch.equal(early[0, 0], early[1, 0])                    # the rounds really differ (sequence 0 holds the chunk)


@pytest.mark.parametrize("config", ["cfg2", "cfg5"])
def test_chunk_write_of_many_tiles_equals_small_chunks(config):
    """More 128-token tiles than the GPU has SMs: a CTA of the tensor-core write then takes several tiles, and the
    epilogue of one runs under the MMAs of the next. Same pages, bit for bit, as the same tokens written 4096 at a
    time (a CTA per tile), the ragged last tile included."""
    spec = synth.make_layer(config, 0)
    pk = PhasorKey.from_spec(spec, device="cuda")
    pk.set_second(0.02)
    n = 148 * 128 * 2 + 300
    g = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn((n, pk.d_model), generator=g, device="cuda").to(torch.bfloat16)
    pos = torch.arange(n, dtype=torch.int32, device="cuda") + 1000
    caches, rows = [], []
    for chunk in (n, 4096):
        cache = pk.new_cache(1, n, with_v=False)
        out = torch.zeros((n, pk.cache_width), device="cuda")
        slots = cache.slots(torch.zeros(n, dtype=torch.int32, device="cuda"), torch.arange(n, dtype=torch.int32, device="cuda"))
        for t0 in range(0, n, chunk):
            t1 = min(n, t0 + chunk)
            pk.write_paged(cache, x[t0:t1], pos[t0:t1], slots[t0:t1], latent_out=out[t0:t1])
        torch.cuda.synchronize()
        assert int(pk._dev["status"].abs().sum()) == 0
        caches.append(cache), rows.append(out)
    assert float(rows[0].abs().max()) > 0
    assert torch.equal(rows[0], rows[1])
    assert torch.equal(caches[0].latent, caches[1].latent)


# ------------------------------------------------------------------------------------------------
# tensor-core kernel (tcgen05 block-scaled NVFP4 scores, bf16 P.V): same checks, same tolerances
# ------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("T", [1, 15, 16, 17, 127, 128, 129, 1000])
def test_tc_decode_lengths(T):
    _check_decode(Scenario("cfg2", seqlens=(T,), pos0=4000), n_split=3, simt=False)


@pytest.mark.parametrize("config,gain", [("cfg2", 1.0), ("cfg2", 256.0), ("cfg3", 1.0), ("cfg3", 256.0), ("cfg5", 1.0),
                                         ("cfg5", 256.0)])
def test_tc_decode_ragged_batch(config, gain):
    _check_decode(Scenario(config, seqlens=(513, 0, 77, 300), gain=gain, pos0=100000), n_split=4, simt=False)


@pytest.mark.parametrize("gain", [1.0, 256.0])
def test_tc_decode_eight_heads_per_kv_head(gain):
    """32 query heads on 4 kv heads: the third grouping the tensor-core kernel is built for (1, 4 or 8 heads per kv head)."""
    _check_decode(Scenario("cfg2", seqlens=(513, 0, 77, 300), gain=gain, pos0=100000, n_kv=4), n_split=4, simt=False)


def test_tc_decode_long_single_split():
    """Many pages through one CTA: every pipeline stage and barrier phase wraps several times."""
    _check_decode(Scenario("cfg2", seqlens=(4096 + 37,), gain=64.0, pos0=28000), n_split=1, simt=False)


def test_tc_matches_simt_partials():
    sc = Scenario("cfg2", seqlens=(700, 256), gain=32.0)
    outs = []
    for simt in (True, False):
        ws = sc.pk.workspace(sc.B, 2)
        sc.pk.absorb_step(sc.q.cuda(), sc.qpos.cuda(), ws, operand=not simt)
        sc.pk.attend_step(sc.cache, ws, simt=simt)
        sc.pk.merge_step(ws, packed=True)
        outs.append((ws.out.clone(), ws.packed.clone()))
    assert rel(outs[1][0].cpu(), outs[0][0].cpu()) < OUT_TOL
    lse = lambda p: p[..., -2].double() + torch.log2(p[..., -1].double())
    assert torch.allclose(lse(outs[1][1]).cpu(), lse(outs[0][1]).cpu(), atol=2e-3)


def test_tc_scores_only():
    sc = Scenario("cfg2", seqlens=(400, 130), gain=64.0)
    ws = sc.pk.workspace(sc.B, 2)
    sc.pk.absorb_step(sc.q.cuda(), sc.qpos.cuda(), ws, operand=True)
    sc.pk.attend_step(sc.cache, ws, simt=False, scores_only=True)
    sc.pk.merge_step(ws, normalise=False, packed=True)
    torch.cuda.synchronize()
    assert int(ws.status.abs().sum()) == 0
    for b, T in enumerate(sc.seqlens):
        _, S_ref, _ = sc.oracle_scores_and_output(b, sc.dequantised(b))
        s2 = S_ref.double() * (po.LOG2E * sc.spec.head_dim ** -0.5)
        lse = torch.log2(torch.exp2(s2 - s2.amax(-1, keepdim=True)).sum(-1)) + s2.amax(-1)
        got = ws.packed[b, :, -2].double().cpu() + torch.log2(ws.packed[b, :, -1].double().cpu())
        assert torch.allclose(got, lse, atol=2e-3)


def test_query_operand_expansion():
    """The operand written by the absorb kernel (four NVFP4 residual terms with per-row tensor scales)
    sums back to the fp32 absorbed query within 3e-4."""
    sc = Scenario("cfg3", seqlens=(16,))
    ws = sc.pk.workspace(sc.B, 1)
    sc.pk.absorb_step(sc.q.cuda(), sc.qpos.cuda(), ws, operand=True)
    blob = ws.qop[:ws.qop_bytes].cpu()
    W = sc.spec.cache_width
    lv = torch.cat([po.E2M1_LEVELS, -po.E2M1_LEVELS])
    codes_b, scales_b = blob[:128 * 128], blob[128 * 128:128 * 128 + 2048]
    head_scale = blob[128 * 128 + 2048:128 * 128 + 2048 + 128].view(torch.float32)              # [32]
    n = torch.arange(128)[:, None]
    col = torch.arange(256)[None, :]
    o = n * 128 + col // 2
    o = o ^ ((o >> 3) & 0x70)
    nib = (codes_b[o] >> ((col & 1) * 4)) & 15
    j = col // 16
    so = (j // 4) * 512 + (n % 32) * 16 + (n // 32) * 4 + j % 4
    sc_f = scales_b[so].view(torch.float8_e4m3fn).float()
    vals = lv[nib.long()] * sc_f * head_scale[(n % 32).squeeze(1)][:, None]                   # [128 = term*32 + head, 256]
    recon = vals.reshape(4, 32, 256).sum(0)[:, :W]
    assert rel(recon, ws.qabs[0].cpu()) < 3e-4


@pytest.mark.parametrize("n_split", [12, 20, 70])
def test_tc_merge_many_splits(n_split):
    """More partials per sequence than one pass of the merge kernel keeps in registers."""
    _check_decode(Scenario("cfg2", seqlens=(9000, 129), gain=64.0, pos0=10000), n_split=n_split, simt=False)


def test_tc_packed_output_for_sharding():
    """The merged, not normalised triple a rank contributes to the all-gather, written by the attention
    launch itself, equals what the separate merge kernel packs."""
    sc = Scenario("cfg2", seqlens=(700, 0, 256), gain=32.0)
    ws = sc.pk.workspace(sc.B, 3)
    sc.pk.absorb_step(sc.q.cuda(), sc.qpos.cuda(), ws, operand=True)
    fused = torch.zeros_like(ws.packed)
    sc.pk.attend_step(sc.cache, ws, packed_out=fused)
    sc.pk.merge_step(ws, normalise=False, packed=True)
    torch.cuda.synchronize()
    assert torch.equal(fused[..., -2], ws.packed[..., -2])                       # maxima
    assert torch.allclose(fused, ws.packed, rtol=1e-5, atol=1e-6)
    gathered = torch.stack([fused, fused])                                       # two identical shards
    out = torch.empty_like(ws.out)
    sc.pk.merge_gathered(gathered, out)
    sc.pk.merge_step(ws)
    assert rel(out[0].cpu(), ws.out[0].cpu()) < 1e-5


def test_exchange_merge_emulated_ranks():
    """The fused exchange-and-merge kernel with 4 ranks' buffers on one GPU, driven phase by phase
    (all pushes, then all merges: kernels that wait on one another never share a GPU). Three rounds,
    so both slots and the epoch bookkeeping are exercised; every rank must obtain the merge of all
    ranks' triples."""
    from phasorkv_b200.sharded import ShardExchange
    from phasorkv_b200 import _lib
    G, B, H, d = 4, 3, 32, 128
    ranks = ShardExchange.local_group(G, B, H, d)
    pk = PhasorKey.from_spec(synth.make_layer("cfg2", 0))
    gen = torch.Generator().manual_seed(5)
    for rnd in range(3):
        packed = torch.randn((G, B, H, d + 2), generator=gen)
        packed[..., -2] *= 20.0                                        # maxima far apart
        packed[..., -1] = packed[..., -1].abs() + 0.1                  # positive sums
        packed[1, 2] = 0.0
        packed[1, 2, :, -2] = float("-inf")                            # a rank that saw no token of sequence 2
        dev = packed.cuda()
        want = torch.empty((B, H, d), device="cuda")
        pk.merge_gathered(dev, want)
        outs = [torch.full((B, H, d), float("nan"), device="cuda") for _ in range(G)]
        for r in range(G):
            ranks[r].run(dev[r], None, _lib.EXCHANGE_PUSH)
        for r in range(G):
            ranks[r].run(None, outs[r], _lib.EXCHANGE_MERGE)
        torch.cuda.synchronize()
        for r in range(G):
            assert int(ranks[r].status.abs().sum()) == 0
            assert torch.allclose(outs[r], want, rtol=1e-5, atol=1e-6), (rnd, r)
            assert int(ranks[r]._epoch[0]) == rnd + 1


def test_merge_exchange_one_launch_emulated_ranks():
    """Merge of the local split-T partials and the exchange in ONE launch. With the ranks' buffers on
    one GPU the peers' triples are delivered first (push phase of the separate kernel), then rank 0 runs
    the fused launch: it merges its own partials, pushes, finds the peers' words and must obtain the
    merge of everything. Two rounds (both slots)."""
    from phasorkv_b200.sharded import ShardExchange
    from phasorkv_b200 import _lib
    G, B, H, d, NS = 3, 2, 32, 128, 7
    ranks = ShardExchange.local_group(G, B, H, d, n_cta=B * H)
    pk = PhasorKey.from_spec(synth.make_layer("cfg2", 0))
    gen = torch.Generator().manual_seed(9)
    for rnd in range(2):
        parts = torch.randn((B, NS, H, d + 2), generator=gen)
        parts[..., -2] *= 10.0
        parts[..., -1] = parts[..., -1].abs() + 0.1
        parts[1, 3, :, :] = 0.0
        parts[1, 3, :, -2] = float("-inf")                             # an empty split
        parts = parts.cuda()
        mine = torch.empty((B, H, d + 2), device="cuda")               # what rank 0 contributes
        _lib.check(_lib.load().pkv_merge(_lib.ptr(parts), NS * H * (d + 2), H * (d + 2), NS, B, H, d, None, _lib.ptr(mine),
                                         _lib.current_stream()), "pkv_merge")
        peers = torch.randn((G - 1, B, H, d + 2), generator=gen)
        peers[..., -2] *= 10.0
        peers[..., -1] = peers[..., -1].abs() + 0.1
        peers = peers.cuda()
        want = torch.empty((B, H, d), device="cuda")
        pk.merge_gathered(torch.cat([mine[None], peers]), want)
        for r in range(1, G):
            ranks[r].run(peers[r - 1], None, _lib.EXCHANGE_PUSH)
        out = torch.full((B, H, d), float("nan"), device="cuda")
        ranks[0].run_parts(parts, NS, out)
        torch.cuda.synchronize()
        assert int(ranks[0].status.abs().sum()) == 0
        assert torch.allclose(out, want, rtol=1e-5, atol=1e-6), rnd
        assert int(ranks[0]._epoch.min()) == rnd + 1
        for r in range(1, G):                                          # the silent peers follow the epoch by hand
            ranks[r]._epoch.fill_(rnd + 1)


def test_exchange_gives_up_when_a_rank_never_pushes():
    """A peer that never delivers: the merge phase runs out of its bounded wait, reports it in the
    status word and leaves the output untouched; the context stays usable."""
    from phasorkv_b200.sharded import ShardExchange
    from phasorkv_b200 import _lib
    G, B, H, d = 2, 1, 32, 128
    ranks = ShardExchange.local_group(G, B, H, d, n_cta=4)
    packed = torch.ones((B, H, d + 2), device="cuda")
    out = torch.full((B, H, d), 7.0, device="cuda")
    ranks[0].run(packed, None, _lib.EXCHANGE_PUSH)                     # rank 1 stays silent
    ranks[0].run(None, out, _lib.EXCHANGE_MERGE)
    torch.cuda.synchronize()
    assert ranks[0].status[0].item() == 3
    assert float(out.min()) == 7.0 and int(ranks[0]._epoch.sum()) == 0
    assert float((packed * 2).sum()) > 0                               # the device still answers


def test_tc_reports_page_index_outside_the_pool():
    """A corrupt page-table entry is reported through the status word and never dereferenced; the other
    sequences of the batch are unaffected and the context stays usable."""
    sc = Scenario("cfg2", seqlens=(300, 200))
    good = sc.cache.page_table.clone()
    ws = sc.pk.workspace(sc.B, 1)
    sc.pk.absorb_step(sc.q.cuda(), sc.qpos.cuda(), ws)
    sc.pk.attend_step(sc.cache, ws, out=ws.out)
    want = ws.out.clone()
    sc.cache.page_table[0, 1] = 10 ** 6
    ws.out.zero_()
    sc.pk.attend_step(sc.cache, ws, out=ws.out)
    torch.cuda.synchronize()
    assert ws.status[0].item() == 2 and ws.status[1].item() == 1
    assert rel(ws.out[1].cpu(), want[1].cpu()) < 1e-6
    sc.cache.page_table.copy_(good)
    ws.status.zero_()
    sc.pk.attend_step(sc.cache, ws, out=ws.out)
    torch.cuda.synchronize()
    assert int(ws.status.abs().sum()) == 0 and rel(ws.out.cpu(), want.cpu()) < 1e-6


def test_bench_decode_cli_small(tmp_path):
    """The decode-benchmark CLI end to end on a small sweep: result file in the reference's form, and
    an interrupted sweep resumes (keys present are not re-timed)."""
    import json
    from phasorkv_b200 import bench_decode as bd
    out, shp = tmp_path / "r.json", tmp_path / "s.json"
    argv = ["--configs", "cfg2", "--lens", "1024,4096", "--batches", "2", "--layers", "2", "--iters", "3",
            "--out", str(out), "--shapes-out", str(shp)]
    assert bd.main(argv) == 0
    res = json.load(open(out))
    keys = sorted(res)
    assert len(keys) == 2 and keys[0].startswith("cfg2|T1024|B2|algo=tc,n_split=")
    for v in res.values():
        assert v["ms"] > 0 and v["gbs"] > 0 and v["tflops"] > 0
    before = dict(res)
    assert bd.main(argv) == 0
    assert json.load(open(out)) == before


def test_hf_llama_attention_patch_decodes_like_the_model():
    """The patch object installed into the attention modules of a small random Hugging Face Llama whose
    key projections ARE the factors' W_hat: prefill runs the model's own attention and fills the latent
    caches, every decode step runs write + absorb + latent attention instead of rebuilding keys. The
    logits follow the unpatched model (with its own KV cache) up to the NVFP4 error of the latent."""
    transformers = pytest.importorskip("transformers")
    import copy
    from phasorkv_b200.patch import PhasorKeyPatch
    cfg = transformers.LlamaConfig(vocab_size=256, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                                   num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                                   max_position_embeddings=4096, attn_implementation="eager")
    torch.manual_seed(3)
    model = transformers.LlamaForCausalLM(cfg).cuda().float().eval()
    inv_freq = model.model.rotary_emb.inv_freq.double().cpu()
    specs = []
    for l, layer in enumerate(model.model.layers):
        spec = synth.make_layer("cfg2", l, d_model=512, factor_gain=48.0)
        spec.inv_freq = inv_freq
        W = po.w_hat(spec.A, spec.B, spec.freq, spec.n_kv, spec.head_dim)
        layer.self_attn.k_proj.weight.data.copy_(W.float())
        specs.append(spec)
    ref = copy.deepcopy(model)
    patch = PhasorKeyPatch(install_forward=True, max_tokens=512)
    undos = [patch.patch(l, layer, specs[l], 8, 128, 32, "cuda") for l, layer in enumerate(model.model.layers)]
    g = torch.Generator().manual_seed(4)
    ids = torch.randint(0, 256, (2, 200), generator=g).cuda()
    with torch.no_grad():
        r = ref(input_ids=ids, use_cache=True)
        o = model(input_ids=ids, use_cache=False)
        assert rel(o.logits, r.logits) < 1e-5                                  # prefill: the model's own attention
        past, errs = r.past_key_values, []
        nxt = r.logits[:, -1].argmax(-1)[:, None]
        for step in range(4):
            r = ref(input_ids=nxt, past_key_values=past, use_cache=True)
            o = model(input_ids=nxt, use_cache=False)
            errs.append(rel(o.logits, r.logits))
            past, nxt = r.past_key_values, r.logits[:, -1].argmax(-1)[:, None]
    torch.cuda.synchronize()
    print("decode logits rel errors", errs)
    assert all(int(st.ws.status.abs().sum()) == 0 for st in patch.states.values())
    assert patch.states[0].length == 204
    assert max(errs) < 5e-3                                                    # measured 2.4e-3
    for u in undos:
        u()
    assert "forward" not in model.model.layers[0].self_attn.__dict__ and not patch.states
    with torch.no_grad():
        assert rel(model(input_ids=ids).logits, ref(input_ids=ids).logits) < 1e-6


def test_real_factorization_at_llama_head_shape():
    """Factors of a reference Factorization(W, Cx, q2, 8, 128, "band8", "xq") with water-filled ranks (32 query heads,
    8 kv heads, head_dim 128, rope base 500000; energy-sorted dims, 110 complex + 36 slow reals = width 256), positions
    beyond 100000: constructor arrays -> write -> absorb -> scores against the reference's own output and against keys
    rebuilt from W_hat with HF's rotary (oracle #2); then the quantised cache through the tensor-core decode against
    fp32 scoring on the dequantised cache (oracle #1)."""
    g = _golden("phasorkey_llama_heads.npz")
    D, n_q, n_kv, d = (int(v) for v in g["dims"])
    t = lambda k: torch.from_numpy(g[k])
    inv_freq = t("inv_freq")
    pk = PhasorKey.from_factors(t("A"), t("B"), t("freq"), n_q, n_kv, d, inv_freq, t("A_s"), t("B_s"), t("slow"))
    assert pk.cache_width == 256 and pk.R == 110 and pk.R_s == 36
    x, q = t("x"), t("q")
    ph_k, ph_q = po.rope_phasors(inv_freq, t("pos_k")), po.rope_phasors(inv_freq, t("pos_q"))
    rows, qabs = pk.write(x, ph_k), pk.absorb(q, ph_q)
    assert rel(rows.cpu(), t("rows")) < 1e-5 and rel(qabs.cpu(), t("qabs")) < 1e-5
    S = PhasorKey.scores(qabs, rows).cpu()
    assert rel(S, t("scores")) < 1e-5
    assert rel(S, t("scores_hf")) < LOGIT_TOL
    # quantised cache, decode on the tensor cores
    T = x.shape[0]
    pk.calibrate_second(rows)
    cache = pk.new_cache(1, T)
    lp = torch.arange(T, dtype=torch.int32, device="cuda")
    slots = cache.slots(torch.zeros_like(lp), lp)
    gen = torch.Generator().manual_seed(9)
    v = synth.make_values(gen, T, n_kv, d)
    pk.write_paged(cache, x.cuda(), t("pos_k").to(torch.int32).cuda(), slots, v=v.cuda())
    cache.seqlens.fill_(T)
    ws = pk.workspace(1, 2)
    Sd = torch.zeros((1, n_q, T), device="cuda")
    pk.absorb_step(q[:, 0][None].contiguous().cuda(), t("pos_q").to(torch.int32).cuda(), ws)
    pk.attend_step(cache, ws, scores_out=Sd, out=ws.out, after_absorb=True)
    torch.cuda.synchronize()
    assert int(ws.status.abs().sum()) == 0
    hat, codes, scales = cache.read(slots, pk.second)
    # the stored bits are the reference quantiser's bits of the rows the write kernel itself produced
    out = torch.empty((T, 256), device="cuda")
    pk.write_paged(None, x.cuda(), t("pos_k").to(torch.int32).cuda(), None, latent_out=out)
    o_codes, o_scales, _ = po.nvfp4_quantize(out.cpu(), torch.tensor([pk.second]))
    assert torch.equal(codes.cpu(), po.pack_nibbles(o_codes)) and torch.equal(scales.cpu(), o_scales)
    S_ref = PhasorKey.scores(qabs, hat)[:, 0].cpu()
    assert rel(Sd[0].cpu(), S_ref) < LOGIT_TOL
    assert rel(ws.out[0].cpu(), po.attend(S_ref, v, n_kv, d)) < OUT_TOL


def test_mean_direction_split_through_the_kernels():
    """The mean-direction split (k = A Q(B_perp x) + alpha * W mu, phasorkv/kvmethods.py:895-899) as a PhasorKey
    with d/2 further latent dims: the CUDA write / absorb / scores reproduce 'rebuild the split keys, rotate with
    HF rotary' on hidden states with a strong mean component, and the tensor-core decode meets the oracle on
    the dequantised cache."""
    spec = synth.make_layer("cfg2", 1)
    g = torch.Generator().manual_seed(41)
    A, B, freq = spec.A[:, ::2], spec.B[::2], spec.freq[::2]                   # rank 1 per frequency: 64 complex dims
    mu = torch.randn(4096, generator=g, dtype=torch.float64) * 0.3 + 1.0
    kbar = torch.randn(spec.n_kv * spec.head_dim, generator=g, dtype=torch.float64) * 0.05
    pk = PhasorKey.with_mean_direction(A, B, freq, mu, kbar, spec.n_q, spec.n_kv, spec.head_dim, spec.inv_freq)
    assert pk.cache_width == 256
    T, pos0 = 300, 7000
    x = synth.make_hidden(g, T, 4096) * 0.2 + (torch.rand(T, 1, generator=g) + 0.5) * mu.float()[None, :]   # alpha in 0.5 .. 1.5
    v = synth.make_values(g, T, spec.n_kv, spec.head_dim)
    q = synth.make_query(g, 1, spec.n_q, spec.head_dim)
    pos = torch.arange(T) + pos0
    ph_k = po.rope_phasors(spec.inv_freq, pos)
    ph_q = po.rope_phasors(spec.inv_freq, torch.tensor([T + pos0]))
    # exact (unquantised) rows and scores against the split keys rebuilt densely
    mu_scaled = mu / mu.dot(mu)
    Bc = B.to(torch.complex128)
    B_perp = Bc - (Bc @ mu.to(torch.complex128))[:, None] * mu_scaled.to(torch.complex128)[None, :]
    W_split = po.w_hat(A, B_perp, freq, spec.n_kv, spec.head_dim)
    W_mean = kbar[:, None] * mu_scaled[None, :]                                # alpha * kbar as a dense rank-1 projection
    S_split = po.rebuilt_scores(W_split + W_mean, x, q[0][:, None, :], ph_k, ph_q, spec.n_q, spec.n_kv, spec.head_dim)[:, 0]
    rows, qabs = pk.write(x, ph_k), pk.absorb(q[0][:, None, :], ph_q)
    S = PhasorKey.scores(qabs, rows)[:, 0].cpu()
    assert rel(S, S_split) < 2e-5
    # quantised cache, tensor-core decode, oracle on the dequantised rows
    pk.calibrate_second(rows)
    cache = pk.new_cache(1, T)
    lp = torch.arange(T, dtype=torch.int32, device="cuda")
    slots = cache.slots(torch.zeros_like(lp), lp)
    pk.write_paged(cache, x.cuda(), pos.to(torch.int32).cuda(), slots, v=v.cuda())
    cache.seqlens.fill_(T)
    ws = pk.workspace(1, 2)
    Sd = torch.zeros((1, spec.n_q, T), device="cuda")
    pk.absorb_step(q.cuda(), torch.tensor([T + pos0], dtype=torch.int32, device="cuda"), ws)
    pk.attend_step(cache, ws, scores_out=Sd, out=ws.out, after_absorb=True)
    hat, _, _ = cache.read(slots, pk.second, codes=False)
    S_ref = PhasorKey.scores(qabs.float(), hat)[:, 0].cpu()
    assert rel(Sd[0].cpu(), S_ref) < LOGIT_TOL
    assert rel(ws.out[0].cpu(), po.attend(S_ref, v, spec.n_kv, spec.head_dim)) < OUT_TOL


@pytest.mark.parametrize("v_bits", [0, 3])
def test_patched_layer_state_keeps_one_length_per_sequence(v_bits):
    """A ragged batch through the decode state of a patched layer (V pages in bf16, or as per-token 3-bit codes: the
    oracle then attends over the dequantised value rows) (prefill right-padded with per-sequence
    token counts, as the reference's runner passes them in attn.kv_lengths, phasorkv/runner.py:94-99; then two
    decode steps): every sequence is written and attended at its own positions, so each gives what it gives
    alone in a batch of one, and what the oracle gives."""
    from phasorkv_b200.patch import LayerDecodeState
    spec = synth.make_layer("cfg2", 0)
    pk = PhasorKey.from_spec(spec, device="cuda")
    pk.set_second(0.02)
    g = torch.Generator().manual_seed(31)
    lens, T, steps = [200, 77, 129], 200, 2
    B = len(lens)
    x = synth.make_hidden(g, B * (T + steps), 4096).view(B, T + steps, 4096).cuda()
    v = synth.make_values(g, B * (T + steps), spec.n_kv, spec.head_dim).view(B, T + steps, spec.n_kv, spec.head_dim).cuda()
    q = torch.randn((B, steps, spec.n_q, spec.head_dim), generator=g).cuda()

    def run(rows):
        st = LayerDecodeState(pk, len(rows), 512, v_bits=v_bits)
        st.calibrated = True                                  # keep the tensor scale set above
        xs = torch.stack([x[b, :T] for b in rows]); vs = torch.stack([v[b, :T] for b in rows])
        st.prefill(xs, vs, lengths=[lens[b] for b in rows])
        outs = []
        for k in range(steps):                                # token k of a sequence follows its own last token
            xn = torch.stack([x[b, T + k] for b in rows]); vn = torch.stack([v[b, T + k] for b in rows])
            outs.append(st.decode(xn, torch.stack([q[b, k] for b in rows]), vn).clone())
        assert st.lengths == [lens[b] + steps for b in rows]
        return st, outs
    st, outs = run(list(range(B)))
    opk = po.PhasorKeyOracle.from_spec(spec)
    for b in range(B):
        _, alone = run([b])
        for k in range(steps):
            assert rel(outs[k][b], alone[k][0]) < 1e-5, (b, k)
        # the oracle on what the cache holds: tokens 0 .. lens[b] + steps - 1 at positions 0 .., query at the last one
        n = lens[b] + steps
        slots = st.cache.slots(torch.full((n,), b, dtype=torch.int32, device="cuda"), torch.arange(n, dtype=torch.int32, device="cuda"))
        rows_hat, _, _ = st.cache.read(slots, pk.second, codes=False)
        ph_q = po.rope_phasors(spec.inv_freq, torch.tensor([n - 1]), spec.attn_scale)
        qa = opk.absorb(q[b, steps - 1].cpu()[:, None, :], ph_q)[:, 0]
        O_ref = po.attend(opk.scores(qa, rows_hat.cpu()), st.cache.v_rows(slots).cpu().float(), spec.n_kv, spec.head_dim)
        assert rel(outs[steps - 1][b].cpu(), O_ref) < OUT_TOL, b


@pytest.mark.parametrize("config,n_sink,n_recent", [("cfg2", 4, 128), ("cfg3", 4, 128), ("cfg5", 2, 37), ("cfg2", 0, 0)])
def test_exact_token_side_path(config, n_sink, n_recent):
    """Attention sinks and a recent window kept as rotated bf16 keys join the softmax of the latent
    tokens: the extra partial triple, merged with the splits, reproduces softmax over the concatenation
    [exact tokens | latent tokens] (the reference's latent_decode with `exact`)."""
    pos0 = 1000
    sc = Scenario(config, seqlens=(300, 129), gain=48.0, pos0=pos0)
    spec, B, E = sc.spec, sc.B, n_sink + n_recent
    g = torch.Generator().manual_seed(31)
    W = po.w_hat(spec.A, spec.B, spec.freq, spec.n_kv, spec.head_dim, spec.A_s, spec.B_s, spec.slow)
    slow = spec.slow if spec.slow is not None else torch.zeros(0, dtype=torch.long)
    k_e = torch.zeros((B, spec.n_kv, max(E, 1), spec.head_dim), dtype=torch.bfloat16)
    v_e = torch.zeros_like(k_e)
    for b, T in enumerate(sc.seqlens):
        # sinks at positions 0.., the recent window right behind the latent tokens; the query follows it
        pos_e = torch.cat([torch.arange(n_sink), pos0 + T + torch.arange(n_recent)])
        sc.qpos[b] = pos0 + T + n_recent
        if E == 0:
            continue
        x_e = synth.make_hidden(g, E)
        ph = po.rope_phasors(spec.inv_freq, pos_e, spec.attn_scale).clone()
        if slow.numel():
            ph[:, slow] = ph[0, 0].abs().to(ph.dtype)
        k = (x_e.double() @ W.T).reshape(E, spec.n_kv, spec.head_dim).transpose(0, 1)
        cos, sin = torch.cat([ph.real, ph.real], -1), torch.cat([ph.imag, ph.imag], -1)
        k_e[b, :, :E] = po.hf_rotate(k, cos[None], sin[None]).to(torch.bfloat16)
        v_e[b, :, :E] = synth.make_values(g, E, spec.n_kv, spec.head_dim).transpose(0, 1)
    ws = sc.pk.workspace(B, 3)
    q, qpos = sc.q.cuda(), sc.qpos.cuda()
    sc.pk.absorb_step(q, qpos, ws)
    sc.pk.attend_step(sc.cache, ws, after_absorb=True)
    n_e = torch.full((B,), E, dtype=torch.int32, device="cuda")
    sc.pk.exact_step(q, qpos, k_e.cuda(), v_e.cuda(), ws, n_exact=n_e)
    sc.pk.merge_step(ws, exact=True)
    torch.cuda.synchronize()
    assert int(ws.status.abs().sum()) == 0
    for b, T in enumerate(sc.seqlens):
        _, S_lat, _ = sc.oracle_scores_and_output(b, sc.dequantised(b))
        ph_q = po.rope_phasors(spec.inv_freq, sc.qpos[b:b + 1], spec.attn_scale).clone()
        if slow.numel():
            ph_q[:, slow] = ph_q[0, 0].abs().to(ph_q.dtype)
        cq, sq = torch.cat([ph_q.real, ph_q.real], -1), torch.cat([ph_q.imag, ph_q.imag], -1)
        qr = po.hf_rotate(sc.q[b].double(), cq, sq)                                       # [H, d]
        ke = k_e[b, :, :E].double().repeat_interleave(spec.n_q // spec.n_kv, dim=0)      # [H, E, d]
        S_ex = torch.einsum("hd,hed->he", qr, ke).float()
        S = torch.cat([S_ex, S_lat], dim=1)
        V = torch.cat([v_e[b, :, :E].transpose(0, 1), sc.v[b]], dim=0)
        O_ref = po.attend(S, V, spec.n_kv, spec.head_dim)
        assert rel(ws.out[b].cpu(), O_ref) < OUT_TOL, (b, T)
        if E:                                                                            # the side path matters in this test
            assert rel(po.attend(S_lat, sc.v[b], spec.n_kv, spec.head_dim), O_ref) > 5 * OUT_TOL


@pytest.mark.parametrize("config", ["cfg2", "cfg3"])
def test_layer_handle_from_host_arrays(config):
    """pkv_layer_create (a host without a tensor library uploads PhasorKey's arrays once) gives a layer
    that writes, quantises and reads back exactly what the torch-owned layer does; the entry points
    under the reference's names (quantize_nvfp4, dequant, status_read) answer like their originals."""
    import ctypes
    from phasorkv_b200 import _lib
    lib = _lib.load()
    sc = Scenario(config, seqlens=(200,), pos0=777)
    spec, pk = sc.spec, sc.pk
    f32 = lambda t: np.ascontiguousarray(t.numpy().astype(np.float32))
    keep = dict(B_re=f32(spec.B.real), B_im=f32(spec.B.imag), A_re=f32(spec.A.real), A_im=f32(spec.A.imag),
                freq=np.ascontiguousarray(spec.freq.numpy().astype(np.int32)),
                inv_freq=np.ascontiguousarray(spec.inv_freq.numpy().astype(np.float64)))
    if spec.R_s:
        keep.update(B_s=f32(spec.B_s), A_s=f32(spec.A_s), slow=np.ascontiguousarray(spec.slow.numpy().astype(np.int32)))
    p = lambda k: keep[k].ctypes.data if k in keep else None
    host = _lib.LayerHost(spec.d_model, spec.n_q, spec.n_kv, spec.head_dim, spec.R, spec.R_s,
                          0 if spec.slow is None else int(spec.slow.numel()), spec.attn_scale, sc.second,
                          p("B_re"), p("B_im"), p("B_s"), p("A_re"), p("A_im"), p("A_s"), p("freq"), p("slow"), p("inv_freq"))
    handle = ctypes.POINTER(_lib.Layer)()
    _lib.check(lib.pkv_layer_create(ctypes.byref(host), ctypes.byref(handle)), "pkv_layer_create")
    try:
        n, W = 200, spec.cache_width
        slots = sc.slots_of(0)
        for dt in (torch.float32, torch.bfloat16):                   # CUDA-core and tensor-core write kernels
            x = sc.x[0].cuda().to(dt)
            cache2 = pk.new_cache(1, n)
            out = torch.zeros((n, W), device="cuda")
            pos = sc.pos[0].to(torch.int32).cuda()
            _lib.check(lib.pkv_cache_write(handle, ctypes.byref(cache2.c), _lib.ptr(x), pk._xdt(x), _lib.ptr(pos), None,
                                           _lib.ptr(slots), n, _lib.ptr(out), None, None, _lib.ptr(pk._dev["status"]),
                                           _lib.current_stream()), "pkv_cache_write")
            cache3 = pk.new_cache(1, n)
            out3 = torch.zeros_like(out)
            pk.write_paged(cache3, x, pos, slots, latent_out=out3)
            torch.cuda.synchronize()
            assert torch.equal(out, out3) and torch.equal(cache2.latent, cache3.latent)
        # the aliases
        rows = torch.empty((n, W), device="cuda")
        _lib.check(lib.pkv_dequant(ctypes.byref(cache3.c), _lib.ptr(slots), n, sc.second, _lib.ptr(rows), _lib.current_stream()),
                   "pkv_dequant")
        want, _, _ = cache3.read(slots, sc.second, codes=False)
        cache4 = pk.new_cache(1, n)
        _lib.check(lib.pkv_quantize_nvfp4(ctypes.byref(cache4.c), _lib.ptr(out3), _lib.ptr(slots), n, sc.second,
                                          _lib.current_stream()), "pkv_quantize_nvfp4")
        host_status = (ctypes.c_int32 * 4)(9, 9, 9, 9)
        _lib.check(lib.pkv_status_read(_lib.ptr(pk._dev["status"]), host_status, _lib.current_stream()), "pkv_status_read")
        assert torch.equal(rows, want)
        assert torch.equal(cache4.latent, cache3.latent)              # quantising the dumped rows again: same codes
        assert list(host_status) == [0, 0, 0, 0]
    finally:
        _lib.check(lib.pkv_layer_destroy(handle), "pkv_layer_destroy")
    assert lib.pkv_layer_create(None, ctypes.byref(handle)) != 0


@pytest.mark.parametrize("config,gain", [("cfg2", 1.0), ("cfg2", 128.0), ("cfg3", 64.0), ("cfg5", 64.0)])
def test_attention_absorbs_raw_queries_itself(config, gain):
    """pkv_decode_attn_q (the attention kernel forms the NVFP4 query operand in shared memory) gives the
    bits of pkv_absorb followed by pkv_decode_attn, in both kernel modes, and the oracle's result."""
    sc = Scenario(config, seqlens=(700, 0, 129, 300), gain=gain, pos0=90000)
    pk, B = sc.pk, sc.B
    q, qpos = sc.q.cuda(), sc.qpos.cuda()
    Tmax = max(sc.seqlens)
    for n_split in (1, 3):
        ws_a, ws_b = pk.workspace(B, n_split), pk.workspace(B, n_split)
        Sa = torch.zeros((B, sc.spec.n_q, Tmax), device="cuda")
        Sb = torch.zeros_like(Sa)
        pk.absorb_step(q, qpos, ws_a)
        pk.attend_step(sc.cache, ws_a, scores_out=Sa, out=ws_a.out)
        pk.attend_q_step(sc.cache, q, qpos, ws_b, scores_out=Sb, out=ws_b.out)
        torch.cuda.synchronize()
        assert int(ws_b.status.abs().sum()) == 0
        assert torch.equal(Sa, Sb) and torch.equal(ws_a.out, ws_b.out) and float(ws_b.out.abs().max()) > 0
        # scores-only mode: log-sum-exp partials
        pk.attend_step(sc.cache, ws_a, scores_only=True)
        pk.attend_q_step(sc.cache, q, qpos, ws_b, scores_only=True)
        torch.cuda.synchronize()
        assert torch.equal(ws_a.partials[..., -2:], ws_b.partials[..., -2:])
    for b, T in enumerate(sc.seqlens):
        if T:
            _, S_ref, O_ref = sc.oracle_scores_and_output(b, sc.dequantised(b))
            assert rel(Sb[b, :, :T].cpu(), S_ref) < LOGIT_TOL and rel(ws_b.out[b].cpu(), O_ref) < OUT_TOL


@pytest.mark.parametrize("n_split", [1, 3])
def test_raw_query_attention_behind_a_write_only_prologue(n_split):
    """The decode step as the bench chains it: the newest token's write alone, then attention on raw queries
    that starts at once (pages stream early, the query is declared ready) and waits for the write only
    before it fetches the page being written."""
    sc = Scenario("cfg2", seqlens=(300, 129, 128, 1), pos0=5000)
    pk, B = sc.pk, sc.B
    g = torch.Generator().manual_seed(78)
    x_new = (synth.make_hidden(g, B, 4096) * 3.0).cuda()
    v_new = (synth.make_values(g, B, sc.spec.n_kv, sc.spec.head_dim) * 4.0)
    lens = torch.tensor(sc.seqlens, dtype=torch.int32, device="cuda")
    slots = sc.cache.slots(torch.arange(B, dtype=torch.int32, device="cuda"), lens - 1)
    wpos = (lens - 1 + 5000).contiguous()
    ws = pk.workspace(B, n_split)
    q, qpos = sc.q.cuda(), sc.qpos.cuda()
    out_early = torch.zeros((B, sc.spec.n_q, sc.spec.head_dim), device="cuda")
    for _ in range(3):
        pk.prologue_step(sc.cache, x_new, wpos, slots, None, None, ws, v=v_new.cuda())
        pk.attend_q_step(sc.cache, q, qpos, ws, out=out_early, early=True, tail_written=True, query_ready=True)
    torch.cuda.synchronize()
    assert int(ws.status.abs().sum()) == 0
    out_late = torch.zeros_like(out_early)
    pk.absorb_step(q, qpos, ws)
    pk.attend_step(sc.cache, ws, out=out_late)
    torch.cuda.synchronize()
    assert torch.equal(out_early, out_late)
    for b, T in enumerate(sc.seqlens):
        sc.v[b][T - 1] = v_new[b]
        _, _, O_ref = sc.oracle_scores_and_output(b, sc.dequantised(b))
        assert rel(out_early[b].cpu(), O_ref) < OUT_TOL
