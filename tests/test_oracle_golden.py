"""The CPU oracle (oracle/) against vectors produced by the unmodified reference (tests/golden/)."""
import os

import numpy as np
import torch

from oracle import c_oracle
from oracle import phasor_oracle as po

from conftest import GOLDEN


def _load(name):
    return np.load(os.path.join(GOLDEN, name))


def test_nvfp4_torch_oracle_bit_exact():
    g = _load("nvfp4_cases.npz")
    x, second = torch.from_numpy(g["x"]), torch.from_numpy(g["second"])
    codes, scales, xhat = po.nvfp4_quantize(x, second)
    assert np.array_equal(codes.numpy(), g["codes"])
    assert np.array_equal(scales.numpy(), g["scales"])
    assert np.array_equal(xhat.numpy(), g["xhat"])
    assert np.array_equal(po.pack_nibbles(codes).numpy(), g["packed"])
    assert torch.equal(po.unpack_nibbles(torch.from_numpy(g["packed"])), codes)
    assert np.array_equal(po.nvfp4_dequantize(codes, scales, second).numpy(), g["xhat"])


def test_nvfp4_c_oracle_bit_exact():
    g = _load("nvfp4_cases.npz")
    codes, scales, xhat = c_oracle.nvfp4_quantize(g["x"], float(g["second"][0]))
    assert np.array_equal(codes, g["codes"])
    assert np.array_equal(scales, g["scales"])
    assert np.array_equal(xhat, g["xhat"])
    assert np.array_equal(c_oracle.nvfp4_dequantize(codes, scales, float(g["second"][0])), g["xhat"])


def test_nvfp4_scale_round_up_oracles_bit_exact():
    """PHASORKV_SCALE_UP=1 of the reference (quant.py:57,85-88): block scales rounded up. Both oracles
    against vectors the reference produced with that switch, and the two modes do differ."""
    g, g0 = _load("nvfp4_cases_scale_up.npz"), _load("nvfp4_cases.npz")
    assert np.array_equal(g["x"], g0["x"]) and not np.array_equal(g["scales"], g0["scales"])
    x, second = torch.from_numpy(g["x"]), torch.from_numpy(g["second"])
    codes, scales, xhat = po.nvfp4_quantize(x, second, scale_up=True)
    assert np.array_equal(codes.numpy(), g["codes"])
    assert np.array_equal(scales.numpy(), g["scales"])
    assert np.array_equal(xhat.numpy(), g["xhat"])
    c_codes, c_scales, c_xhat = c_oracle.nvfp4_quantize(g["x"], float(g["second"][0]), scale_up=True)
    assert np.array_equal(c_codes, g["codes"]) and np.array_equal(c_scales, g["scales"]) and np.array_equal(c_xhat, g["xhat"])
    # rounded-up scales never clip the block maximum: |x| <= 6 * scale wherever the scale is not saturated
    sc = torch.from_numpy(g["scales"]).view(torch.float8_e4m3fn).float() * second
    amax = x.reshape(x.shape[0], -1, 16).abs().amax(-1)
    free = torch.from_numpy(g["scales"]) != 0x7E
    assert bool((amax[free] <= 6.0 * sc[free] * (1 + 1e-6)).all())


def test_nvfp4_known_behaviours():
    """Ties go to the lower magnitude, no signed zero, zero block -> scale byte 0, saturation."""
    g = _load("nvfp4_cases.npz")
    codes, scales = g["codes"], g["scales"]
    assert list(codes[0, :7]) == [0, 1, 2, 3, 4, 5, 6]            # 0.25->0, 0.75->0.5, ... 5->4
    assert list(codes[0, 7:14]) == [0, 9, 10, 11, 12, 13, 14]     # -0.25 -> +0 (no sign bit)
    assert codes[0, 14] == 7 and codes[0, 15] == 15
    assert scales[0, 1] == 0 and not codes[0, 16:32].any()        # all-zero block
    assert not (codes == 8).any()                                 # code 0x8 (-0) never produced
    assert scales[0, 3] == 0x7E                                   # scale saturates at 448


def test_static_second():
    g = _load("nvfp4_cases.npz")
    s = po.nv_static_second(torch.from_numpy(g["static_var"]))
    assert np.array_equal(s.numpy(), g["static_second"])


def _pk(g, tag, dt=None):
    A, B = torch.from_numpy(g[f"{tag}_A"]), torch.from_numpy(g[f"{tag}_B"])
    A_s = torch.from_numpy(g[f"{tag}_A_s"]) if f"{tag}_A_s" in g else None
    B_s = torch.from_numpy(g[f"{tag}_B_s"]) if f"{tag}_B_s" in g else None
    slow = torch.from_numpy(g[f"{tag}_slow"]) if f"{tag}_slow" in g else None
    D, n_q, n_kv, d = (int(v) for v in g["dims"])
    return po.PhasorKeyOracle(A, B, torch.from_numpy(g[f"{tag}_freq"]), n_q, n_kv, d, A_s, B_s, slow), (D, n_q, n_kv, d)


def test_phasors_match_reference():
    g = _load("phasorkey_injected.npz")
    inv = torch.from_numpy(g["inv_freq"])
    for tag in ("freq", "band"):
        ph = po.rope_phasors(inv, torch.from_numpy(g[f"{tag}_pos_k"]))
        assert np.array_equal(ph.numpy(), g[f"{tag}_ph_k"])


def test_phasorkey_injected_fp32():
    g = _load("phasorkey_injected.npz")
    for tag in ("freq", "band"):
        pk, _ = _pk(g, tag)
        ph_k, ph_q = torch.from_numpy(g[f"{tag}_ph_k"]), torch.from_numpy(g[f"{tag}_ph_q"])
        rows = pk.write(torch.from_numpy(g[f"{tag}_x"]), ph_k)
        qa = pk.absorb(torch.from_numpy(g[f"{tag}_q"]), ph_q)
        S = pk.scores(qa, rows)
        assert np.array_equal(rows.numpy(), g[f"{tag}_rows"])
        assert np.array_equal(qa.numpy(), g[f"{tag}_qabs"])
        assert np.array_equal(S.numpy(), g[f"{tag}_scores"])


def test_phasorkey_factorized_and_hf_identity():
    g = _load("phasorkey_factorized.npz")
    x, q = torch.from_numpy(g["x"]), torch.from_numpy(g["q"])
    ph_k, ph_q = torch.from_numpy(g["ph_k"]), torch.from_numpy(g["ph_q"])
    for tag in ("freq", "band"):
        pk, (D, n_q, n_kv, d) = _pk(g, tag)
        rows = pk.write(x, ph_k)
        qa = pk.absorb(q, ph_q)
        S = pk.scores(qa, rows)
        for got, key in ((rows, "rows"), (qa, "qabs"), (S, "scores")):
            ref = torch.from_numpy(g[f"{tag}_{key}"])
            assert (got - ref).norm() / ref.norm() < 1e-14
        # oracle #2: dense keys from W_hat rotated the HF way; W_hat rebuilt from the factors
        W = po.w_hat(pk.A, pk.B, pk.freq, n_kv, d, pk.A_s, pk.B_s, pk.slow if pk.R_s else None)
        Wref = torch.from_numpy(g[f"{tag}_W_hat"])
        assert (W - Wref).norm() / Wref.norm() < 1e-13
        S2 = po.rebuilt_scores(W, x, q, ph_k, ph_q, n_q, n_kv, d, pk.slow)
        S2ref = torch.from_numpy(g[f"{tag}_scores_hf"])
        assert (S2 - S2ref).norm() / S2ref.norm() < 1e-14
        assert (S - S2).norm() / S2.norm() < 2e-15 * 10       # README.md:75-77 states 2e-15


def test_split_merge_equals_unsplit():
    gen = torch.Generator().manual_seed(7)
    H, T, n_kv, d = 8, 300, 2, 16
    S = torch.randn(H, T, generator=gen) * 40
    V = torch.randn(T, n_kv, d, generator=gen).to(torch.bfloat16)
    full = po.attend(S, V, n_kv, d)
    parts = [po.partial_attend(S[:, a:b], V[a:b], n_kv, d) for a, b in ((0, 7), (7, 128), (128, 300))]
    m, l, o = (torch.stack(t) for t in zip(*parts))
    assert torch.allclose(po.merge_partials(m, l, o), full, rtol=2e-5, atol=1e-6)


def test_attend_and_split_merge_against_reference_vectors():
    """softmax . V and the split-T combine of the oracle against what the reference's own code produced:
    `metrics.LayerReference` for the attention output of one decode query, and the closing statements of
    `dense_decode` (executed from its source by the generator) for the merge of ragged splits."""
    g = _load("attend_merge.npz")
    D, n_q, n_kv, d, T = (int(v) for v in g["dims"])
    S, V = torch.from_numpy(g["S_unscaled"]), torch.from_numpy(g["V"])
    O = po.attend(S, V, n_kv, d)
    assert float((O - torch.from_numpy(g["O"])).norm() / torch.from_numpy(g["O"]).norm()) < 2e-6
    bounds = g["bounds"].tolist()
    ms, ls, os_ = [], [], []
    for lo, hi in zip(bounds[:-1], bounds[1:]):
        m, l, o = po.partial_attend(S[:, lo:hi], V[lo:hi], n_kv, d)
        ms.append(m); ls.append(l); os_.append(o)
    m, l, o = torch.stack(ms), torch.stack(ls), torch.stack(os_)
    assert torch.allclose(m, torch.from_numpy(g["om"]), rtol=0, atol=2e-5)          # base-2 maxima of each split
    assert torch.allclose(l, torch.from_numpy(g["ol"]), rtol=2e-5, atol=0)
    assert torch.allclose(o, torch.from_numpy(g["oo"]), rtol=1e-4, atol=1e-5)
    # the merge itself on the reference's own triples: same statements, same bits
    merged = po.merge_partials(torch.from_numpy(g["om"]), torch.from_numpy(g["ol"]), torch.from_numpy(g["oo"]))
    assert torch.equal(merged, torch.from_numpy(g["merged"]))
    assert float((po.merge_partials(m, l, o) - O).norm() / O.norm()) < 2e-6


def test_per_token_v_tiers_bit_exact():
    """The oracle's per-token 3-bit and 2-bit tiers against the reference's quantize_per_token output."""
    g = _load("v_tiers.npz")
    x = torch.from_numpy(g["x"])
    for nbits in (3, 2):
        codes, scale, xhat = po.quantize_per_token(x, nbits)
        assert np.array_equal(codes.numpy(), g[f"codes{nbits}"])
        assert np.array_equal(scale.view(torch.int16).numpy(), g[f"scale{nbits}"])
        assert np.array_equal(xhat.numpy(), g[f"xhat{nbits}"])
        assert torch.equal(po.e2m1_decode(codes) * scale.float()[:, None], xhat)


def test_nvfp4_with_one_scale_per_tier_bit_exact():
    """One static tensor scale per span of the row (the reference's tiers): the oracle with a per-block scale vector
    against the reference's span-by-span quantisation."""
    g = _load("nvfp4_tiers.npz")
    x = torch.from_numpy(g["x"])
    sb = torch.zeros(x.shape[1] // 16)
    for (lo, hi), sec in zip(g["spans"].tolist(), g["seconds"].tolist()):
        sb[lo // 16:hi // 16] = sec
    codes, scales, xhat = po.nvfp4_quantize(x, sb)
    assert np.array_equal(codes.numpy(), g["codes"]) and np.array_equal(scales.numpy(), g["scales"])
    assert np.array_equal(xhat.numpy(), g["xhat"])
    assert np.array_equal(po.nvfp4_dequantize(codes, scales, sb).numpy(), g["xhat"])
