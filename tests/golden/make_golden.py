"""Generate the golden vectors under tests/golden/ by running the UNMODIFIED reference.

Run once on a machine that has the reference checked out, with its path in $PHASORKV_REFERENCE; the
produced .npz files are committed, this script is not needed to run the tests. Everything is seeded;
sizes are small so the fixtures stay a few hundred KB.

  PHASORKV_REFERENCE=<checkout of PhasorKV> python tests/golden/make_golden.py
  PHASORKV_SCALE_UP=1 PHASORKV_REFERENCE=<checkout> python tests/golden/make_golden.py   # nvfp4_cases_scale_up.npz
  PHASORKV_REFERENCE=<checkout> python tests/golden/make_golden.py attend_merge          # only the named fixtures
"""
import os
import sys

import numpy as np
import torch

REF = os.environ.get("PHASORKV_REFERENCE")
if not REF or not os.path.isdir(os.path.join(REF, "phasorkv")):
    raise SystemExit("set PHASORKV_REFERENCE to a checkout of the reference (the directory that holds phasorkv/)")
sys.path.insert(0, REF)
HERE = os.path.dirname(os.path.abspath(__file__))

from phasorkv import quant                                   # noqa: E402
from phasorkv.factorize import Factorization                 # noqa: E402
from phasorkv.kernels import nvfp4                           # noqa: E402
from phasorkv.latent import PhasorKey                        # noqa: E402
from phasorkv.rope import rope_phasors                       # noqa: E402
from transformers.models.llama.modeling_llama import apply_rotary_pos_emb   # noqa: E402


class _Rotary:
    def __init__(self, inv_freq, scale=1.0):
        self.inv_freq = inv_freq
        self.attention_scaling = scale


def nvfp4_cases():
    g = torch.Generator().manual_seed(4401)
    rows = []
    second = torch.tensor([0.0125], dtype=torch.float32)
    unit = float(second) * 1.0                                # block scale byte for 1.0 -> scale == second
    # 1. exact E2M1 midpoints (ties) in a block whose scale is exactly `second` * 1.0 (amax = 6*second)
    mids = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    tie = torch.zeros(16)
    tie[:7] = mids * unit
    tie[7:14] = -mids * unit
    tie[14] = 6.0 * unit
    tie[15] = -6.0 * unit
    rows.append(tie)
    # 2. all-zero block, 3. tiny values that round to zero with a sign, 4. saturation of the block scale
    rows.append(torch.zeros(16))
    small = torch.zeros(16); small[0] = 6.0 * unit; small[1:] = -0.2 * unit
    rows.append(small)
    sat = torch.randn(16, generator=g) * 1e4
    rows.append(sat)
    # 5. scales in the E4M3 subnormal range and below (2^-9 steps; 2^-10 ties to zero)
    for e in (-6, -7, -8, -9, -10, -11):
        blk = torch.randn(16, generator=g)
        blk = blk / blk.abs().max() * 6.0 * float(second) * 2.0 ** e
        rows.append(blk)
    # 6. scale ties in E4M3 (halfway between two scale codes)
    for s in (1.0625, 1.1875, 17.0, 19.0, 0.001953125 * 1.5):
        blk = torch.randn(16, generator=g)
        blk = blk / blk.abs().max() * 6.0 * float(second) * s
        rows.append(blk)
    special = torch.stack(rows)                              # [n, 16]
    pad = (-special.shape[0]) % 4
    special = torch.cat([special, torch.zeros(pad, 16)])
    special = special.reshape(-1, 64)
    # 7. random rows over many decades
    mag = torch.exp(torch.randn(96, 1, generator=g) * 3.0)
    rnd = torch.randn(96, 64, generator=g) * mag * float(second)
    x = torch.cat([special, rnd]).float()
    codes, s, xhat = nvfp4.quantize_nv_block(x, "nvfp4", second)
    fake = quant.block_quant(x, "nvfp4", -1, second)
    assert torch.equal(fake, xhat)
    out = dict(x=x.numpy(), second=second.numpy(), codes=codes.numpy(),
               scales=s.view(torch.uint8).numpy(), xhat=xhat.numpy(),
               packed=nvfp4.pack_nibbles(codes).numpy())
    # dynamic second (quant.block_quant default) and the static rule
    out["second_dynamic"] = (x.abs().amax().clamp_min(1e-30) / (448.0 * 6.0)).reshape(1).numpy()
    var = torch.rand(64, generator=g) * 3.0
    out["static_var"] = var.numpy()
    out["static_second"] = quant.nv_static_second(var, "nvfp4").numpy()
    if quant.SCALE_UP:                                        # the reference reads PHASORKV_SCALE_UP once, at import
        keep = ("x", "second", "codes", "scales", "xhat", "packed")
        np.savez_compressed(os.path.join(HERE, "nvfp4_cases_scale_up.npz"), **{k: out[k] for k in keep})
        print("nvfp4_cases_scale_up", x.shape)
        return
    np.savez_compressed(os.path.join(HERE, "nvfp4_cases.npz"), **out)
    print("nvfp4_cases", x.shape)


def inject(A, B, freq, n_q, n_kv, h, A_s=None, B_s=None, slow=None):
    pk = object.__new__(PhasorKey)
    pk.A, pk.B, pk.freq = A, B, freq
    pk.A_s, pk.B_s = A_s, B_s
    pk.slow = slow if slow is not None else torch.zeros(0, dtype=torch.long)
    pk.n_q, pk.n_kv, pk.h = n_q, n_kv, h
    pk.R = B.shape[0]
    pk.R_s = 0 if B_s is None else B_s.shape[0]
    return pk


def phasorkey_injected():
    """Reference PhasorKey on injected random factors (the benchmark configurations' convention)."""
    g = torch.Generator().manual_seed(4402)
    D, n_q, n_kv, d = 192, 8, 2, 64
    h = d // 2
    T, Tq = 40, 3
    inv_freq = torch.pow(torch.tensor(500000.0, dtype=torch.float64), -2.0 * torch.arange(h, dtype=torch.float64) / d)
    out = {}
    for tag, n_slow in (("freq", 0), ("band", 4)):
        ranks = torch.randint(0, 4, (h - n_slow,), generator=g)
        ranks[0] = 2
        freq = torch.repeat_interleave(torch.arange(h - n_slow), ranks)
        R = freq.numel()
        A = torch.complex(torch.randn(n_kv, R, generator=g), torch.randn(n_kv, R, generator=g)) * 0.3
        B = torch.complex(torch.randn(R, D, generator=g), torch.randn(R, D, generator=g)) * 0.05
        A_s = B_s = slow = None
        if n_slow:
            R_s = 8
            slow = torch.arange(h - n_slow, h)
            A_s = torch.randn(n_kv, 2 * n_slow, R_s, generator=g) * 0.3
            B_s = torch.randn(R_s, D, generator=g) * 0.05
        pk = inject(A, B, freq, n_q, n_kv, h, A_s, B_s, slow)
        pos_k = torch.tensor([0, 1, 2, 3, 5, 17, 255, 4095, 4096, 29999, 30000, 65535, 131071] + list(range(100000, 100027)))
        pos_q = torch.tensor([4096, 30000, 131072])
        rot = _Rotary(inv_freq, 1.0)
        ph_k = rope_phasors(rot, pos_k)
        ph_q = rope_phasors(rot, pos_q)
        x = torch.randn(T, D, generator=g)
        q = torch.randn(n_q, Tq, d, generator=g)
        rows = pk.write(x, ph_k)
        qa = pk.absorb(q, ph_q)
        S = pk.scores(qa, rows)
        out.update({f"{tag}_A": A.numpy(), f"{tag}_B": B.numpy(), f"{tag}_freq": freq.numpy(),
                    f"{tag}_x": x.numpy(), f"{tag}_q": q.numpy(), f"{tag}_pos_k": pos_k.numpy(),
                    f"{tag}_pos_q": pos_q.numpy(), f"{tag}_ph_k": ph_k.numpy(), f"{tag}_ph_q": ph_q.numpy(),
                    f"{tag}_rows": rows.numpy(), f"{tag}_qabs": qa.numpy(), f"{tag}_scores": S.numpy()})
        if n_slow:
            out.update({f"{tag}_A_s": A_s.numpy(), f"{tag}_B_s": B_s.numpy(), f"{tag}_slow": slow.numpy()})
    out["inv_freq"] = inv_freq.numpy()
    out["dims"] = np.array([D, n_q, n_kv, d])
    np.savez_compressed(os.path.join(HERE, "phasorkey_injected.npz"), **out)
    print("phasorkey_injected")


def phasorkey_factorized():
    """Reference Factorization -> PhasorKey (fp64) and the W_hat + HF-rotary identity (README.md:75-77)."""
    g = torch.Generator().manual_seed(4403)
    D, n_q, n_kv, d = 96, 8, 2, 32
    h = d // 2
    T, Tq = 24, 2
    inv_freq = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * torch.arange(h, dtype=torch.float64) / d)
    W = torch.randn(n_kv * d, D, generator=g, dtype=torch.float64) / D ** 0.5
    X = torch.randn(4 * D, D, generator=g, dtype=torch.float64)
    Cx = X.T @ X / X.shape[0]
    q2 = torch.rand(n_q, d, generator=g, dtype=torch.float64) + 0.1
    out = dict(inv_freq=inv_freq.numpy(), dims=np.array([D, n_q, n_kv, d]))
    rot = _Rotary(inv_freq, 1.0)
    pos_k = torch.arange(29976, 30000)
    pos_q = torch.tensor([30000, 30001])
    ph_k, ph_q = rope_phasors(rot, pos_k), rope_phasors(rot, pos_q)
    x = torch.randn(T, D, generator=g, dtype=torch.float64)
    q = torch.randn(n_q, Tq, d, generator=g, dtype=torch.float64)
    for tag, structure in (("freq", "freq"), ("band", "band4")):
        fac = Factorization(W, Cx, q2, n_kv, d, structure, "xq", device="cpu")
        ranks = fac.ranks(fac.full_size // 2)
        pk = PhasorKey(fac, ranks, n_q)
        rows = pk.write(x, ph_k)
        qa = pk.absorb(q, ph_q)
        S = pk.scores(qa, rows)
        W_hat = fac.reconstruct(ranks)
        # rebuild keys with W_hat and rotate with HF's own function; slow frequencies unrotated
        pk_, pq_ = ph_k.clone(), ph_q.clone()
        if fac.nope.any():
            pk_[:, fac.nope] = pk_[0, 0].abs().to(pk_.dtype)
            pq_[:, fac.nope] = pq_[0, 0].abs().to(pq_.dtype)
        k = (x @ W_hat.T).reshape(T, n_kv, d).transpose(0, 1)[None]               # [1, n_kv, T, d]
        cos_k, sin_k = torch.cat([pk_.real, pk_.real], -1)[None], torch.cat([pk_.imag, pk_.imag], -1)[None]
        cos_q, sin_q = torch.cat([pq_.real, pq_.real], -1)[None], torch.cat([pq_.imag, pq_.imag], -1)[None]
        _, kr = apply_rotary_pos_emb(k, k, cos_k, sin_k)
        qr, _ = apply_rotary_pos_emb(q[None], q[None], cos_q, sin_q)
        S2 = qr[0] @ kr[0].repeat_interleave(n_q // n_kv, dim=0).transpose(1, 2)
        rel = ((S - S2).norm() / S2.norm()).item()
        print(tag, "ranks", ranks, "identity rel", rel)
        assert rel < 1e-12
        # the block data PhasorKey.__init__ consumes (factorize.Block fields), for the constructor check
        out[f"{tag}_ranks"] = np.array(ranks)
        out[f"{tag}_nope"] = fac.nope.numpy()
        for bi, blk in enumerate(fac.blocks):
            out[f"{tag}_blk{bi}_U"] = blk.U.numpy()
            out[f"{tag}_blk{bi}_s2"] = blk.s2.numpy()
            out[f"{tag}_blk{bi}_sq"] = blk.sq.numpy()
            out[f"{tag}_blk{bi}_Mw"] = blk.Mw.numpy()
            out[f"{tag}_blk{bi}_cost"] = np.array(blk.cost)
            out[f"{tag}_blk{bi}_where"] = np.array(blk.where if blk.cost == 2 else -1)
        out[f"{tag}_nblocks"] = np.array(len(fac.blocks))
        out[f"{tag}_energy"] = pk.energy.numpy()
        out.update({f"{tag}_A": pk.A.numpy(), f"{tag}_B": pk.B.numpy(), f"{tag}_freq": pk.freq.numpy(),
                    f"{tag}_rows": rows.numpy(), f"{tag}_qabs": qa.numpy(), f"{tag}_scores": S.numpy(),
                    f"{tag}_W_hat": W_hat.numpy(), f"{tag}_scores_hf": S2.numpy(),
                    f"{tag}_slow": pk.slow.numpy()})
        if pk.R_s:
            out.update({f"{tag}_A_s": pk.A_s.numpy(), f"{tag}_B_s": pk.B_s.numpy()})
    out.update(x=x.numpy(), q=q.numpy(), pos_k=pos_k.numpy(), pos_q=pos_q.numpy(),
               ph_k=ph_k.numpy(), ph_q=ph_q.numpy())
    np.savez_compressed(os.path.join(HERE, "phasorkey_factorized.npz"), **out)
    print("phasorkey_factorized")


def attend_merge():
    """Softmax . V as the reference forms it (metrics.LayerReference: logits * d^-0.5, log_softmax, P @ V with
    the kv heads repeated over their query heads, phasorkv/metrics.py:23,29-35) for one decode query over T
    tokens, and the split-T combine: the three statements that close dense_decode
    (phasorkv/kernels/dense_attn.py:72-74) are taken from its source and executed here on per-split
    (max, sum, output) triples in base 2, which is how its kernel leaves them (LOG2E in qk_scale, :68)."""
    import inspect
    import textwrap
    from phasorkv import metrics
    from phasorkv.kernels import dense_attn
    g = torch.Generator().manual_seed(4404)
    D, n_q, n_kv, d, T = 64, 8, 2, 32, 96
    h = d // 2
    inv_freq = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * torch.arange(h, dtype=torch.float64) / d)
    ph = rope_phasors(_Rotary(inv_freq, 1.0), torch.arange(T))
    x = torch.randn(T, D, generator=g)
    Wq = torch.randn(n_q * d, D, generator=g) * 0.6 / D ** 0.5            # peaked enough that the split maxima differ
    Wk = torch.randn(n_kv * d, D, generator=g) * 4.0 / D ** 0.5
    Wv = torch.randn(n_kv * d, D, generator=g) / D ** 0.5
    qpos = torch.tensor([T - 1])                                           # one query row that sees every token
    ref = metrics.LayerReference([x], Wq, Wk, Wv, ph.to(torch.complex64), qpos, n_kv, d)
    it = ref.items[0]
    S_scaled = it["S"][:, 0]                                               # [H, T] logits * d^-0.5
    O = it["O"][:, 0]                                                      # [H, d]
    V = (x @ Wv.T).reshape(T, n_kv, d)                                     # [T, n_kv, d] before the head expansion
    S_unscaled = S_scaled / ref.scale
    # per-split triples in base 2 over ragged splits, then the reference's own merge statements
    bounds = [0, 17, 48, 49, T]
    s2 = S_scaled.double() * dense_attn.LOG2E
    Vh = it["v"].double()                                                  # [H, T, d]
    om, ol, oo = [], [], []
    for lo, hi in zip(bounds[:-1], bounds[1:]):
        m = s2[:, lo:hi].amax(-1)
        p = torch.exp2(s2[:, lo:hi] - m[:, None])
        om.append(m); ol.append(p.sum(-1)); oo.append(torch.einsum("ht,htd->hd", p, Vh[:, lo:hi]))
    om, ol, oo = torch.stack(om)[None].float(), torch.stack(ol)[None].float(), torch.stack(oo)[None].float()   # [1, S, H(, d)]
    tail = inspect.getsource(dense_attn.dense_decode).rstrip().splitlines()[-3:]
    code = textwrap.dedent("\n".join(tail)).replace("return ", "merged = ")
    assert code.count("merged = ") == 1 and "torch.exp2(om - M)" in code, code
    ns = dict(torch=torch, om=om, ol=ol, oo=oo)
    exec(code, ns)
    merged = ns["merged"][0]                                               # [H, d]
    err = ((merged.double() - O.double()).norm() / O.double().norm()).item()
    print("attend_merge: merged splits vs LayerReference O", err)
    assert err < 1e-5
    np.savez_compressed(os.path.join(HERE, "attend_merge.npz"), S_unscaled=S_unscaled.numpy(), S_scaled=S_scaled.numpy(),
                        V=V.numpy(), O=O.numpy(), lp=it["lp"][:, 0].numpy(), bounds=np.array(bounds), om=om[0].numpy(),
                        ol=ol[0].numpy(), oo=oo[0].numpy(), merged=merged.numpy(), dims=np.array([D, n_q, n_kv, d, T]))
    print("attend_merge")


def phasorkey_llama_heads():
    """A real Factorization(..., "band8", "xq") at the Llama-3.1-8B head shape (32 query heads, 8 kv heads,
    head_dim 128, rope base 500000; d_model cut to 512 to keep the fixture small) with water-filled ranks at 25 %
    of K: the arrays PhasorKey builds from it, its write / absorb / scores on seeded inputs at long positions, and
    the scores from keys rebuilt with W_hat and rotated by HF's apply_rotary_pos_emb (slow band unrotated)."""
    g = torch.Generator().manual_seed(4406)
    D, n_q, n_kv, d = 512, 32, 8, 128
    h = d // 2
    T = 200
    inv_freq = torch.pow(torch.tensor(500000.0, dtype=torch.float64), -2.0 * torch.arange(h, dtype=torch.float64) / d)
    W = torch.randn(n_kv * d, D, generator=g, dtype=torch.float64) / D ** 0.5
    W *= torch.exp(-torch.arange(D, dtype=torch.float64) / 96.0)[None, :] * 4.0      # a falling spectrum: low ranks carry most
    X = torch.randn(4 * D, D, generator=g, dtype=torch.float64)
    Cx = X.T @ X / X.shape[0]
    q2 = torch.rand(n_q, d, generator=g, dtype=torch.float64) + 0.1
    fac = Factorization(W, Cx, q2, n_kv, d, "band8", "xq", device="cpu")
    ranks = fac.ranks(fac.full_size // 4)
    pk = PhasorKey(fac, ranks, n_q)
    rot = _Rotary(inv_freq, 1.0)
    pos_k = torch.arange(T) + 100000
    pos_q = torch.tensor([100000 + T])
    ph_k, ph_q = rope_phasors(rot, pos_k), rope_phasors(rot, pos_q)
    x = torch.randn(T, D, generator=g, dtype=torch.float64)
    q = torch.randn(n_q, 1, d, generator=g, dtype=torch.float64)
    rows, qa = pk.write(x, ph_k), pk.absorb(q, ph_q)
    S = pk.scores(qa, rows)
    W_hat = fac.reconstruct(ranks)
    pk_, pq_ = ph_k.clone(), ph_q.clone()
    pk_[:, fac.nope] = pk_[0, 0].abs().to(pk_.dtype)
    pq_[:, fac.nope] = pq_[0, 0].abs().to(pq_.dtype)
    k = (x @ W_hat.T).reshape(T, n_kv, d).transpose(0, 1)[None]
    cos_k, sin_k = torch.cat([pk_.real, pk_.real], -1)[None], torch.cat([pk_.imag, pk_.imag], -1)[None]
    cos_q, sin_q = torch.cat([pq_.real, pq_.real], -1)[None], torch.cat([pq_.imag, pq_.imag], -1)[None]
    _, kr = apply_rotary_pos_emb(k, k, cos_k, sin_k)
    qr, _ = apply_rotary_pos_emb(q[None], q[None], cos_q, sin_q)
    S2 = qr[0] @ kr[0].repeat_interleave(n_q // n_kv, dim=0).transpose(1, 2)
    rel = ((S - S2).norm() / S2.norm()).item()
    print("llama heads: ranks sum", sum(ranks), "R", pk.R, "R_s", pk.R_s, "width", pk.cache_width, "identity rel", rel)
    assert rel < 1e-12 and pk.cache_width <= 256
    np.savez_compressed(os.path.join(HERE, "phasorkey_llama_heads.npz"), dims=np.array([D, n_q, n_kv, d]), inv_freq=inv_freq.numpy(),
                        ranks=np.array(ranks), A=pk.A.to(torch.complex64).numpy(), B=pk.B.to(torch.complex64).numpy(),
                        freq=pk.freq.numpy(), slow=pk.slow.numpy(), A_s=pk.A_s.float().numpy(), B_s=pk.B_s.float().numpy(),
                        x=x.float().numpy(), q=q.float().numpy(), pos_k=pos_k.numpy(), pos_q=pos_q.numpy(),
                        rows=rows.float().numpy(), qabs=qa.float().numpy(), scores=S.float().numpy(), scores_hf=S2.float().numpy())
    print("phasorkey_llama_heads")


def nvfp4_tiers():
    """NVFP4 with one static tensor scale per tier: the reference's cache write quantises every span of the latent
    row on its own (kernels/latent_attn.write: quantize_nv_block per k_tier with quant.nv_static_second of the span's
    variances). Spans of a falling spectrum, so that the scales differ by orders of magnitude."""
    g = torch.Generator().manual_seed(4407)
    W, n = 256, 96
    sigma = torch.exp(-torch.arange(W) / 40.0)
    x = torch.randn(n, W, generator=g) * sigma[None, :]
    spans = [(0, 32), (32, 96), (96, 240), (240, 256)]
    var = x.var(0)
    codes = torch.zeros(n, W, dtype=torch.uint8)
    scales = torch.zeros(n, W // 16, dtype=torch.float8_e4m3fn)
    xhat = torch.zeros(n, W)
    seconds = []
    for lo, hi in spans:
        sec = quant.nv_static_second(var[lo:hi], "nvfp4")
        c, s, h = nvfp4.quantize_nv_block(x[:, lo:hi], "nvfp4", sec)
        codes[:, lo:hi], scales[:, lo // 16:hi // 16], xhat[:, lo:hi] = c, s, h
        seconds.append(float(sec))
    np.savez_compressed(os.path.join(HERE, "nvfp4_tiers.npz"), x=x.numpy(), spans=np.array(spans), seconds=np.array(seconds, dtype=np.float32),
                        codes=codes.numpy(), scales=scales.view(torch.uint8).numpy(), xhat=xhat.numpy(),
                        packed=nvfp4.pack_nibbles(codes).numpy())
    print("nvfp4_tiers", seconds)


def v_tiers():
    """Per-token low-bit tiers of the reference (kernels/nvfp4.quantize_per_token) on rows of 128 values, the
    shape of one (token, kv head) value row: 3-bit and 2-bit, with ties, an all-zero row, a row below the
    1e-5 floor, large and tiny magnitudes."""
    g = torch.Generator().manual_seed(4405)
    rows = [torch.randn(128, generator=g) * m for m in (1.0, 0.02, 37.0, 1e-3, 4e3)]
    rows += [torch.zeros(128), torch.full((128,), 3e-6)]
    tie = torch.zeros(128)
    tie[0] = 3.0                                               # scale exactly 1: x / s lands on .5 ties and the clamp
    tie[1:9] = torch.tensor([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, -3.5, -4.2])
    rows.append(tie)
    tie2 = torch.zeros(128)
    tie2[0] = 1.5
    tie2[1:7] = torch.tensor([1.0, -1.0, 0.999, 1.001, 0.0, -0.0])
    rows.append(tie2)
    x = torch.cat([torch.stack(rows), torch.randn(64, 128, generator=g) * torch.exp(torch.randn(64, 1, generator=g) * 2)])
    x = x.to(torch.bfloat16).float()                           # value rows are bf16 where this format is used
    out = dict(x=x.numpy())
    for nbits in (3, 2):
        codes, scale, xhat = nvfp4.quantize_per_token(x, nbits)
        out[f"codes{nbits}"] = codes.numpy()
        out[f"scale{nbits}"] = scale.view(torch.int16).numpy()          # bf16 bit patterns
        out[f"xhat{nbits}"] = xhat.numpy()
    np.savez_compressed(os.path.join(HERE, "v_tiers.npz"), **out)
    print("v_tiers", x.shape)


if __name__ == "__main__":
    torch.set_num_threads(4)
    only = set(sys.argv[1:])                                  # optional: names of the fixtures to (re)write
    want = lambda name: not only or name in only
    if want("nvfp4_cases"):
        nvfp4_cases()
    if not quant.SCALE_UP:                                    # PHASORKV_SCALE_UP=1: only the quantiser vectors differ
        if want("phasorkey_injected"):
            phasorkey_injected()
        if want("phasorkey_factorized"):
            phasorkey_factorized()
        if want("attend_merge"):
            attend_merge()
        if want("v_tiers"):
            v_tiers()
        if want("nvfp4_tiers"):
            nvfp4_tiers()
        if want("phasorkey_llama_heads"):
            phasorkey_llama_heads()
