"""Seeded synthetic layers and activations with the shapes of the benchmark configurations.

The reference measures its latent kernels on random factors and random caches
(scripts/bench_decode.py:4-8, phasorkv/kernels/latent_attn.py:171-201) and has no public data
set on the PhasorKey path, so every input here is drawn from ``torch.Generator().manual_seed``.
A layer is described by the same arrays ``phasorkv.latent.PhasorKey`` exposes after construction
(phasorkv/latent.py:47-54): ``A [n_kv, R]`` and ``B [R, D]`` complex, ``freq [R]``, and for the
band layouts the real slow block ``A_s [n_kv, 2*n_slow, R_s]``, ``B_s [R_s, D]``, ``slow``.
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch


@dataclasses.dataclass
class LayerSpec:
    """Factors of one layer in PhasorKey's attribute convention (phasorkv/latent.py:47-54)."""
    d_model: int
    n_q: int
    n_kv: int
    head_dim: int
    inv_freq: torch.Tensor            # float64 [head_dim/2], fastest frequency first (HF order)
    A: torch.Tensor                   # complex64 [n_kv, R]
    B: torch.Tensor                   # complex64 [R, D]
    freq: torch.Tensor                # int64 [R]  frequency index of each complex latent dim
    A_s: Optional[torch.Tensor] = None   # float32 [n_kv, 2*n_slow, R_s]
    B_s: Optional[torch.Tensor] = None   # float32 [R_s, D]
    slow: Optional[torch.Tensor] = None  # int64 [n_slow] frequencies scored without RoPE
    attn_scale: float = 1.0

    @property
    def R(self) -> int:
        return int(self.B.shape[0])

    @property
    def R_s(self) -> int:
        return 0 if self.B_s is None else int(self.B_s.shape[0])

    @property
    def h(self) -> int:
        return self.head_dim // 2

    @property
    def cache_width(self) -> int:
        return 2 * self.R + self.R_s


#: name -> (n_q, n_kv, rope base, layout, batch, context)
CONFIGS = {
    "cfg1": dict(n_q=32, n_kv=8, base=500000.0, layout="freq2", batch=1, context=4096, quant=False),
    "cfg2": dict(n_q=32, n_kv=8, base=500000.0, layout="freq2", batch=16, context=32768, quant=True),
    "cfg3": dict(n_q=32, n_kv=8, base=500000.0, layout="band8", batch=32, context=16384, quant=True),
    "cfg4": dict(n_q=32, n_kv=8, base=500000.0, layout="freq2", batch=4, context=131072, quant=True),
    "cfg5": dict(n_q=32, n_kv=32, base=10000.0, layout="freq1", batch=64, context=32768, quant=True,
                 chunk=2048),
}
CONFIG_INDEX = {"cfg1": 1, "cfg2": 2, "cfg3": 3, "cfg4": 4, "cfg5": 5}


def rope_inv_freq(head_dim: int, base: float) -> torch.Tensor:
    """theta_j = base^(-2j/head_dim), j = 0..head_dim/2-1, in float64 (HF order: fastest first)."""
    j = torch.arange(head_dim // 2, dtype=torch.float64)
    return torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * j / head_dim)


def _cnormal(gen, shape, var):
    s = (var / 2.0) ** 0.5
    re = torch.randn(shape, generator=gen, dtype=torch.float32) * s
    im = torch.randn(shape, generator=gen, dtype=torch.float32) * s
    return torch.complex(re, im)


def band_ranks(gen, n_fast: int = 56, total: int = 120, rmax: int = 6) -> list[int]:
    """Water-filled stand-in: round(total * Dirichlet(1)) clipped to 0..rmax, repaired to sum `total`."""
    # a seeded Dirichlet(1,...,1) draw: normalised exponentials from the given generator
    e = -torch.log(torch.rand(n_fast, generator=gen, dtype=torch.float64).clamp_min(1e-300))
    w = e / e.sum()
    r = torch.clamp(torch.round(total * w), 0, rmax).to(torch.int64)
    order = torch.argsort(w, descending=True).tolist()
    i = 0
    while int(r.sum()) != total:                       # repair: walk the frequencies by weight
        j = order[i % n_fast]
        if int(r.sum()) < total and r[j] < rmax:
            r[j] += 1
        elif int(r.sum()) > total and r[j] > 0:
            r[j] -= 1
        i += 1
    return r.tolist()


def make_layer(config: str, layer: int = 0, d_model: int = 4096, head_dim: int = 128,
               factor_gain: float = 1.0, n_q: Optional[int] = None, n_kv: Optional[int] = None) -> LayerSpec:
    """Seeded factors of one layer; seed = 1000*config_index + layer.

    Entries of A_j and B_j are i.i.d. complex normal with E|.|^2 = 1/4096 (the reference's
    synthetic packs scale by 1/sqrt(D) likewise, phasorkv/kernels/latent_attn.py:193).
    ``factor_gain`` multiplies A (a stress variant that makes the softmax peaked).
    """
    c = CONFIGS[config]
    n_q = c["n_q"] if n_q is None else n_q
    n_kv = c["n_kv"] if n_kv is None else n_kv
    gen = torch.Generator().manual_seed(1000 * CONFIG_INDEX[config] + layer)
    h = head_dim // 2
    var = 1.0 / 4096.0
    A_s = B_s = slow = None
    if c["layout"] == "band8":
        n_slow, R_s = 8, 16
        ranks = band_ranks(gen) + [0] * n_slow
        slow = torch.arange(h - n_slow, h)
        A_s = torch.randn((n_kv, 2 * n_slow, R_s), generator=gen) * var ** 0.5 * factor_gain
        B_s = torch.randn((R_s, d_model), generator=gen) * var ** 0.5
    else:
        ranks = [int(c["layout"][4:])] * h
    freq = torch.repeat_interleave(torch.arange(h), torch.tensor(ranks))
    R = int(freq.numel())
    A = _cnormal(gen, (n_kv, R), var) * factor_gain
    B = _cnormal(gen, (R, d_model), var)
    return LayerSpec(d_model, n_q, n_kv, head_dim, rope_inv_freq(head_dim, c["base"]), A, B, freq,
                     A_s, B_s, slow)


def make_hidden(gen: torch.Generator, n_tokens: int, d_model: int = 4096,
                outlier_frac: float = 0.01, outlier_gain: float = 20.0) -> torch.Tensor:
    """x_t ~ N(0,1) with a seeded 1 % of channels multiplied by 20 (outlier channels)."""
    n_out = max(1, int(round(outlier_frac * d_model)))
    ch = torch.randperm(d_model, generator=gen)[:n_out]
    x = torch.randn((n_tokens, d_model), generator=gen, dtype=torch.float32)
    x[:, ch] *= outlier_gain
    return x


def make_query(gen: torch.Generator, batch: int, n_q: int = 32, head_dim: int = 128) -> torch.Tensor:
    return torch.randn((batch, n_q, head_dim), generator=gen, dtype=torch.float32)


def make_values(gen: torch.Generator, n_tokens: int, n_kv: int = 8, head_dim: int = 128) -> torch.Tensor:
    return torch.randn((n_tokens, n_kv, head_dim), generator=gen, dtype=torch.float32).to(torch.bfloat16)
