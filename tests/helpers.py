"""Shared scenario builder for the GPU parity tests: one layer, a ragged batch of sequences written
through the CUDA path, and the oracle's view of the same data."""
from __future__ import annotations

import types

import torch

from oracle import phasor_oracle as po
from phasorkv_b200 import synth
from phasorkv_b200.latent import PhasorKey


class Scenario:
    def __init__(self, config="cfg2", seqlens=(300,), layer=0, gain=1.0, seed=11, d_model=4096, pos0=0,
                 fused_write=True, x_dtype=torch.float32, v_bits=0, n_kv=None):
        self.spec = synth.make_layer(config, layer, d_model=d_model, factor_gain=gain, n_kv=n_kv)
        self.pk = PhasorKey.from_spec(self.spec, device="cuda")
        self.opk = po.PhasorKeyOracle.from_spec(self.spec)
        self.seqlens = list(seqlens)
        self.B = len(self.seqlens)
        gen = torch.Generator().manual_seed(seed)
        spec = self.spec
        # calibration of the tensor scale from a seeded oracle write (static rule of the reference)
        xc = synth.make_hidden(gen, 256, d_model)
        rows_c = self.opk.write(xc, po.rope_phasors(spec.inv_freq, torch.arange(256)))
        self.second = float(po.nv_static_second(rows_c.var(0)))
        self.pk.set_second(self.second)
        Tmax = max(max(self.seqlens), 1)
        self.cache = self.pk.new_cache(self.B, Tmax, v_bits=v_bits)
        self.x, self.v, self.pos, self.rows_ref = [], [], [], []
        for b, T in enumerate(self.seqlens):
            x = synth.make_hidden(gen, T, d_model).to(x_dtype)
            v = synth.make_values(gen, T, spec.n_kv, spec.head_dim)
            pos = torch.arange(T) + pos0
            self.x.append(x); self.v.append(v); self.pos.append(pos)
            rows = self.opk.write(x.float(), po.rope_phasors(spec.inv_freq, pos, spec.attn_scale)) if T else torch.zeros(0, spec.cache_width)
            self.rows_ref.append(rows)
            if T == 0:
                continue
            seq = torch.full((T,), b, dtype=torch.int32, device="cuda")
            lp = torch.arange(T, dtype=torch.int32, device="cuda")
            slots = self.cache.slots(seq, lp)
            if fused_write:
                self.pk.write_paged(self.cache, x.cuda(), pos.to(torch.int32).cuda(), slots, v=v.cuda())
            else:
                self.cache.quantize_rows(rows.cuda(), slots, self.second)
                self.cache.write_v(v.cuda(), slots)
        self.cache.seqlens.copy_(torch.tensor(self.seqlens, dtype=torch.int32))
        self.q = synth.make_query(gen, self.B, spec.n_q, spec.head_dim)
        self.qpos = torch.tensor([T + pos0 for T in self.seqlens], dtype=torch.int32)

    def slots_of(self, b):
        T = self.seqlens[b]
        seq = torch.full((T,), b, dtype=torch.int32, device="cuda")
        return self.cache.slots(seq, torch.arange(T, dtype=torch.int32, device="cuda"))

    def dequantised(self, b):
        """What the device cache holds for sequence b, as fp32 rows on the CPU."""
        rows, _, _ = self.cache.read(self.slots_of(b), self.second, codes=False)
        return rows.cpu()

    def oracle_scores_and_output(self, b, rows, V=None):
        """Oracle absorbed query, scores and output of sequence b on the given cache rows (and value rows V
        [T, n_kv, d]; default: the values the scenario wrote)."""
        spec = self.spec
        ph = po.rope_phasors(spec.inv_freq, self.qpos[b:b + 1], spec.attn_scale)
        qa = self.opk.absorb(self.q[b][:, None, :], ph)[:, 0]
        S = self.opk.scores(qa, rows)
        O = po.attend(S, self.v[b] if V is None else V, spec.n_kv, spec.head_dim)
        return qa, S, O


def rel(a: torch.Tensor, b: torch.Tensor) -> float:
    """Frobenius-norm relative error of a against b."""
    return float((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-300))


class Blk(types.SimpleNamespace):
    """One block of a reference Factorization (phasorkv/factorize.py:56-63): U, s2, sq, Mw, where, cost."""


def fac_from_golden(g, tag):
    """A Factorization-like object rebuilt from the block data that tests/golden/make_golden.py stored from a
    reference `Factorization`; returns (fac, n_q)."""
    blocks = []
    for bi in range(int(g[f"{tag}_nblocks"])):
        t = lambda k: torch.from_numpy(g[f"{tag}_blk{bi}_{k}"])
        blocks.append(Blk(U=t("U"), s2=t("s2"), sq=t("sq"), Mw=t("Mw"), cost=int(g[f"{tag}_blk{bi}_cost"]),
                          where=int(g[f"{tag}_blk{bi}_where"])))
    D, n_q, n_kv, d = (int(v) for v in g["dims"])
    return types.SimpleNamespace(blocks=blocks, n_kv=n_kv, d=d, absorbed=True, nope=torch.from_numpy(g[f"{tag}_nope"])), n_q
