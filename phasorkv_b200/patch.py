"""Per-layer patch object for the B200 PhasorKey path.

The reference drives every KV method through one duck-typed protocol
(phasorkv/kvmethods.py:457,1032,1071; caller phasorkv/runner.py:89-107): an object with

    name                                     identifies the method in result tables
    layer_stats[i] = {bits_k, bits_v, ...}   cache bits per token, read by kvmethods.compression
    patch(i, layer, prep, n_kv, d, n_q, device) -> undo      undo() takes no argument

This class keeps that protocol. ``patch`` builds the layer's ``PhasorKey`` from ``prep`` and hangs it
on the attention module as ``layer.self_attn.phasor_key`` (with the layer index as
``phasor_layer``); ``undo`` removes both. ``prep`` is either a ready ``PhasorKey``, a
``synth.LayerSpec``, or a mapping with ``fac`` and ``ranks`` (the reference's ``Factorization``
and its water-filled ranks) and optionally ``inv_freq`` / ``second``.
"""
from __future__ import annotations

from .latent import PhasorKey

NVFP4_BITS = 4.5          # E2M1 code + one E4M3 scale per 16 codes (phasorkv/quant.py:9)


class PhasorKeyPatch:
    def __init__(self, tag: str = "phasor.nvfp4", bits_v: float = 16.0):
        self.tag = tag
        self.bits_v = bits_v
        self.layer_stats = {}
        self.keys = {}

    @property
    def name(self) -> str:
        return self.tag

    def patch(self, i, layer, prep, n_kv, d, n_q, device):
        if isinstance(prep, PhasorKey):
            pk = prep
        elif hasattr(prep, "cache_width") and hasattr(prep, "inv_freq"):          # synth.LayerSpec
            pk = PhasorKey.from_spec(prep, device=device)
        else:
            pk = PhasorKey(prep["fac"], prep["ranks"], n_q, inv_freq=prep.get("inv_freq"),
                           attn_scale=prep.get("attn_scale", 1.0), device=device)
            if "second" in prep:
                pk.set_second(prep["second"])
        if pk.n_kv != n_kv or pk.head_dim != d or pk.n_q != n_q:
            raise ValueError(f"layer {i}: factors are for (n_q, n_kv, d) = ({pk.n_q}, {pk.n_kv}, {pk.head_dim}), "
                             f"the model has ({n_q}, {n_kv}, {d})")
        attn = layer.self_attn
        had = (getattr(attn, "phasor_key", None), getattr(attn, "phasor_layer", None))
        attn.phasor_key, attn.phasor_layer = pk, i
        self.keys[i] = pk
        self.layer_stats[i] = dict(bits_k=NVFP4_BITS * pk.cache_width, bits_v=self.bits_v * n_kv * d,
                                   width=pk.cache_width, R=pk.R, R_s=pk.R_s)

        def undo():
            attn.phasor_key, attn.phasor_layer = had
            if had[0] is None:
                del attn.phasor_key, attn.phasor_layer
        return undo
