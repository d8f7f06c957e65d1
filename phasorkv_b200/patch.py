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

With ``install_forward=True`` the patch also replaces the forward of a Hugging Face Llama attention
module (``hidden_states, position_embeddings, attention_mask, past_key_values, **kwargs`` ->
``(attn_output, None)``), the way the reference's patches wrap ``self_attn.forward``
(phasorkv/kvmethods.py:560-611):

  prefill (more than one query token)  the module's own forward computes the output with exact keys;
                                       beside it every token's rotated latent and V row go into this
                                       layer's paged caches (``write_paged``, chunked),
  decode (one query token)             ``prologue_step`` (write + absorb) -> ``attend_step`` ->
                                       ``o_proj``: keys are never rebuilt, the Hugging Face KV cache
                                       is not touched.

Positions are counted by the layer's own cache (``seqlens``, one length per sequence), so the caller runs
the model with ``use_cache=False`` and feeds one new token per sequence and decode call. A ragged batch is
prefilled right-padded with ``attn.kv_lengths`` set to the valid token counts, the contract of the reference's
runner (phasorkv/runner.py:94-99); a decode step then places every sequence's token at its own position. ``undo`` restores the original forward
and drops the caches.
"""
from __future__ import annotations

from typing import Optional

import torch

from .latent import PAGE_TOKENS, PhasorKey

NVFP4_BITS = 4.5          # E2M1 code + one E4M3 scale per 16 codes (phasorkv/quant.py:9)


class LayerDecodeState:
    """Paged caches, workspace and position bookkeeping of one patched attention layer.

    Every sequence of the batch has its own length (the reference's runner hands ragged batches to a
    patched layer as ``attn.kv_lengths``, phasorkv/runner.py:94-99): ``lengths[b]`` tokens of sequence b are
    cached, the next token of b is written at position ``lengths[b]`` and attends to positions
    ``0 .. lengths[b]``."""

    def __init__(self, pk: PhasorKey, batch: int, max_tokens: int, write_chunk: int = 4096, v_bits: int = 0):
        self.pk, self.batch, self.max_tokens, self.write_chunk = pk, batch, max_tokens, write_chunk
        self.cache = pk.new_cache(batch, max_tokens, v_bits=v_bits)     # v_bits 3 / 2: V as per-token low-bit codes
        self.ws = pk.workspace(batch, pk.default_splits(batch, max_tokens))
        self.seq = torch.arange(batch, dtype=torch.int32, device=pk.device)
        self.lengths = [0] * batch                          # tokens cached per sequence (host copy of cache.seqlens)
        self.calibrated = False

    @property
    def length(self) -> int:
        """Longest cached sequence."""
        return max(self.lengths)

    def reset(self) -> None:
        self.lengths = [0] * self.batch
        self.cache.seqlens.zero_()

    def _need(self, b: int, n: int) -> None:
        if self.lengths[b] + n > self.max_tokens:
            raise RuntimeError(f"latent cache holds {self.max_tokens} tokens per sequence; {self.lengths[b] + n} asked")

    def prefill(self, x: torch.Tensor, v: torch.Tensor, lengths=None) -> None:
        """x [B, T, D] layer input, v [B, T, n_kv, d] value rows: append the first ``lengths[b]`` (default: all T)
        tokens of row b to sequence b (rows are right-padded, as the reference's batches are)."""
        B, T = x.shape[0], x.shape[1]
        n_new = [T] * B if lengths is None else [int(n) for n in lengths]
        if len(n_new) != B or min(n_new) < 0 or max(n_new) > T:
            raise ValueError(f"lengths must give 0 .. {T} valid tokens for each of the {B} sequences")
        pk = self.pk
        if not self.calibrated:                             # static tensor scale from the first tokens seen (phasorkv/quant.py:119-124)
            b0 = max(range(B), key=lambda b: n_new[b])
            n = min(n_new[b0], 4096)
            if n:
                pos = torch.arange(self.lengths[b0], self.lengths[b0] + n, dtype=torch.int32, device=pk.device)
                rows = torch.empty((n, pk.cache_width), dtype=torch.float32, device=pk.device)
                pk.write_paged(None, x[b0, :n].contiguous(), pos, None, latent_out=rows)
                pk.calibrate_second(rows)
                self.calibrated = True
        for b in range(B):
            self._need(b, n_new[b])
            for t0 in range(0, n_new[b], self.write_chunk):
                n = min(self.write_chunk, n_new[b] - t0)
                lp = torch.arange(self.lengths[b] + t0, self.lengths[b] + t0 + n, dtype=torch.int32, device=pk.device)
                slots = self.cache.slots(torch.full((n,), b, dtype=torch.int32, device=pk.device), lp)
                pk.write_paged(self.cache, x[b, t0:t0 + n].contiguous(), lp, slots, v=v[b, t0:t0 + n].contiguous())
            self.lengths[b] += n_new[b]
        self.cache.seqlens.copy_(torch.tensor(self.lengths, dtype=torch.int32))

    def decode(self, x: torch.Tensor, q: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        """x [B, D], q [B, n_q, d] pre-RoPE, v [B, n_kv, d] of the one new token of every sequence -> O [B, n_q, d] fp32."""
        for b in range(self.batch):
            self._need(b, 1)
        pk = self.pk
        pos = torch.tensor(self.lengths, dtype=torch.int32, device=pk.device)      # each sequence at its own position
        slots = self.cache.slots(self.seq, pos)
        self.lengths = [n + 1 for n in self.lengths]
        self.cache.seqlens.copy_(pos + 1)
        # the newest token attends to itself too: query position = its own position
        pk.prologue_step(self.cache, x.contiguous(), pos, slots, q.float().contiguous(), pos, self.ws, v=v)
        pk.attend_step(self.cache, self.ws, out=self.ws.out, after_prologue=True)
        return self.ws.out


def _patched_forward(attn, state_of, original):
    def forward(hidden_states, position_embeddings=None, attention_mask=None, past_key_values=None, **kwargs):
        B, T = hidden_states.shape[0], hidden_states.shape[1]
        st: LayerDecodeState = state_of(B)
        d = attn.head_dim
        v = attn.v_proj(hidden_states).view(B, T, -1, d)
        if T > 1:
            out = original(hidden_states, position_embeddings=position_embeddings, attention_mask=attention_mask,
                           past_key_values=None, **kwargs)
            # ragged batch: the runner's per-sequence token counts (phasorkv/runner.py:94-99); rows are right-padded
            st.prefill(hidden_states, v, lengths=getattr(attn, "kv_lengths", None))
            return out
        q = attn.q_proj(hidden_states).view(B, -1, d)
        o = st.decode(hidden_states[:, 0], q, v[:, 0])
        o = o.to(hidden_states.dtype).reshape(B, 1, -1)
        return attn.o_proj(o), None
    return forward


class PhasorKeyPatch:
    def __init__(self, tag: str = "phasor.nvfp4", bits_v: float = 16.0, install_forward: bool = False,
                 max_tokens: int = 4096, v_bits: int = 0):
        self.tag = tag
        self.bits_v = bits_v
        self.v_bits = v_bits              # 0: bf16 V pages; 3 / 2: the reference's per-token tiers (phasorkv/kernels/nvfp4.py:58-67)
        self.install_forward = install_forward
        self.max_tokens = ((max_tokens + PAGE_TOKENS - 1) // PAGE_TOKENS) * PAGE_TOKENS
        self.layer_stats = {}
        self.keys = {}
        self.states = {}

    def reset(self) -> None:
        """Forget the cached tokens of every patched layer (a new prompt follows)."""
        for st in self.states.values():
            st.reset()

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
        bits_v = (self.v_bits * d + 16) * n_kv if self.v_bits else self.bits_v * n_kv * d      # codes + one bf16 scale per (token, kv head)
        self.layer_stats[i] = dict(bits_k=NVFP4_BITS * pk.cache_width, bits_v=bits_v,
                                   width=pk.cache_width, R=pk.R, R_s=pk.R_s)

        original = None
        if self.install_forward:
            original = attn.forward
            own_forward = attn.__dict__.get("forward")          # an earlier instance-level override, if any
            max_tokens = self.max_tokens

            def state_of(batch, i=i, pk=pk):
                st = self.states.get(i)
                if st is None or st.batch != batch:
                    st = self.states[i] = LayerDecodeState(pk, batch, max_tokens, v_bits=self.v_bits)
                return st
            attn.forward = _patched_forward(attn, state_of, original)

        def undo():
            attn.phasor_key, attn.phasor_layer = had
            if had[0] is None:
                del attn.phasor_key, attn.phasor_layer
            if original is not None:
                if own_forward is not None:
                    attn.forward = own_forward
                else:
                    del attn.forward                          # back to the class's forward
                self.states.pop(i, None)
        return undo
