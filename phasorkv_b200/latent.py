"""Host side of the B200 PhasorKey path: the reference's ``phasorkv.latent.PhasorKey`` interface
(constructor, attributes, ``write`` / ``absorb`` / ``scores``; phasorkv/latent.py:27-88) on top of
the CUDA library, plus the batched, paged, quantised entry points a decode loop uses.

All arithmetic of the path runs in libphasorkv_b200.so; torch is used for device memory, streams
and index bookkeeping only. Nothing here falls back to a CPU or eager-torch implementation of the
path: without the library or without a GPU the calls raise.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional, Sequence

import torch

from . import _lib
from ._lib import PAGE_TOKENS


def rope_phasors(inv_freq: torch.Tensor, positions: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """``scale * e^{i t theta_j}`` as complex128 [len(positions), h], the angle formed in float64
    (same contract as phasorkv/rope.py:23-32, taking inv_freq instead of the rotary module)."""
    ang = positions.to(torch.float64)[:, None] * inv_freq.to(device=positions.device, dtype=torch.float64)[None, :]
    return torch.polar(torch.full_like(ang, float(scale)), ang)


def _aligned_bytes(n: int, device, align: int = 1024) -> torch.Tensor:
    """A zeroed uint8 tensor of n bytes whose address is a multiple of `align`."""
    raw = torch.zeros(n + align, dtype=torch.uint8, device=device)
    off = (-raw.data_ptr()) % align
    return raw[off:off + n]


class PagedLatentCache:
    """Paged NVFP4 latent + bf16 V cache of one layer (layout in include/phasorkv_b200.h).

    ``page_table[b, p]`` is the pool page holding tokens ``[128 p, 128 p + 128)`` of sequence b's
    local cache; ``seqlens[b]`` counts the tokens stored. The reference has no paging: its packed
    precedent is a dense [B, T, W/2] code tensor (phasorkv/kernels/latent_attn.py:207-212).
    """

    def __init__(self, W: int, n_kv: int, head_dim: int, batch: int, max_tokens: int, device="cuda",
                 with_v: bool = True, n_pages: Optional[int] = None, v_bits: int = 0):
        lib = _lib.load()
        self.W, self.n_kv, self.head_dim, self.batch = W, n_kv, head_dim, batch
        self.max_pages = (max_tokens + PAGE_TOKENS - 1) // PAGE_TOKENS
        self.n_pages = batch * self.max_pages if n_pages is None else n_pages
        self.page_bytes = int(lib.pkv_latent_page_bytes(W))
        if self.page_bytes <= 0:
            raise _lib.PhasorKVError(f"latent width {W} is not supported (multiple of 16, <= {_lib.MAX_WIDTH})")
        self.device = torch.device(device)
        self.latent = _aligned_bytes(self.n_pages * self.page_bytes, self.device)
        # V pages are head-major: the tile of one (page, kv head) is one contiguous block of 128 x head_dim values
        # v_bits = 3 or 2: V pages hold per-token low-bit codes (phasorkv/kernels/nvfp4.py:58-67) instead of bf16
        self.v_bits = int(v_bits) if with_v else 0
        if self.v_bits not in (0, 2, 3):
            raise ValueError("v_bits must be 0 (bf16 V pages), 3 or 2")
        self.v = (torch.zeros((self.n_pages, n_kv, PAGE_TOKENS, head_dim), dtype=torch.bfloat16, device=self.device)
                  if with_v and not self.v_bits else None)
        self.vq = None
        if self.v_bits:
            tile = int(lib.pkv_vq_page_bytes(n_kv, head_dim))
            if tile <= 0:
                raise _lib.PhasorKVError("quantised V pages need head_dim 128")
            self.vq = _aligned_bytes(self.n_pages * tile, self.device)
        # contiguous default mapping: sequence b owns pages [b*max_pages, (b+1)*max_pages)
        pt = torch.arange(batch * self.max_pages, dtype=torch.int32).reshape(batch, self.max_pages)
        self.page_table = (pt % self.n_pages).to(self.device)
        self.seqlens = torch.zeros(batch, dtype=torch.int32, device=self.device)
        self.c = _lib.Cache(self.latent.data_ptr(), 0 if self.v is None else self.v.data_ptr(), self.n_pages, W,
                            n_kv, head_dim, 0 if self.vq is None else self.vq.data_ptr(), self.v_bits)

    def slots(self, seq: torch.Tensor, local_pos: torch.Tensor) -> torch.Tensor:
        """Slot (page * 128 + row) of token `local_pos` of sequence `seq`; int32 tensors on the device."""
        page = self.page_table[seq.long(), (local_pos // PAGE_TOKENS).long()]
        return (page * PAGE_TOKENS + (local_pos % PAGE_TOKENS).to(torch.int32)).to(torch.int32)

    def v_rows(self, slots: torch.Tensor) -> torch.Tensor:
        """Value rows [n, n_kv, head_dim] stored at `slots` (page * 128 + row); quantised pages: dequantised fp32."""
        if self.v_bits:
            return self.read_vq(slots)[0]
        s = slots.long()
        return self.v[s // PAGE_TOKENS, :, s % PAGE_TOKENS, :]

    def set_v_rows(self, slots: torch.Tensor, rows: torch.Tensor) -> None:
        """Store value rows [n, n_kv, head_dim] (or [n, n_kv * head_dim]) at `slots`."""
        if self.v_bits:
            return self.write_v(rows, slots)
        s = slots.long()
        self.v[s // PAGE_TOKENS, :, s % PAGE_TOKENS, :] = rows.reshape(-1, self.v.shape[1], self.v.shape[3]).to(self.v.dtype)

    def write_v(self, v: torch.Tensor, slots: torch.Tensor) -> None:
        """bf16 value rows [n, n_kv, head_dim] into the V pages (quantised per (token, kv head) if v_bits)."""
        v = v.to(device=self.device, dtype=torch.bfloat16).contiguous()
        if self.v_bits:
            _lib.check(_lib.load().pkv_vq_write(ctypes.byref(self.c), _lib.ptr(v), _lib.ptr(slots), v.shape[0],
                                                _lib.current_stream()), "pkv_vq_write")
            return
        _lib.check(_lib.load().pkv_v_write(ctypes.byref(self.c), _lib.ptr(v), _lib.ptr(slots), v.shape[0],
                                           _lib.current_stream()), "pkv_v_write")

    def read_vq(self, slots: torch.Tensor):
        """Quantised V pages -> (rows fp32 [n, n_kv, d] = value * scale, codes uint8 [n, n_kv, d], scales bf16 [n, n_kv])."""
        n = slots.numel()
        rows = torch.empty((n, self.n_kv, self.head_dim), dtype=torch.float32, device=self.device)
        codes = torch.empty((n, self.n_kv, self.head_dim), dtype=torch.uint8, device=self.device)
        scales = torch.empty((n, self.n_kv), dtype=torch.bfloat16, device=self.device)
        _lib.check(_lib.load().pkv_vq_read(ctypes.byref(self.c), _lib.ptr(slots), n, _lib.ptr(rows), _lib.ptr(codes),
                                           _lib.ptr(scales), _lib.current_stream()), "pkv_vq_read")
        return rows, codes, scales

    def quantize_rows(self, rows: torch.Tensor, slots: torch.Tensor, second) -> None:
        """Given fp32 latent rows [n, W] -> NVFP4 codes + scales in the pages (bit-exact quantiser). `second`: the
        fp32 tensor scale, or a float32 tensor [W/16] with one scale per 16-column block (tiers)."""
        rows = rows.to(torch.float32).contiguous()
        if torch.is_tensor(second):
            sb = second.to(device=self.device, dtype=torch.float32).contiguous()
            _lib.check(_lib.load().pkv_quantize_rows_tiered(ctypes.byref(self.c), _lib.ptr(rows), _lib.ptr(slots), rows.shape[0],
                                                            _lib.ptr(sb), _lib.current_stream()), "pkv_quantize_rows_tiered")
            return
        _lib.check(_lib.load().pkv_quantize_rows(ctypes.byref(self.c), _lib.ptr(rows), _lib.ptr(slots), rows.shape[0],
                                                 ctypes.c_float(second), _lib.current_stream()), "pkv_quantize_rows")

    def read(self, slots: torch.Tensor, second, rows: bool = True, codes: bool = True):
        """-> (rows fp32 [n, W] | None, packed codes uint8 [n, W/2] | None, scale bytes uint8 [n, W/16] | None).
        `second` as for `quantize_rows`."""
        n = slots.numel()
        r = torch.empty((n, self.W), dtype=torch.float32, device=self.device) if rows else None
        c = torch.empty((n, self.W // 2), dtype=torch.uint8, device=self.device) if codes else None
        s = torch.empty((n, self.W // 16), dtype=torch.uint8, device=self.device) if codes else None
        if torch.is_tensor(second):
            sb = second.to(device=self.device, dtype=torch.float32).contiguous()
            _lib.check(_lib.load().pkv_cache_read_tiered(ctypes.byref(self.c), _lib.ptr(slots), n, _lib.ptr(sb),
                                                         _lib.ptr(r), _lib.ptr(c), _lib.ptr(s), _lib.current_stream()),
                       "pkv_cache_read_tiered")
            return r, c, s
        _lib.check(_lib.load().pkv_cache_read(ctypes.byref(self.c), _lib.ptr(slots), n, ctypes.c_float(second),
                                              _lib.ptr(r), _lib.ptr(c), _lib.ptr(s), _lib.current_stream()),
                   "pkv_cache_read")
        return r, c, s


class DecodeWorkspace:
    """Caller-owned scratch of one decode call: absorbed query (fp32 and operand form), the split
    partials, the output. Reused across layers and steps so that the timed path allocates nothing."""

    def __init__(self, batch: int, n_q: int, head_dim: int, W: int, n_split: int, device):
        lib = _lib.load()
        self.batch, self.n_split = batch, n_split
        self.qabs = torch.empty((batch, n_q, W), dtype=torch.float32, device=device)
        self.qop_bytes = int(lib.pkv_query_operand_bytes(W))
        self.qop = _aligned_bytes(batch * self.qop_bytes, device)
        self.partials = torch.empty((batch, n_split, n_q, head_dim + 2), dtype=torch.float32, device=device)
        self.packed = torch.empty((batch, n_q, head_dim + 2), dtype=torch.float32, device=device)
        self.out = torch.empty((batch, n_q, head_dim), dtype=torch.float32, device=device)
        self.status = torch.zeros(4, dtype=torch.int32, device=device)
        # operand-ready counters of this workspace's query operand (absorb_step / prologue_step with signal=True,
        # attend_step with polled=True): [ready per sequence | consumers done per sequence]
        self.qsync = torch.zeros(2 * batch, dtype=torch.int32, device=device)
        self.wscratch = None                                                  # decode-time write, see write_scratch()
        self.exact = None                                                     # exact-token partial, see exact_step()


class PhasorKey:
    """The phasor key cache of one layer.

    Constructor and attributes follow the reference (phasorkv/latent.py:28-59): ``PhasorKey(fac,
    ranks, n_q)`` takes a ``Factorization``-like object (``blocks`` with ``U, s2, sq, Mw, where,
    cost``; ``nope``; ``n_kv``; ``d``; ``absorbed``) and builds ``A [n_kv, R]``, ``B [R, D]``,
    ``freq``, ``energy``, ``slow``, ``A_s``, ``B_s`` with latent dims sorted by energy.
    ``from_factors`` injects those arrays directly (synthetic layers).
    """

    def __init__(self, fac, ranks: Sequence[int], n_q: int, inv_freq: Optional[torch.Tensor] = None,
                 attn_scale: float = 1.0, device="cuda"):
        if not getattr(fac, "absorbed", False):
            raise AssertionError("PhasorKey needs an absorbed layout ('freq' or 'bandN')")
        a_cols, b_rows, freq, energy = [], [], [], []
        A_s = B_s = None
        for blk, r in zip(fac.blocks, ranks):
            r = int(r)
            top = blk.U[:, :r]
            if blk.cost == 1:                                       # real slow band, scored without RoPE
                if r:
                    A_s = (top / blk.sq[:, None]).reshape(fac.n_kv, -1, r)
                    B_s = top.T @ blk.Mw
                continue
            if r == 0:
                continue
            a_cols.append(top / blk.sq[:, None])
            b_rows.append(top.conj().T @ blk.Mw)
            freq.append(torch.full((r,), int(blk.where), dtype=torch.long))
            energy.append(blk.s2[:r])
        en = torch.cat(energy)
        order = torch.argsort(en, descending=True)
        self._init(torch.cat(a_cols, dim=1)[:, order], torch.cat(b_rows, dim=0)[order], torch.cat(freq)[order.cpu()],
                   n_q, fac.n_kv, fac.d, inv_freq, A_s, B_s, fac.nope.nonzero().flatten(), en[order], attn_scale, device)

    @classmethod
    def from_factors(cls, A, B, freq, n_q, n_kv, head_dim, inv_freq, A_s=None, B_s=None, slow=None,
                     energy=None, attn_scale: float = 1.0, device="cuda") -> "PhasorKey":
        self = object.__new__(cls)
        self._init(A, B, freq, n_q, n_kv, head_dim, inv_freq, A_s, B_s, slow, energy, attn_scale, device)
        return self

    @classmethod
    def with_mean_direction(cls, A, B, freq, mu, kbar, n_q, n_kv, head_dim, inv_freq, A_s=None, B_s=None, slow=None,
                            attn_scale: float = 1.0, device="cuda") -> "PhasorKey":
        """The mean-direction split of the reference's latent projections (phasorkv/kvmethods.py:895-899:
        ``k = A Q(B x) + alpha * W mu`` with ``alpha = x . mu / |mu|^2`` and ``B`` folded with the projection
        that removes the mean direction) in rotated-latent form.

        After RoPE the mean term of token t is ``alpha_t * kbar_j * e^{i theta_j t}`` at every frequency j
        (``kbar = W mu`` [n_kv * d] in the rotate-half layout): not one cached number per token but one rank-1
        component per frequency, i.e. ``d/2`` further complex latent dims with ``A[:, j] = kbar_j`` and the
        same row ``B[j] = mu / |mu|^2``. This constructor appends them to the given factors (whose ``B`` it
        first makes blind to the mean direction) and returns an ordinary PhasorKey: write, absorb and the decode
        kernels run unchanged; the cache grows by ``d`` reals per token. (The reference keeps alpha in bf16; here
        it is part of the NVFP4 latent.)"""
        h = int(head_dim) // 2
        mu = mu.to(torch.float64)
        mu_scaled = mu / mu.dot(mu)
        Bc = B.to(torch.complex128)
        B_perp = Bc - (Bc @ mu.to(torch.complex128))[:, None] * mu_scaled.to(torch.complex128)[None, :]
        kb = kbar.to(torch.float64).reshape(n_kv, head_dim)
        A_mean = torch.complex(kb[:, :h], kb[:, h:])                                     # [n_kv, h]
        B_mean = mu_scaled.to(torch.complex128)[None, :].expand(h, -1)
        A_all = torch.cat([A.to(torch.complex128), A_mean], dim=1)
        B_all = torch.cat([B_perp, B_mean], dim=0)
        freq_all = torch.cat([freq.long(), torch.arange(h)])
        if B_s is not None:                                                              # the slow block sees no mean either
            B_s = B_s.to(torch.float64) - (B_s.to(torch.float64) @ mu)[:, None] * mu_scaled[None, :]
        return cls.from_factors(A_all, B_all, freq_all, n_q, n_kv, head_dim, inv_freq, A_s, B_s, slow, None, attn_scale, device)

    @classmethod
    def from_spec(cls, spec, device="cuda") -> "PhasorKey":
        return cls.from_factors(spec.A, spec.B, spec.freq, spec.n_q, spec.n_kv, spec.head_dim, spec.inv_freq,
                                spec.A_s, spec.B_s, spec.slow, None, spec.attn_scale, device)

    def _init(self, A, B, freq, n_q, n_kv, head_dim, inv_freq, A_s, B_s, slow, energy, attn_scale, device):
        self.A, self.B, self.freq = A, B, freq.long()
        self.A_s, self.B_s = A_s, B_s
        self.slow = slow.long() if slow is not None else torch.zeros(0, dtype=torch.long)
        self.energy = energy
        self.n_q, self.n_kv, self.h = int(n_q), int(n_kv), int(head_dim) // 2
        self.R = int(B.shape[0])
        self.R_s = 0 if B_s is None else int(B_s.shape[0])
        self.head_dim, self.d_model = int(head_dim), int(B.shape[1])
        self.inv_freq = None if inv_freq is None else inv_freq.to(torch.float64).cpu()
        self.attn_scale = float(attn_scale)
        self.second = 1.0
        self.second_blocks = None                          # tiers: one tensor scale per 16-column block (set_second_tiers)
        self.device = torch.device(device)
        self._dev = None

    # ------------------------------------------------------------------ reference surface
    @property
    def cache_width(self) -> int:
        """Cached reals per token (shared by all heads)."""
        return 2 * self.R + self.R_s

    def write(self, x: torch.Tensor, ph: torch.Tensor) -> torch.Tensor:
        """Tokens x [T, D] at phasors ph [T, d/2] -> cache rows [T, 2R + R_s] (unquantised): fp64 rows for
        fp64 x, fp32 rows otherwise, as the reference (phasorkv/latent.py:63-64)."""
        if x.dtype == torch.float64:
            t = self._f64()
            xd = x.to(self.device).contiguous()
            phd = torch.view_as_real(ph.to(torch.complex128)).to(self.device).contiguous()
            out = torch.empty((xd.shape[0], self.cache_width), dtype=torch.float64, device=self.device)
            _lib.check(_lib.load().pkv_write_rows_f64(_lib.ptr(t["Bw"]), _lib.ptr(t["freq"]), self.d_model, self.R, self.R_s,
                                                      self.h, _lib.ptr(xd), _lib.ptr(phd), xd.shape[0], _lib.ptr(out),
                                                      _lib.current_stream()), "pkv_write_rows_f64")
            return out
        L = self._layer()
        x = self._x(x)
        phd = self._ph(ph)
        out = torch.empty((x.shape[0], self.cache_width), dtype=torch.float32, device=self.device)
        _lib.check(_lib.load().pkv_cache_write(ctypes.byref(L), None, _lib.ptr(x), self._xdt(x), None, _lib.ptr(phd),
                                               None, x.shape[0], _lib.ptr(out), None, None, None, _lib.current_stream()),
                   "pkv_cache_write")
        return out

    def absorb(self, q: torch.Tensor, ph: torch.Tensor) -> torch.Tensor:
        """Pre-RoPE queries q [H, Tq, d] at phasors ph [Tq, d/2] -> [H, Tq, 2R + R_s] (fp64 for fp64 q)."""
        if q.dtype == torch.float64:
            t = self._f64()
            qd = q.to(self.device).transpose(0, 1).contiguous()
            phd = torch.view_as_real(ph.to(torch.complex128)).to(self.device).contiguous()
            out = torch.empty((qd.shape[0], self.n_q, self.cache_width), dtype=torch.float64, device=self.device)
            _lib.check(_lib.load().pkv_absorb_rows_f64(_lib.ptr(t["A_re"]), _lib.ptr(t["A_im"]), _lib.ptr(t["A_s"]),
                                                       _lib.ptr(t["freq"]), _lib.ptr(t["slow"]), self.n_q, self.n_kv,
                                                       self.head_dim, self.R, self.R_s, int(self.slow.numel()) if self.R_s else 0,
                                                       _lib.ptr(qd), _lib.ptr(phd), qd.shape[0], _lib.ptr(out),
                                                       _lib.current_stream()), "pkv_absorb_rows_f64")
            return out.transpose(0, 1)
        self._layer()
        L = self._dev["layer_plain"]
        L.second = self.second
        qd = q.to(device=self.device, dtype=torch.float32).transpose(0, 1).contiguous()     # [Tq, H, d]
        phd = self._ph(ph)
        out = torch.empty((qd.shape[0], self.n_q, self.cache_width), dtype=torch.float32, device=self.device)
        _lib.check(_lib.load().pkv_absorb(ctypes.byref(L), _lib.ptr(qd), None, _lib.ptr(phd), qd.shape[0],
                                          _lib.ptr(out), None, _lib.current_stream()), "pkv_absorb")
        return out.transpose(0, 1)

    @staticmethod
    def scores(q_abs: torch.Tensor, cache: torch.Tensor) -> torch.Tensor:
        """Unscaled logits [H, Tq, Tk] = q_abs @ cache^T of the rows given, in q_abs's precision (fp32 or
        fp64), with no quantisation: the reference's static method (phasorkv/latent.py:85-88). The result
        lives on the GPU. `scores_nvfp4` is the score on the quantised cache."""
        if not torch.cuda.is_available():
            raise _lib.PhasorKVError("phasorkv_b200 needs a CUDA device; there is no CPU path")
        dt = torch.float64 if q_abs.dtype == torch.float64 else torch.float32
        dev = q_abs.device if q_abs.is_cuda else torch.device("cuda", torch.cuda.current_device())
        H, Tq, W = q_abs.shape
        qa = q_abs.to(device=dev, dtype=dt).reshape(H * Tq, W).contiguous()
        rows = cache.to(device=dev, dtype=dt).contiguous()
        if rows.shape[1] != W:
            raise ValueError(f"cache rows have width {rows.shape[1]}, the absorbed query {W}")
        out = torch.empty((H * Tq, rows.shape[0]), dtype=dt, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.load().pkv_scores_exact(_lib.ptr(qa), _lib.ptr(rows), H * Tq, rows.shape[0], W,
                                                    _lib.F64 if dt == torch.float64 else _lib.F32, _lib.ptr(out),
                                                    _lib.current_stream()), "pkv_scores_exact")
        return out.view(H, Tq, rows.shape[0])

    def scores_nvfp4(self, q_abs: torch.Tensor, cache) -> torch.Tensor:
        """Unscaled logits [H, Tq, Tk] of absorbed queries against the NVFP4 cache.

        `cache` is either fp32 rows [Tk, W] (they are quantised with this layer's tensor scale into a
        scratch paged cache first) or a tuple ``(PagedLatentCache, sequence index)``."""
        if isinstance(cache, tuple):
            pc, b = cache
        else:
            rows = cache.to(device=self.device, dtype=torch.float32)
            pc, b = PagedLatentCache(self.cache_width, self.n_kv, self.head_dim, 1, rows.shape[0], self.device,
                                     with_v=False), 0
            n = rows.shape[0]
            pos = torch.arange(n, dtype=torch.int32, device=self.device)
            pc.quantize_rows(rows, pc.slots(torch.zeros_like(pos), pos), self.second)
            pc.seqlens.fill_(n)
        Tk = int(pc.seqlens[b])
        qa = q_abs.to(device=self.device, dtype=torch.float32).transpose(0, 1).contiguous()        # [Tq, H, W]
        Tq = qa.shape[0]
        S = torch.empty((Tq, self.n_q, Tk), dtype=torch.float32, device=self.device)
        pt = pc.page_table[b:b + 1].expand(Tq, -1).contiguous()
        sl = pc.seqlens[b:b + 1].expand(Tq).contiguous()
        ws = DecodeWorkspace(Tq, self.n_q, self.head_dim, self.cache_width, 1, self.device)
        L = self._layer()
        _lib.check(_lib.load().pkv_decode_attn(ctypes.byref(L), ctypes.byref(pc.c), _lib.ptr(qa), _lib.ptr(pt),
                                               pc.max_pages, _lib.ptr(sl), Tq, 1,
                                               _lib.ATTN_SCORES_ONLY | _lib.ATTN_SIMT, _lib.ptr(ws.partials),
                                               _lib.ptr(S), Tk, _lib.ptr(ws.status), None,
                                               _lib.current_stream()), "pkv_decode_attn")
        return S.transpose(0, 1)

    # ------------------------------------------------------------------ B200 entry points
    def set_second(self, second: float) -> None:
        """fp32 tensor scale of the NVFP4 latent (phasorkv/quant.py:119-124 gives the static rule)."""
        self.second = float(second)
        if self._dev is not None:
            self._dev["layer"].second = self.second

    def calibrate_second(self, rows: torch.Tensor, span: int = 0):
        """Static rule of the reference: 32 sigma of the widest latent channel over 448 * 6 (phasorkv/quant.py:119-124).
        `span` (a multiple of 16): one such scale per span of that many columns of the energy-sorted latent -- the
        reference's tiers (phasorkv/kernels/latent_attn.py:149-152, 255-262) -- instead of one for the whole row."""
        var = rows.float().var(dim=0)
        rule = lambda v: 32.0 * v.max().clamp_min(1e-30).sqrt() / (448.0 * 6.0)
        self.set_second(float(rule(var)))
        if span:
            if span % 16:
                raise ValueError("a tier span is a multiple of 16 columns")
            W = self.cache_width
            self.set_second_tiers([(lo, min(lo + span, W), float(rule(var[lo:min(lo + span, W)]))) for lo in range(0, W, span)])
        return self.second

    def set_second_tiers(self, tiers) -> None:
        """tiers: [(lo, hi, second)] covering the row in 16-aligned spans (None: back to one scale). Quantising
        calls then use each block's own tensor scale; absorb_step / prologue_step fold `second_tier / second` into the
        query's columns (their fp32 rows ws.qabs are then in the cache's units), the decode kernels are unchanged."""
        self.second_blocks = None
        if tiers is not None:
            nb = (self.cache_width + 15) // 16
            sb = torch.full((nb,), self.second, dtype=torch.float32)
            for lo, hi, sec in tiers:
                if lo % 16 or (hi % 16 and hi != self.cache_width) or not sec > 0:
                    raise ValueError("tiers are 16-aligned spans with positive scales")
                sb[lo // 16:(hi + 15) // 16] = float(sec)
            self.second_blocks = sb
        if self._dev is not None:
            self._dev["second_blocks"] = None if self.second_blocks is None else self.second_blocks.to(self.device)
            self._dev["layer"].second_blocks_dev = 0 if self.second_blocks is None else self._dev["second_blocks"].data_ptr()

    def second_arg(self):
        """What `PagedLatentCache.quantize_rows` / `read` take as `second` for this layer: the scalar, or the tiers."""
        return self.second if getattr(self, "second_blocks", None) is None else self.second_blocks

    def new_cache(self, batch: int, max_tokens: int, with_v: bool = True, v_bits: int = 0) -> PagedLatentCache:
        return PagedLatentCache(self.cache_width, self.n_kv, self.head_dim, batch, max_tokens, self.device, with_v,
                                v_bits=v_bits)

    def write_paged(self, cache: PagedLatentCache, x: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                    v: Optional[torch.Tensor] = None, latent_out: Optional[torch.Tensor] = None,
                    scratch: Optional[torch.Tensor] = None) -> None:
        """Fused write of tokens x [n, D] (fp32 or bf16) at global `positions` into `slots`; V rows too.
        With ``cache=None`` only the unquantised rows are produced (into `latent_out`)."""
        self._need_inv_freq("write_paged")
        L = self._layer()
        x = self._x(x)
        if v is not None and cache is not None and cache.v_bits:       # quantised V pages have their own writer
            cache.write_v(v, slots)
            v = None
        if v is not None:
            v = v.to(torch.bfloat16).contiguous()
        _lib.check(_lib.load().pkv_cache_write(ctypes.byref(L), None if cache is None else ctypes.byref(cache.c),
                                               _lib.ptr(x), self._xdt(x),
                                               _lib.ptr(positions), None, _lib.ptr(slots), x.shape[0],
                                               _lib.ptr(latent_out), _lib.ptr(scratch), _lib.ptr(v),
                                               _lib.ptr(self._dev["status"]), _lib.current_stream()), "pkv_cache_write")

    def workspace(self, batch: int, n_split: int) -> DecodeWorkspace:
        ws = DecodeWorkspace(batch, self.n_q, self.head_dim, self.cache_width, n_split, self.device)
        ws.wscratch = self.write_scratch(batch)
        return ws

    def write_scratch(self, n_tokens: int) -> torch.Tensor:
        """Scratch for the decode-time (<= 64 tokens) write path of `write_paged`."""
        n = int(_lib.load().pkv_write_scratch_floats(max(n_tokens, 1), self.d_model))
        return torch.empty(n, dtype=torch.float32, device=self.device)

    def default_splits(self, batch: int, max_tokens: int, simt: bool = False) -> int:
        """Token splits per sequence so that the grid fills the GPU a whole number of times."""
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        pages = max(1, (max_tokens + PAGE_TOKENS - 1) // PAGE_TOKENS)
        per_sm = 3 if simt else 1
        # one query head per kv head: the tensor-core kernel runs 4 CTAs (8 heads each) per (sequence, split)
        groups = 4 if (not simt and self.n_kv == self.n_q) else 1
        return max(1, min(pages, (sms * per_sm) // max(1, batch * groups)))

    def absorb_step(self, q: torch.Tensor, positions: torch.Tensor, ws: DecodeWorkspace, operand: bool = True,
                    signal: bool = False) -> None:
        """q [B, H, d] fp32 at `positions` [B] -> ws.qabs (fp32) and, if asked, ws.qop (operand form).
        `signal`: raise the workspace's operand-ready counters (for ``attend_step(polled=True)`` right behind)."""
        self._need_inv_freq("absorb_step")
        L = self._layer()
        _lib.check(_lib.load().pkv_absorb_sync(ctypes.byref(L), _lib.ptr(q), _lib.ptr(positions), None, q.shape[0],
                                               _lib.ptr(ws.qabs), _lib.ptr(ws.qop) if operand else None,
                                               _lib.ptr(ws.qsync) if signal else None, _lib.current_stream()), "pkv_absorb")

    def prologue_step(self, cache: PagedLatentCache, x: torch.Tensor, write_positions: torch.Tensor, slots: torch.Tensor,
                      q: Optional[torch.Tensor], query_positions: Optional[torch.Tensor], ws: DecodeWorkspace,
                      v: Optional[torch.Tensor] = None, latent_out: Optional[torch.Tensor] = None,
                      operand: bool = True, signal: bool = False) -> None:
        """`write_paged` of the newest token of every sequence and `absorb_step` of the step's queries
        as one launch (same bits as the two calls). `q=None`: the write alone (the queries then go to
        `attend_q_step`). `signal`: as for `absorb_step`."""
        self._need_inv_freq("prologue_step")
        L = self._layer()
        x = self._x(x)
        if v is not None:                                               # (quantised V pages: the rows are quantised by the same launch)
            v = v.to(torch.bfloat16).contiguous()
        _lib.check(_lib.load().pkv_decode_prologue_sync(ctypes.byref(L), ctypes.byref(cache.c), _lib.ptr(x), self._xdt(x),
                                                        _lib.ptr(write_positions), _lib.ptr(slots), _lib.ptr(v), _lib.ptr(q),
                                                        _lib.ptr(query_positions), x.shape[0], _lib.ptr(latent_out),
                                                        _lib.ptr(getattr(ws, "wscratch", None)), _lib.ptr(ws.qabs),
                                                        _lib.ptr(ws.qop) if operand else None,
                                                        _lib.ptr(ws.qsync) if (signal and q is not None and operand) else None,
                                                        _lib.ptr(self._dev["status"]), _lib.current_stream()),
                   "pkv_decode_prologue")

    def attend_q_step(self, cache: PagedLatentCache, q: torch.Tensor, positions: torch.Tensor, ws: DecodeWorkspace,
                      scores_only: bool = False, scores_out: Optional[torch.Tensor] = None,
                      out: Optional[torch.Tensor] = None, packed_out: Optional[torch.Tensor] = None,
                      early: bool = False, tail_written: bool = False, query_ready: bool = False) -> None:
        """`attend_step` on RAW queries q [B, H, d] fp32 at `positions` [B]: the attention kernel absorbs them
        itself (no `absorb_step`, same bits). `early`: the launch enqueued just before writes nothing this
        kernel reads except, with `tail_written`, rows of each sequence's last page (a write of the newest
        token) and, unless `query_ready`, the queries."""
        self._need_inv_freq("attend_q_step")
        L = self._layer()
        flags = _lib.ATTN_SCORES_ONLY if scores_only else 0
        if early:
            flags |= _lib.ATTN_EARLY_STREAM | (_lib.ATTN_TAIL_WRITTEN if tail_written else 0) | \
                (_lib.ATTN_QUERY_READY if query_ready else 0)
        if packed_out is not None:
            out, flags = packed_out, flags | _lib.ATTN_PACKED_OUT
        stride = 0 if scores_out is None else scores_out.shape[-1]
        _lib.check(_lib.load().pkv_decode_attn_q(ctypes.byref(L), ctypes.byref(cache.c), _lib.ptr(q), _lib.ptr(positions),
                                                 _lib.ptr(cache.page_table), cache.max_pages, _lib.ptr(cache.seqlens),
                                                 ws.batch, ws.n_split, flags, _lib.ptr(ws.partials), _lib.ptr(scores_out),
                                                 stride, _lib.ptr(ws.status), _lib.ptr(out), _lib.current_stream()),
                   "pkv_decode_attn_q")

    def attend_step(self, cache: PagedLatentCache, ws: DecodeWorkspace, simt: bool = False, scores_only: bool = False,
                    scores_out: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                    packed_out: Optional[torch.Tensor] = None, after_absorb: bool = False,
                    after_prologue: bool = False, polled: bool = False) -> None:
        """Split-T attention of the absorbed queries in `ws` over `cache` -> ws.partials; with `out`
        [B, H, d] the splits are merged as well (a merge launch enqueued right behind). `polled` (with
        `after_absorb` / `after_prologue`, whose launch was made with ``signal=True``): the kernel polls the
        workspace's operand-ready counters instead of waiting for that whole launch."""
        L = self._layer()
        flags = (_lib.ATTN_SIMT if simt else 0) | (_lib.ATTN_SCORES_ONLY if scores_only else 0)
        if after_absorb and not simt:                   # the launch enqueued just before was absorb_step: stream pages early
            flags |= _lib.ATTN_EARLY_STREAM
        if after_prologue and not simt:                 # ... was prologue_step: it also writes the newest token's rows
            flags |= _lib.ATTN_EARLY_STREAM | _lib.ATTN_TAIL_WRITTEN
        if packed_out is not None:                      # merged (o, m, l) triple [B, H, d+2] instead of the normalised output
            out, flags = packed_out, flags | _lib.ATTN_PACKED_OUT
        qsrc = ws.qabs if simt else ws.qop
        stride = 0 if scores_out is None else scores_out.shape[-1]
        poll = polled and not simt and (after_absorb or after_prologue)
        _lib.check(_lib.load().pkv_decode_attn_sync(ctypes.byref(L), ctypes.byref(cache.c), _lib.ptr(qsrc),
                                                    _lib.ptr(ws.qsync) if poll else None,
                                                    _lib.ptr(cache.page_table), cache.max_pages, _lib.ptr(cache.seqlens),
                                                    ws.batch, ws.n_split, flags, _lib.ptr(ws.partials), _lib.ptr(scores_out),
                                                    stride, _lib.ptr(ws.status), _lib.ptr(out),
                                                    _lib.current_stream()), "pkv_decode_attn")

    def exact_step(self, q: torch.Tensor, positions: torch.Tensor, k_exact: torch.Tensor, v_exact: torch.Tensor,
                   ws: DecodeWorkspace, n_exact: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Partial triple of the exact (bf16, rotated keys) tokens: k_exact, v_exact [B, n_kv, E, d] bf16,
        optional valid counts n_exact [B] -> ws.exact [B, H, d+2]; merged by ``merge_step(exact=True)``."""
        self._need_inv_freq("exact_step")
        L = self._layer()
        B, E = q.shape[0], k_exact.shape[2]
        if getattr(ws, "exact", None) is None:
            ws.exact = torch.empty((B, self.n_q, self.head_dim + 2), dtype=torch.float32, device=self.device)
        k_exact, v_exact = k_exact.to(torch.bfloat16).contiguous(), v_exact.to(torch.bfloat16).contiguous()
        _lib.check(_lib.load().pkv_exact_partial(ctypes.byref(L), _lib.ptr(q), _lib.ptr(positions), _lib.ptr(k_exact),
                                                 _lib.ptr(v_exact), _lib.ptr(n_exact), E, B, _lib.ptr(ws.exact),
                                                 _lib.current_stream()), "pkv_exact_partial")
        return ws.exact

    def merge_step(self, ws: DecodeWorkspace, normalise: bool = True, packed: bool = False,
                   out: Optional[torch.Tensor] = None, exact: bool = False) -> None:
        """Log-sum-exp merge of ws.partials (and, with `exact`, of ws.exact) -> `out` or ws.out (normalised)
        and / or ws.packed (o, m, l)."""
        pw = self.head_dim + 2
        out = ws.out if out is None else out
        _lib.check(_lib.load().pkv_merge_exact(_lib.ptr(ws.partials), ws.n_split * self.n_q * pw, self.n_q * pw, ws.n_split,
                                               ws.batch, self.n_q, self.head_dim, _lib.ptr(ws.exact) if exact else None,
                                               _lib.ptr(out) if normalise else None,
                                               _lib.ptr(ws.packed) if packed else None, _lib.current_stream()), "pkv_merge_exact")

    def merge_gathered(self, gathered: torch.Tensor, out: torch.Tensor) -> None:
        """gathered [G, B, H, d+2] packed triples of G token shards -> out [B, H, d]."""
        G, B = gathered.shape[0], gathered.shape[1]
        pw = self.head_dim + 2
        _lib.check(_lib.load().pkv_merge(_lib.ptr(gathered), self.n_q * pw, B * self.n_q * pw, G, B, self.n_q,
                                         self.head_dim, _lib.ptr(out), None, _lib.current_stream()), "pkv_merge")

    def decode(self, cache: PagedLatentCache, q: torch.Tensor, positions: torch.Tensor,
               ws: Optional[DecodeWorkspace] = None, simt: bool = False, scores_only: bool = False) -> torch.Tensor:
        """One decode step of this layer: absorb, split-T attention, merge -> O [B, H, d] fp32."""
        if ws is None:
            ws = self.workspace(q.shape[0], self.default_splits(q.shape[0], cache.max_pages * PAGE_TOKENS, simt))
        self.absorb_step(q, positions, ws, operand=not simt)
        self.attend_step(cache, ws, simt=simt, scores_only=scores_only, out=ws.out, after_absorb=True)
        return ws.out

    # ------------------------------------------------------------------ plumbing
    def _layer(self) -> _lib.Layer:
        """Upload the factors once and return the C struct (device pointers stay owned by this object)."""
        if self._dev is None:
            if not torch.cuda.is_available():
                raise _lib.PhasorKVError("phasorkv_b200 needs a CUDA device; there is no CPU path")
            _lib.check(_lib.load().pkv_device_check(), "pkv_device_check")
            dev = self.device
            B = self.B.to(torch.complex64)
            rows = [B.real, B.imag] + ([self.B_s.to(torch.float32)] if self.R_s else [])
            Bw = torch.cat(rows, dim=0).to(device=dev, dtype=torch.float32).contiguous()
            # the factors once more as three bf16 matrices whose sum is Bw to 2^-24 (tensor-core cache write)
            Wp = 128 if Bw.shape[0] <= 128 else 256
            Bp = torch.zeros((Wp, Bw.shape[1]), dtype=torch.float32, device=dev)
            Bp[:Bw.shape[0]] = Bw
            hi = Bp.to(torch.bfloat16)
            mid = (Bp - hi.float()).to(torch.bfloat16)
            lo = (Bp - hi.float() - mid.float()).to(torch.bfloat16)
            t = dict(
                Bw=Bw, Bw3=torch.stack([hi, mid, lo]).contiguous(), status=torch.zeros(4, dtype=torch.int32, device=dev),
                A_re=self.A.real.to(device=dev, dtype=torch.float32).contiguous(),
                A_im=self.A.imag.to(device=dev, dtype=torch.float32).contiguous(),
                A_s=None if not self.R_s else self.A_s.to(device=dev, dtype=torch.float32).contiguous(),
                freq=self.freq.to(device=dev, dtype=torch.int32).contiguous(),
                slow=None if not self.R_s else self.slow.to(device=dev, dtype=torch.int32).contiguous(),
                # without inv_freq (the reference's three-argument constructor) the calls that take ready
                # phasors still work; the calls that take positions refuse (_need_inv_freq)
                inv_freq=(torch.zeros(self.h, dtype=torch.float64) if self.inv_freq is None else self.inv_freq
                          ).to(device=dev, dtype=torch.float64).contiguous(),
            )
            L = _lib.Layer(self.d_model, self.n_q, self.n_kv, self.head_dim, self.R, self.R_s,
                           int(self.slow.numel()) if self.R_s else 0, self.attn_scale, self.second,
                           t["Bw"].data_ptr(), t["A_re"].data_ptr(), t["A_im"].data_ptr(),
                           0 if t["A_s"] is None else t["A_s"].data_ptr(), t["freq"].data_ptr(),
                           0 if t["slow"] is None else t["slow"].data_ptr(), t["inv_freq"].data_ptr(),
                           t["Bw3"].data_ptr() if Bw.shape[0] <= 256 else 0, 0)
            t["layer"] = L
            # the reference's absorb (no tiers folded in) goes through a copy of the struct without them
            t["layer_plain"] = _lib.Layer.from_buffer_copy(L)
            sb = getattr(self, "second_blocks", None)
            if sb is not None:
                t["second_blocks"] = sb.to(dev)
                L.second_blocks_dev = t["second_blocks"].data_ptr()
            self._dev = t
        return self._dev["layer"]

    def _need_inv_freq(self, what: str) -> None:
        if self.inv_freq is None:
            raise _lib.PhasorKVError(f"{what} forms phasors from positions and needs inv_freq: pass it to the constructor "
                                     "(PhasorKey(fac, ranks, n_q, inv_freq=rotary.inv_freq)) or use set_inv_freq")

    def set_inv_freq(self, inv_freq: torch.Tensor, attn_scale: Optional[float] = None) -> None:
        """Rotary inverse frequencies [d/2] (and attention scaling) for the calls that take positions."""
        self.inv_freq = inv_freq.to(torch.float64).cpu()
        if attn_scale is not None:
            self.attn_scale = float(attn_scale)
        if self._dev is not None:
            self._dev["inv_freq"].copy_(self.inv_freq)
            self._dev["layer"].attn_scale = self.attn_scale

    def _f64(self) -> dict:
        """fp64 device copies of the factors for the fp64 forms of write / absorb (made on first use)."""
        if getattr(self, "_dev64", None) is None:
            if not torch.cuda.is_available():
                raise _lib.PhasorKVError("phasorkv_b200 needs a CUDA device; there is no CPU path")
            _lib.check(_lib.load().pkv_device_check(), "pkv_device_check")
            dev = self.device
            B = self.B.to(torch.complex128)
            rows = [B.real, B.imag] + ([self.B_s.to(torch.float64)] if self.R_s else [])
            A = self.A.to(torch.complex128)
            self._dev64 = dict(
                Bw=torch.cat(rows, dim=0).to(device=dev, dtype=torch.float64).contiguous(),
                A_re=A.real.to(device=dev, dtype=torch.float64).contiguous(),
                A_im=A.imag.to(device=dev, dtype=torch.float64).contiguous(),
                A_s=None if not self.R_s else self.A_s.to(device=dev, dtype=torch.float64).contiguous(),
                freq=self.freq.to(device=dev, dtype=torch.int32).contiguous(),
                slow=None if not self.R_s else self.slow.to(device=dev, dtype=torch.int32).contiguous())
        return self._dev64

    def _x(self, x: torch.Tensor) -> torch.Tensor:
        if x.dtype not in (torch.float32, torch.bfloat16):
            x = x.to(torch.float32)
        return x.to(self.device).contiguous()

    @staticmethod
    def _xdt(x: torch.Tensor) -> int:
        return _lib.BF16 if x.dtype == torch.bfloat16 else _lib.F32

    def _ph(self, ph: torch.Tensor) -> torch.Tensor:
        """complex phasors [n, h] -> interleaved float32 [n, h, 2] on the device."""
        return torch.view_as_real(ph.to(torch.complex64)).to(self.device).contiguous()
