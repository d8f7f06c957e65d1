"""Token-sharded decode across the GPUs of one box: buffers and host calls of the fused
exchange-and-merge kernel (`pkv_exchange_merge`).

Each rank keeps the tokens ``[r*T/G, (r+1)*T/G)`` of every sequence in its own paged cache, runs
absorb + attention locally (the attention launch already merges the local splits into one packed
triple per head), and then exchanges ``[B, H, d+2]`` floats with its peers. The reference has no
multi-GPU path; the merge applied across ranks is its split combine
(phasorkv/kernels/dense_attn.py:72-74).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch

from . import _lib


def token_range(rank: int, world: int, n_tokens: int) -> tuple:
    """Contiguous token range [lo, hi) of a sequence of `n_tokens` tokens that rank `rank` of `world`
    holds: ranges are disjoint, cover the sequence, differ by at most one token, and keep global
    positions (the stored phasors need no fix-up)."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside a group of {world}")
    return rank * n_tokens // world, (rank + 1) * n_tokens // world


def owner_of(position: int, world: int, n_tokens: int) -> int:
    """Rank that holds (and therefore writes) the token at `position` of a sequence of `n_tokens`."""
    if not 0 <= position < n_tokens:
        raise ValueError(f"position {position} outside a sequence of {n_tokens} tokens")
    for r in range(world):
        lo, hi = token_range(r, world, n_tokens)
        if lo <= position < hi:
            return r
    raise AssertionError("ranges cover the sequence")


def gather_words(world: int, batch: int, n_q: int, head_dim: int) -> int:
    """8-byte words of one rank's gather buffer: [2 slots][world][B*H*(d+2)]."""
    return 2 * world * batch * n_q * (head_dim + 2)


class ShardExchange:
    """Host handle of one rank. `data_ptrs` are the addresses of every rank's gather buffer as seen
    from this process (own allocation for rank == self, peer mappings otherwise); buffers start zeroed."""

    def __init__(self, world: int, rank: int, batch: int, n_q: int, head_dim: int, data_ptrs: List[int],
                 device, n_cta: int = 64, keep=None):
        self.world, self.rank = world, rank
        self._ptr_data = torch.tensor(data_ptrs, dtype=torch.int64, device=device)
        self._epoch = torch.zeros(n_cta, dtype=torch.int32, device=device)
        self._keep = keep                                  # whatever owns the mapped memory
        self.status = torch.zeros(4, dtype=torch.int32, device=device)
        self.x = _lib.Exchange(world, rank, batch, n_q, head_dim, n_cta, self._ptr_data.data_ptr(),
                               self._epoch.data_ptr())

    def run(self, packed: Optional[torch.Tensor], out: Optional[torch.Tensor],
            phases: int = _lib.EXCHANGE_PUSH | _lib.EXCHANGE_MERGE) -> None:
        _lib.check(_lib.load().pkv_exchange_merge(ctypes.byref(self.x), _lib.ptr(packed), _lib.ptr(out), phases,
                                                  _lib.ptr(self.status), _lib.current_stream()), "pkv_exchange_merge")

    def run_parts(self, partials: torch.Tensor, n_split: int, out: torch.Tensor) -> None:
        """Merge of the local split-T partials [B, n_split, H, d+2] and the exchange in ONE launch
        (`pkv_merge_exchange`); needs a handle made with ``n_cta = batch * n_q``."""
        pw = self.x.head_dim + 2
        _lib.check(_lib.load().pkv_merge_exchange(ctypes.byref(self.x), _lib.ptr(partials), n_split * self.x.n_q * pw,
                                                  self.x.n_q * pw, n_split, _lib.ptr(out), _lib.ptr(self.status),
                                                  _lib.current_stream()), "pkv_merge_exchange")

    # ------------------------------------------------------------------ construction
    @classmethod
    def local_group(cls, world: int, batch: int, n_q: int, head_dim: int, device="cuda", n_cta: int = 64):
        """All `world` ranks on ONE GPU (tests): every rank's buffer is an ordinary allocation of the
        same device, so each handle can address all of them. Drive it phase by phase: all pushes,
        then all merges; kernels that wait on each other must not share a GPU."""
        bufs = [torch.zeros(gather_words(world, batch, n_q, head_dim), dtype=torch.int64, device=device)
                for _ in range(world)]
        dp = [b.data_ptr() for b in bufs]
        return [cls(world, r, batch, n_q, head_dim, dp, device, n_cta, keep=bufs) for r in range(world)]

    @classmethod
    def from_process_group(cls, group, batch: int, n_q: int, head_dim: int, device, n_cta: int = 64):
        """One rank per process: the buffer lives in torch's symmetric memory (peer mappings over
        NVLink), rendezvoused on `group`."""
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        data = symm.empty(gather_words(world, batch, n_q, head_dim), dtype=torch.int64, device=device)
        data.zero_()
        hd = symm.rendezvous(data, group.group_name if hasattr(group, "group_name") else group)
        torch.cuda.synchronize(device)
        dist.barrier(group)                                 # every rank has zeroed its buffer before anyone pushes
        return cls(world, rank, batch, n_q, head_dim, [int(p) for p in hd.buffer_ptrs], device, n_cta, keep=(data, hd))
