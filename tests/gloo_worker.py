"""Child process of tests/test_host_cpu.py: one CPU rank (gloo) of a token-sharded decode computed with
the oracle. Checks the host-side sharding rule of the package (token ranges, owner of the newest token)
and that all-gathered partial triples merge to the unsharded result."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    from oracle import phasor_oracle as po
    from phasorkv_b200 import synth
    from phasorkv_b200.sharded import gather_words, owner_of, token_range
    spec = synth.make_layer("cfg2", 0, d_model=512, factor_gain=32.0)
    pk = po.PhasorKeyOracle.from_spec(spec)
    gen = torch.Generator().manual_seed(17)                     # same seeds on every rank
    T = 301                                                     # not a multiple of the group size
    x = synth.make_hidden(gen, T, 512)
    V = synth.make_values(gen, T, spec.n_kv, spec.head_dim)
    q = synth.make_query(gen, 1, spec.n_q, spec.head_dim)[0]
    rows = pk.write(x, po.rope_phasors(spec.inv_freq, torch.arange(T)))
    qa = pk.absorb(q[:, None, :], po.rope_phasors(spec.inv_freq, torch.tensor([T])))[:, 0]
    S = pk.scores(qa, rows)
    full = po.attend(S, V, spec.n_kv, spec.head_dim)
    lo, hi = token_range(rank, world, T)
    m, l, o = po.partial_attend(S[:, lo:hi], V[lo:hi], spec.n_kv, spec.head_dim)
    packed = torch.cat([o, m[:, None], l[:, None]], dim=1).contiguous()            # [H, d+2], the exchanged triple
    gathered = [torch.empty_like(packed) for _ in range(world)]
    dist.all_gather(gathered, packed)
    g = torch.stack(gathered)
    merged = po.merge_partials(g[:, :, -2], g[:, :, -1], g[:, :, :-2])
    err = float((merged - full).norm() / full.norm())
    # every rank sees the same ranges: disjoint, covering, owner of the newest token is the last rank
    ranges = [token_range(r, world, T) for r in range(world)]
    assert ranges[0][0] == 0 and ranges[-1][1] == T and all(ranges[i][1] == ranges[i + 1][0] for i in range(world - 1))
    assert owner_of(T - 1, world, T) == world - 1 and owner_of(0, world, T) == 0
    assert gather_words(world, 4, 32, 128) == 2 * world * 4 * 32 * 130
    assert err < 1e-5, err
    print(f"rank {rank}: tokens [{lo}, {hi}) merged rel err {err:.2e}", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
