"""Child process of tests/test_gpu_multi.py: one rank of a token-sharded decode on its own GPU."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    from helpers import Scenario, rel
    from phasorkv_b200.sharded import ShardExchange, token_range
    T = 2048
    full = Scenario("cfg2", seqlens=(T, T // 2), gain=64.0, pos0=50000)          # same seeds on every rank
    ws_full = full.pk.workspace(full.B, 2)
    full.pk.absorb_step(full.q.cuda(), full.qpos.cuda(), ws_full)
    full.pk.attend_step(full.cache, ws_full, out=ws_full.out)
    # this rank's token range of every sequence in its own cache
    lens = [token_range(rank, world, Tb)[1] - token_range(rank, world, Tb)[0] for Tb in full.seqlens]
    cache = full.pk.new_cache(full.B, max(lens))
    for b, Tb in enumerate(full.seqlens):
        lo, hi = token_range(rank, world, Tb)
        n = hi - lo
        seq = torch.full((n,), b, dtype=torch.int32, device=dev)
        slots = cache.slots(seq, torch.arange(n, dtype=torch.int32, device=dev))
        full.pk.write_paged(cache, full.x[b][lo:hi].cuda(), full.pos[b][lo:hi].to(torch.int32).cuda(), slots,
                            v=full.v[b][lo:hi].cuda())
    cache.seqlens.copy_(torch.tensor(lens, dtype=torch.int32))
    ex = ShardExchange.from_process_group(dist.group.WORLD, full.B, full.spec.n_q, full.spec.head_dim, dev)
    ws = full.pk.workspace(full.B, 2)
    out = torch.empty_like(ws.out)
    errs = []
    for rnd in range(3):
        full.pk.absorb_step(full.q.cuda(), full.qpos.cuda(), ws)
        full.pk.attend_step(cache, ws, packed_out=ws.packed)
        ex.run(ws.packed, out)
        torch.cuda.synchronize()
        errs.append(rel(out.cpu(), ws_full.out.cpu()))
        assert int(ex.status.abs().sum()) == 0
    # the NCCL route gives the same answer
    gathered = torch.empty((world,) + tuple(ws.packed.shape), device=dev)
    dist.all_gather_into_tensor(gathered, ws.packed)
    out2 = torch.empty_like(out)
    full.pk.merge_gathered(gathered, out2)
    torch.cuda.synchronize()
    errs.append(rel(out2.cpu(), out.cpu()))
    # local merge + exchange in one launch (its own handle: one epoch counter per row)
    ex2 = ShardExchange.from_process_group(dist.group.WORLD, full.B, full.spec.n_q, full.spec.head_dim, dev,
                                           n_cta=full.B * full.spec.n_q)
    out3 = torch.empty_like(out)
    for rnd in range(3):
        full.pk.absorb_step(full.q.cuda(), full.qpos.cuda(), ws)
        full.pk.attend_step(cache, ws, after_absorb=True)
        ex2.run_parts(ws.partials, ws.n_split, out3)
        torch.cuda.synchronize()
        errs.append(rel(out3.cpu(), out.cpu()))
        assert int(ex2.status.abs().sum()) == 0
    # the step as the benchmark runs it: the rank that owns the newest position of every sequence (the last one)
    # rewrites that token with the one-launch prologue, raising the operand-ready counters its attention polls;
    # the other ranks absorb. Reference: the same rewrite on the unsharded cache.
    from phasorkv_b200 import synth
    from phasorkv_b200.sharded import owner_of
    g = torch.Generator().manual_seed(123)
    x_new = (synth.make_hidden(g, full.B, 4096) * 2.0).cuda()
    v_new = (synth.make_values(g, full.B, full.spec.n_kv, full.spec.head_dim) * 3.0).cuda()
    seq = torch.arange(full.B, dtype=torch.int32, device=dev)
    glob_last = torch.tensor([Tb - 1 for Tb in full.seqlens], dtype=torch.int32, device=dev)
    wpos = (glob_last + 50000).contiguous()
    full.pk.prologue_step(full.cache, x_new, wpos, full.cache.slots(seq, glob_last), full.q.cuda(), full.qpos.cuda(), ws_full, v=v_new)
    ref4 = torch.empty_like(out)
    full.pk.attend_step(full.cache, ws_full, out=ref4, after_prologue=True)
    assert all(owner_of(Tb - 1, world, Tb) == world - 1 for Tb in full.seqlens)
    out4 = torch.empty_like(out)
    for rnd in range(2):
        if rank == world - 1:
            loc_last = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=dev)
            full.pk.prologue_step(cache, x_new, wpos, cache.slots(seq, loc_last), full.q.cuda(), full.qpos.cuda(), ws, v=v_new,
                                  signal=True)
            full.pk.attend_step(cache, ws, after_prologue=True, polled=True)
        else:
            full.pk.absorb_step(full.q.cuda(), full.qpos.cuda(), ws)
            full.pk.attend_step(cache, ws, after_absorb=True)
        ex2.run_parts(ws.partials, ws.n_split, out4)
        torch.cuda.synchronize()
        errs.append(rel(out4.cpu(), ref4.cpu()))
        assert int(ex2.status.abs().sum()) == 0 and int(ws.status.abs().sum()) == 0 and int(ws.qsync.abs().sum()) == 0
    assert max(errs[-2:]) < 2e-3 and rel(ref4.cpu(), ws_full.out.cpu()) > 1e-3          # the rewrite changed the answer
    print(f"rank {rank}: rel errors {errs}", flush=True)
    assert max(errs[:3]) < 2e-3 and errs[3] < 1e-5 and max(errs[4:7]) < 1e-5
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
