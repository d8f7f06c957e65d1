#!/usr/bin/env python
"""Decode benchmark of the B200 PhasorKey path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2] [--algo tc|simt]
  python bench.py --impl reference ...        # the CPU PhasorKey path on the host cores

One *step* is one decode step of a whole model-depth stack: for each of 32 layers, the newest token
of every sequence is written into the NVFP4 latent / bf16 V cache, the query is absorbed, and
split-T attention + merge produce the output. Inputs are seeded synthetic tensors with the shapes
of Llama-3.1-8B (the reference benchmarks its kernels on random factors and caches too,
scripts/bench_decode.py:4-8); cache contents are real writes of seeded hidden states.

N > 1 (launched by torch.distributed.run, one rank per GPU): every rank runs its own batch (batch
parallel, no communication, weak scaling); in addition the token-sharded 128k configuration is
timed (`seq_sharded`), where each rank attends over its slice of the tokens and the partial
(o, m, l) triples are exchanged by one NCCL all-gather per layer.

Prints one JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_LAYERS = 32
D_MODEL = 4096
L2_BYTES = 126 * 2 ** 20


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=["cfg2", "cfg3", "cfg5"])
    ap.add_argument("--algo", default=os.environ.get("PKV_BENCH_ALGO", "tc"), choices=["tc", "simt"])
    ap.add_argument("--layers", type=int, default=N_LAYERS)
    ap.add_argument("--batch", type=int, default=0, help="override the configuration's batch (profiling)")
    ap.add_argument("--context", type=int, default=0, help="override the configuration's context (profiling)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sharded", action="store_true")
    ap.add_argument("--collective", default="p2p", choices=["p2p", "nccl"],
                    help="token-sharded exchange: own peer-memory kernel, or NCCL all-gather + merge")
    ap.add_argument("--no-graph", action="store_true", help="time the token-sharded step eagerly instead of as a CUDA graph")
    ap.add_argument("--splits", type=int, default=0)
    return ap.parse_args()


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------

class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            t_end = time.time() + 5.0                       # nvidia-smi needs a moment before its first line
            while not self.rows and time.time() < t_end:
                time.sleep(0.02)
            self.skip = len(self.rows)                      # samples taken before the GPU was under load
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.rows = self.rows[getattr(self, "skip", 0):] or self.rows
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# the GPU arm
# ------------------------------------------------------------------------------------------------

class Stack:
    """32 layers of one configuration with their caches filled by real writes of seeded hidden states."""

    def __init__(self, config: str, n_layers: int, device, algo: str, seed: int, batch: int = 0, context: int = 0,
                 n_split: int = 0):
        from phasorkv_b200 import synth
        from phasorkv_b200.latent import PhasorKey
        c = synth.CONFIGS[config]
        self.config, self.algo = config, algo
        # cfg5 is quoted on 8 GPUs (64 sequences, 8 per GPU: 69 GB of cache per GPU); the others fit one GPU whole
        self.B = batch or (c["batch"] // 8 if config == "cfg5" else c["batch"])
        need = self.B * (context or c["context"]) * n_layers * 2 * 1.02
        spec0 = synth.make_layer(config, 0)
        need *= (spec0.cache_width * 9 // 16 + spec0.n_kv * spec0.head_dim * 2) / 2
        free = torch.cuda.mem_get_info(device)[0]
        if need > 0.9 * free:
            raise SystemExit("workload %s needs %.0f GB of cache on this GPU, %.0f GB are free: lower --batch / --context / --layers"
                             % (config, need / 1e9, free / 1e9))
        self.T = context or c["context"]
        self.device = device
        self.simt = algo == "simt"
        self.fused_prologue = os.environ.get("PKV_BENCH_SEPARATE_PROLOGUE", "0") != "1"
        # PKV_BENCH_INLINE_ABSORB=1: the write alone as prologue and pkv_decode_attn_q (absorption inside the attention
        # kernel). Measured slower at present (251 against 196 us per layer): the default keeps the fused prologue.
        self.inline_absorb = os.environ.get("PKV_BENCH_INLINE_ABSORB", "0") == "1"
        self.layers, self.caches = [], []
        g = torch.Generator(device=device).manual_seed(seed)
        for l in range(n_layers):
            pk = PhasorKey.from_spec(synth.make_layer(config, l), device=device)
            self.layers.append(pk)
        pk0 = self.layers[0]
        self.n_q, self.n_kv, self.d = pk0.n_q, pk0.n_kv, pk0.head_dim
        self.W = pk0.cache_width
        # tensor scale per layer: the reference's static rule on a 4096-token calibration write
        n_out = max(1, round(0.01 * D_MODEL))
        self.outliers = torch.randperm(D_MODEL, generator=g, device=device)[:n_out]
        xc = self._hidden(g, 4096)
        pos = torch.arange(4096, dtype=torch.int32, device=device)
        rows = torch.empty((4096, self.W), dtype=torch.float32, device=device)
        for pk in self.layers:
            pk.write_paged(None, xc, pos, None, latent_out=rows)
            pk.calibrate_second(rows)
        del rows, xc
        for pk in self.layers:
            self.caches.append(pk.new_cache(self.B, self.T))
        chunk = 16384
        for b in range(self.B):
            for t0 in range(0, self.T, chunk):
                n = min(chunk, self.T - t0)
                x = self._hidden(g, n).to(torch.bfloat16)
                lp = torch.arange(t0, t0 + n, dtype=torch.int32, device=device)
                seq = torch.full((n,), b, dtype=torch.int32, device=device)
                for pk, cache in zip(self.layers, self.caches):
                    slots = cache.slots(seq, lp)
                    pk.write_paged(cache, x, lp, slots)
                    cache.set_v_rows(slots, torch.randn((n, self.n_kv * self.d), generator=g, device=device,
                                                        dtype=torch.float32))
        for cache in self.caches:
            cache.seqlens.fill_(self.T)
        self.n_split = n_split or pk0.default_splits(self.B, self.T, self.simt)
        self.ws = [pk0.workspace(self.B, self.n_split) for _ in range(2)]
        # per-step inputs (all layers): newest hidden state, its V row, the query; output buffer
        L = n_layers
        self.x_new = torch.empty((L, self.B, D_MODEL), dtype=torch.bfloat16, device=device)
        self.v_new = torch.empty((L, self.B, self.n_kv * self.d), dtype=torch.bfloat16, device=device)
        self.q = torch.empty((L, self.B, self.n_q, self.d), dtype=torch.float32, device=device)
        self.out = torch.empty((L, self.B, self.n_q, self.d), dtype=torch.float32, device=device)
        self.x_new.copy_(self._hidden(g, L * self.B).view(L, self.B, D_MODEL))
        self.v_new.copy_(torch.randn(self.v_new.shape, generator=g, device=device))
        self.q.copy_(torch.randn(self.q.shape, generator=g, device=device))
        self.qpos = torch.full((self.B,), self.T, dtype=torch.int32, device=device)
        self.wpos = torch.full((self.B,), self.T - 1, dtype=torch.int32, device=device)
        seq = torch.arange(self.B, dtype=torch.int32, device=device)
        self.wslots = [c.slots(seq, self.wpos) for c in self.caches]
        self.launches_per_layer = 0

    def _hidden(self, g, n):
        x = torch.randn((n, D_MODEL), generator=g, device=self.device, dtype=torch.float32)
        x[:, self.outliers] *= 20.0
        return x

    def step(self, events=None, scores_only=False, write=True, pre=None, post=None):
        """One decode step over all layers. `events`: list receiving (start, end) CUDA events around
        each attention launch. `pre(l)` / `post(l)` run on the host before / after layer l is enqueued."""
        n = 0
        for l, (pk, cache) in enumerate(zip(self.layers, self.caches)):
            ws = self.ws[l & 1]
            if pre is not None:
                pre(l)
            fused = write and not self.simt and self.fused_prologue
            inline = fused and self.inline_absorb and not scores_only
            if inline:                                                # the write alone; attention absorbs the raw queries
                pk.prologue_step(cache, self.x_new[l], self.wpos, self.wslots[l], None, None, ws, v=self.v_new[l])
                n += 1
            elif fused:                                               # newest token's write + absorb: one launch
                pk.prologue_step(cache, self.x_new[l], self.wpos, self.wslots[l], self.q[l], self.qpos, ws, v=self.v_new[l])
                n += 1
            else:
                if write:
                    pk.write_paged(cache, self.x_new[l], self.wpos, self.wslots[l], v=self.v_new[l], scratch=ws.wscratch)
                    n += 2
                pk.absorb_step(self.q[l], self.qpos, ws, operand=not self.simt)
                n += 1
            if events is not None:
                e0 = torch.cuda.Event(enable_timing=True)
                e1 = torch.cuda.Event(enable_timing=True)
                e0.record()
            if inline:
                # the queries of the step exist before the layer's first launch: attention starts with the write,
                # streams pages and absorbs at once, and waits for the write only before the page being written
                pk.attend_q_step(cache, self.q[l], self.qpos, ws, early=events is None, tail_written=True, query_ready=True)
            else:
                pk.attend_step(cache, ws, simt=self.simt, scores_only=scores_only, after_absorb=events is None and not fused,
                               after_prologue=events is None and fused)
            if events is not None:
                e1.record()
                events.append((e0, e1))
            pk.merge_step(ws, out=self.out[l])
            n += 2
            if post is not None:
                post(l)
        self.launches_per_layer = n // len(self.layers)
        return n

    # bytes one attention launch must move (per layer): NVFP4 codes + scales, and bf16 V
    def bytes_k(self):
        return self.B * self.T * (self.W // 2 + self.W // 16)

    def bytes_full(self):
        return self.bytes_k() + self.B * self.T * self.n_kv * self.d * 2


def timed(fn, steps, warmup, dist=None):
    """W warm-up calls, then exactly K calls between barrier + synchronize; device time by CUDA events."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    ms = a.elapsed_time(b)
    if dist is not None:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t)
    return ms / steps


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p)), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


def run_b200(args):
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    # stdout carries the one JSON line and nothing else: libraries that greet on file descriptor 1
    # (NCCL prints its version there) are pointed at stderr until the line is written
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    if world > 1:
        import torch.distributed as dist_
        dist_.init_process_group("nccl", device_id=device)
        dist = dist_
    from phasorkv_b200 import _lib
    _lib.check(_lib.load().pkv_device_check(), "pkv_device_check")

    st = Stack(args.workload, args.layers, device, args.algo, seed=1234 + rank, batch=args.batch, context=args.context,
               n_split=args.splits)
    torch.cuda.synchronize()

    # ---- device-resident timing of exactly K steps
    sampler = ClockSampler(local)
    sampler.start()
    launches = {"n": 0}

    def full_step():
        launches["n"] += st.step()
    ms_step = timed(full_step, args.steps, args.warmup, dist)
    # ---- the same K steps once more with CUDA events around every attention launch: the per-launch
    # duration the roofline is computed from (the events sit between kernels of the chain, so this pass
    # is kept apart from the one that gives `value`)
    events = []
    ms_step_ev = timed(lambda: st.step(events=events), args.steps, 1, dist)
    clocks = sampler.stop()
    timed_events = events[-args.steps * args.layers:]
    attn_ms = sum(a.elapsed_time(b) for a, b in timed_events) / len(timed_events)
    gpu_launches = st.launches_per_layer * args.layers * args.steps

    # ---- K path only (logits + log-sum-exp, V never read): the "K-path us/layer" of the metric
    ev_k = []
    ms_k = timed(lambda: st.step(events=ev_k, scores_only=True, write=False), max(2, args.steps // 2), 2, dist)
    k_events = ev_k[-max(2, args.steps // 2) * args.layers:]
    attn_k_ms = sum(a.elapsed_time(b) for a, b in k_events) / len(k_events)

    # ---- end to end through the host API: pinned host inputs in, outputs back, every step
    L = args.layers
    hx = torch.empty(st.x_new.shape, dtype=st.x_new.dtype).pin_memory()
    hv = torch.empty(st.v_new.shape, dtype=st.v_new.dtype).pin_memory()
    hq = torch.empty(st.q.shape, dtype=st.q.dtype).pin_memory()
    ho = torch.empty(st.out.shape, dtype=st.out.dtype).pin_memory()
    hx.copy_(st.x_new); hv.copy_(st.v_new); hq.copy_(st.q)

    # Host copies ride on their own streams in groups of layers, so that the inputs of the next group
    # arrive and the outputs of the previous one leave while a group computes; every byte still crosses
    # inside the timed region, which ends only after the last output has landed in host memory.
    GROUP = 4
    groups = [(g, min(g + GROUP, L)) for g in range(0, L, GROUP)]
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in groups]
    ev_done = [torch.cuda.Event() for _ in groups]

    def e2e_step():
        main = torch.cuda.current_stream()
        s_in.wait_stream(main)                      # the previous step has consumed its inputs
        with torch.cuda.stream(s_in):
            for gi, (a, b_) in enumerate(groups):
                st.x_new[a:b_].copy_(hx[a:b_], non_blocking=True)
                st.v_new[a:b_].copy_(hv[a:b_], non_blocking=True)
                st.q[a:b_].copy_(hq[a:b_], non_blocking=True)
                ev_in[gi].record(s_in)

        def pre(l):
            if l % GROUP == 0:
                main.wait_event(ev_in[l // GROUP])

        def post(l):
            if (l + 1) % GROUP == 0 or l == L - 1:
                gi = l // GROUP
                ev_done[gi].record(main)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_done[gi])
                    a, b_ = groups[gi]
                    ho[a:b_].copy_(st.out[a:b_], non_blocking=True)
        st.step(pre=pre, post=post)
        main.wait_stream(s_out)
    ms_e2e = timed(e2e_step, args.steps, args.warmup, dist)
    h2d = hx.numel() * hx.element_size() + hv.numel() * hv.element_size() + hq.numel() * hq.element_size()
    d2h = ho.numel() * ho.element_size()

    # ---- token-sharded long context (cfg4): the same pools viewed as B=4, T=131072/world per rank
    sharded = None
    if not args.no_sharded and args.workload == "cfg2" and not args.batch and not args.context:
        try:
            sharded = run_sharded(st, args, dist, world)
        except Exception as e:                       # the headline line is still reported
            sys.stderr.write("token-sharded run failed: %r\n" % (e,))
            sharded = {"workload": "cfg4", "error": repr(e)[:300]}

    pk, src = peaks()
    # DRAM traffic per launch: an ncu capture of this kernel at B=16, T=8192 (W=256, 8 kv heads) read
    # 287.82 MB for 131072 tokens, 1.002 x the algorithmic bytes; reads scale with the tokens streamed, the
    # split partials written (B x n_split x 32 x 130 floats) do not.
    traffic = None
    if args.algo == "tc" and st.W == 256 and st.n_kv == 8:
        traffic = int(287.82e6 * (st.B * st.T) / 131072 + st.B * st.n_split * 32 * 130 * 4)
    achieved = st.bytes_full() / (attn_ms * 1e-3) / 1e9
    roof = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
            "frac": round(achieved / pk["hbm_gbs"], 4), "traffic": traffic, "peak_source": src,
            "kernel": "pkv_attn_%s" % args.algo, "bytes_per_launch": st.bytes_full(),
            "us_per_launch": round(attn_ms * 1e3, 2),
            "timed_over": "%d launches of a second pass of the same %d steps with CUDA events around each attention "
                          "launch (%.4f ms per step in that pass)" % (len(timed_events), args.steps, ms_step_ev)}
    line = {
        "metric": "decode tokens/s (B=%d, T=%d, %d layers; K-path us/layer and HBM GB/s beside it)" % (st.B, st.T, L),
        "value": round(world * st.B / (ms_step * 1e-3), 2), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4 latent (e2m1 x ue4m3) x nvfp4 query, fp32 accumulate; bf16 V",
        "data": "synthetic",
        "config": {"workload": "%s: %s layer shape, B=%d per GPU, T=%d, NVFP4 latent W=%d, bf16 V %dx%d, %d layers"
                   % (args.workload, "7B multi-head-attention" if st.n_kv == st.n_q else "Llama-3.1-8B", st.B, st.T, st.W,
                      st.n_kv, st.d, L),
                   "algo": args.algo, "n_split": st.n_split, "parallelism": "batch-parallel x%d" % world,
                   "l2": "inputs larger than L2 (%.2f GB streamed per layer, %.1f GB per step)"
                         % (st.bytes_full() / 1e9, L * st.bytes_full() / 1e9)},
        "k_path_us_per_layer": round(attn_k_ms * 1e3, 2),
        "k_path_gbs": round(st.bytes_k() / (attn_k_ms * 1e-3) / 1e9, 1),
        "full_us_per_layer": round(ms_step * 1e3 / L, 2),
        "hbm_gbs": round(achieved, 1),
        "roofline": roof,
        "e2e": {"value": round(world * st.B / (ms_e2e * 1e-3), 2), "unit": "tokens/s", "ms_per_step": round(ms_e2e, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": gpu_launches,
        "clocks": clocks,
    }
    if sharded is not None:
        line["seq_sharded"] = sharded
    if rank == 0 and not args.no_cpu_baseline and world == 1:
        line["cpu_baseline"] = cpu_baseline(args.workload, budget_s=15.0)
    sys.stdout.flush()
    os.dup2(real_stdout, 1)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_sharded(st, args, dist, world):
    """cfg4: B=4, T=131072 with the token axis split evenly over the ranks; one all-gather per layer."""
    B4, T4 = 4, 131072
    Tl = T4 // world
    pages = Tl // 128
    dev = st.device
    pt = torch.arange(B4 * pages, dtype=torch.int32, device=dev).reshape(B4, pages)
    seqlens = torch.full((B4,), Tl, dtype=torch.int32, device=dev)
    pk0 = st.layers[0]
    n_split = max(1, min(pages, (torch.cuda.get_device_properties(dev).multi_processor_count * (3 if st.simt else 1)) // B4))
    ws = pk0.workspace(B4, n_split)
    gathered = torch.empty((world, B4, st.n_q, st.d + 2), dtype=torch.float32, device=dev)
    out = torch.empty((B4, st.n_q, st.d), dtype=torch.float32, device=dev)
    qpos = torch.full((B4,), T4, dtype=torch.int32, device=dev)
    saved = [(c.page_table, c.seqlens, c.max_pages) for c in st.caches]
    ex = None
    if world > 1 and args.collective == "p2p":
        # peer buffers in torch symmetric memory; if any rank cannot set them up, every rank takes the NCCL route
        from phasorkv_b200.sharded import ShardExchange
        ok = 1
        try:
            ex = ShardExchange.from_process_group(dist.group.WORLD, B4, st.n_q, st.d, dev, n_cta=B4 * st.n_q)
        except Exception as e:
            ok = 0
            sys.stderr.write("symmetric-memory exchange unavailable, using NCCL all-gather: %r\n" % (e,))
        agreed = torch.tensor([ok], dtype=torch.int32, device=dev)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if int(agreed.item()) == 0:
            ex = None
    # the newest token (global position T-1) belongs to the last rank: only that rank writes it
    from phasorkv_b200.sharded import owner_of
    owner = int(os.environ.get("RANK", 0)) == owner_of(T4 - 1, world, T4) and not st.simt
    wpos = torch.full((B4,), T4 - 1, dtype=torch.int32, device=dev)
    wslots = (pt[:, (Tl - 1) // 128] * 128 + (Tl - 1) % 128).to(torch.int32).contiguous()

    inline = st.inline_absorb and not st.simt

    def attend(pk, cache, l, **out_kw):
        """attention of layer l on this rank's shard: raw queries absorbed in the kernel, or absorb launch + operand"""
        if inline:
            if owner:                                       # the write alone; attention waits for it before the last page only
                pk.prologue_step(cache, st.x_new[l, :B4], wpos, wslots, None, None, ws, v=st.v_new[l, :B4])
            pk.attend_q_step(cache, st.q[l, :B4], qpos, ws, early=True, tail_written=owner, query_ready=True, **out_kw)
        else:
            if owner:
                pk.prologue_step(cache, st.x_new[l, :B4], wpos, wslots, st.q[l, :B4], qpos, ws, v=st.v_new[l, :B4])
            else:
                pk.absorb_step(st.q[l, :B4], qpos, ws, operand=not st.simt)
            early = dict(after_prologue=True) if owner else dict(after_absorb=True)
            pk.attend_step(cache, ws, simt=st.simt, **early, **out_kw)

    def step():
        for l, (pk, cache) in enumerate(zip(st.layers, st.caches)):
            if world > 1:
                if ex is not None:
                    attend(pk, cache, l)
                    ex.run_parts(ws.partials, ws.n_split, out)      # local merge + peer stores + merge, one kernel
                else:
                    attend(pk, cache, l, packed_out=ws.packed)      # local splits merged by a launch behind
                    dist.all_gather_into_tensor(gathered, ws.packed)
                    pk.merge_gathered(gathered, out)
            else:
                attend(pk, cache, l, out=out)
    for c in st.caches:
        c.page_table, c.seqlens, c.max_pages = pt, seqlens, pages
    graphed = False
    try:
        fn = step
        if not args.no_graph:
            # at 1/8 of the tokens per GPU a layer lasts tens of microseconds: the step is replayed as one
            # CUDA graph (kernels, all-gather and all) so that the host is out of the loop, as the
            # reference times its kernels (scripts/bench_decode.py:29-49)
            try:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    step()
                    step()
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    step()
                fn, graphed = g.replay, True
            except Exception as e:                                  # capture refused: time the eager step
                sys.stderr.write("graph capture of the sharded step failed: %r\n" % (e,))
                torch.cuda.synchronize()
        ms = timed(fn, args.steps, args.warmup, dist)
    finally:
        for c, s in zip(st.caches, saved):
            c.page_table, c.seqlens, c.max_pages = s
    per_gpu_bytes = B4 * Tl * (st.W // 2 + st.W // 16 + st.n_kv * st.d * 2)
    return {"workload": "cfg4: B=4, T=131072, tokens split evenly over %d GPU(s), %d layers" % (world, args.layers),
            "value": round(B4 / (ms * 1e-3), 2), "unit": "tokens/s", "ms_per_step": round(ms, 4), "n_gpus": world,
            "scaling": "strong", "cuda_graph": graphed, "newest_token_written_by": "rank %d (fused prologue)" % (world - 1),
            "collective": "none" if world == 1 else ("local merge + exchange + merge in one kernel over NVLink peer memory, [B,H,d+2] fp32 per layer"
                                                     if ex is not None else "NCCL all_gather of [B,H,d+2] fp32 per layer + merge"),
            "allgather_bytes_per_gpu_per_layer": B4 * st.n_q * (st.d + 2) * 4 if world > 1 else 0,
            "hbm_gbs_per_gpu": round(per_gpu_bytes * args.layers / (ms * 1e-3) / 1e9, 1)}


# ------------------------------------------------------------------------------------------------
# the CPU arm: the reference's PhasorKey arithmetic (oracle port) on the host cores
# ------------------------------------------------------------------------------------------------

def cpu_sample(workload: str, n_seq: int = 1):
    """One (layer, sequence) unit of the workload prepared for the CPU path; returns a closure that
    runs absorb + scores + softmax + P.V once, and the unit's description."""
    from oracle import phasor_oracle as po
    from phasorkv_b200 import synth
    c = synth.CONFIGS[workload]
    T = c["context"]
    spec = synth.make_layer(workload, 0)
    pk = po.PhasorKeyOracle.from_spec(spec)
    gen = torch.Generator().manual_seed(99)
    rows = []
    for t0 in range(0, T, 4096):
        x = synth.make_hidden(gen, 4096)
        rows.append(pk.write(x, po.rope_phasors(spec.inv_freq, torch.arange(t0, t0 + 4096))))
    rows = torch.cat(rows)
    second = po.nv_static_second(rows[:4096].var(0))
    rows = po.nvfp4_quantize(rows, second)[2]                      # the dequantised latent, fp32 [T, W]
    V = synth.make_values(gen, T, spec.n_kv, spec.head_dim)
    q = synth.make_query(gen, 1, spec.n_q, spec.head_dim)[0]
    ph_q = po.rope_phasors(spec.inv_freq, torch.tensor([T]))

    def unit():
        return po.decode_step(pk, q, ph_q, rows, V, spec.head_dim)
    return unit, c


def cpu_baseline(workload: str, budget_s: float = 15.0) -> dict:
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    unit, c = cpu_sample(workload)
    unit(); unit()
    ts = []
    t_end = time.perf_counter() + budget_s
    while len(ts) < 5 or (time.perf_counter() < t_end and len(ts) < 50):
        t0 = time.perf_counter()
        unit()
        ts.append(time.perf_counter() - t0)
    ts.sort()
    t_unit = ts[len(ts) // 2]
    step_s = t_unit * c["batch"] * N_LAYERS
    return {"value": round(c["batch"] / step_s, 4), "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": "1 layer x 1 sequence of T=%d (absorb + scores + softmax + P.V, fp32 on the dequantised latent, "
                      "bf16 V), median of %d runs = %.2f ms, scaled x%d sequences x%d layers"
                      % (c["context"], len(ts), t_unit * 1e3, c["batch"], N_LAYERS)}


def run_reference(args):
    """--impl reference: the CPU path timed as the step itself; rank 0 only."""
    if int(os.environ.get("RANK", 0)) != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    unit, c = cpu_sample(args.workload)
    for _ in range(max(1, min(args.warmup, 3))):
        unit()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        unit()
    t_unit = (time.perf_counter() - t0) / args.steps
    step_s = t_unit * c["batch"] * N_LAYERS
    val = round(c["batch"] / step_s, 4)
    sample = ("each step = 1 layer x 1 sequence of T=%d through the oracle port of PhasorKey (absorb + scores + softmax + "
              "P.V), %.2f ms; scaled x%d sequences x%d layers to a full decode step" % (c["context"], t_unit * 1e3, c["batch"], N_LAYERS))
    line = {"impl": "reference",
            "metric": "decode tokens/s (B=%d, T=%d, %d layers; K-path us/layer and HBM GB/s beside it)" % (c["batch"], c["context"], N_LAYERS),
            "value": val, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(step_s * 1e3, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": "%s: Llama-3.1-8B layer shape, B=%d, T=%d, fp32 dequantised latent, bf16 V, %d layers"
                       % (args.workload, c["batch"], c["context"], N_LAYERS)},
            "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_b200(a)
