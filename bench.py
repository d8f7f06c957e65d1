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
timed (`seq_sharded`; `--workload cfg4` makes it the headline line), where each rank attends over its
slice of the tokens and the partial (o, m, l) triples are exchanged by the library's own peer-memory
kernel over NVLink (`--collective nccl`: one NCCL all-gather per layer + merge). After the timed
replays the sharded run checks itself: status words, the two exchange routes against each other and
the tensor-core result against the CUDA-core kernel (`seq_sharded.check`).

`--workload cfg5` is the 7B multi-head shape with, per step and layer, a 2048-token chunk write for
each of the GPU's 8 sequences (tensor-core cache write) plus the decode step.

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
    ap.add_argument("--workload", default="cfg2", choices=["cfg2", "cfg3", "cfg4", "cfg5"])
    ap.add_argument("--no-chunk-write", action="store_true", help="cfg5 without its 2048-token chunk write per step")
    ap.add_argument("--v-format", default="bf16", choices=["bf16", "q3", "q2"],
                    help="V pages: bf16 (the configurations as stated) or per-token 3-bit / 2-bit tiers (quantised V)")
    ap.add_argument("--algo", default=os.environ.get("PKV_BENCH_ALGO", "tc"), choices=["tc", "simt"])
    ap.add_argument("--layers", type=int, default=N_LAYERS)
    ap.add_argument("--batch", type=int, default=0, help="override the configuration's batch (profiling)")
    ap.add_argument("--context", type=int, default=0, help="override the configuration's context (profiling)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sharded", action="store_true")
    ap.add_argument("--collective", default="p2p", choices=["p2p", "nccl"],
                    help="token-sharded exchange: own peer-memory kernel, or NCCL all-gather + merge")
    ap.add_argument("--no-graph", action="store_true", help="time the steps as eager launches instead of CUDA graph replays")
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
                 n_split: int = 0, chunk_write: bool = True, v_bits: int = 0):
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
        # PKV_BENCH_POLLED=0: the attention waits for the whole launch before it instead of polling the
        # operand-ready counters that launch raises
        self.polled = os.environ.get("PKV_BENCH_POLLED", "1") == "1"
        # behind the small absorb launch (the K-path pass) the plain dependent launch is as fast: off unless asked for
        self.polled_absorb = os.environ.get("PKV_BENCH_POLLED_ABSORB", "0") == "1"
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
            self.caches.append(pk.new_cache(self.B, self.T, v_bits=v_bits))
        self.v_bits = v_bits
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
        # cfg5: per step and layer a chunk of `chunk` tokens is written for every sequence (a chunked prefill
        # riding along with the decode step): the tokens just before the newest one, the same seeded hidden
        # states for all layers (134 MB of bf16 x at 8 x 2048 tokens: larger than L2)
        self.chunk = int(c.get("chunk", 0)) if chunk_write else 0
        if self.chunk:
            n = self.B * self.chunk
            self.x_chunk = self._hidden(g, n).to(torch.bfloat16)
            seqs = torch.arange(self.B, dtype=torch.int32, device=device).repeat_interleave(self.chunk)
            lp = (self.T - 1 - self.chunk + torch.arange(self.chunk, dtype=torch.int32, device=device)).repeat(self.B)
            self.chunk_pos = lp.contiguous()
            self.chunk_slots = self.caches[0].slots(seqs, lp)            # every layer's cache has the same page table

    def _hidden(self, g, n):
        x = torch.randn((n, D_MODEL), generator=g, device=self.device, dtype=torch.float32)
        x[:, self.outliers] *= 20.0
        return x

    def step(self, events=None, scores_only=False, write=True, pre=None, post=None, chunk_events=None, chain=None, merge=True):
        """One decode step over all layers. `events`: list receiving (start, end) CUDA events around
        each attention launch (`chunk_events`: around each chunk write). `pre(l)` / `post(l)` run on the
        host before / after layer l is enqueued. `chain`: launch the attention as part of the dependent-launch
        chain (default: whenever no events sit between the kernels)."""
        n = 0
        chained = (events is None) if chain is None else chain
        for l, (pk, cache) in enumerate(zip(self.layers, self.caches)):
            ws = self.ws[l & 1]
            if pre is not None:
                pre(l)
            if self.chunk and write:
                if chunk_events is not None:
                    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    c0.record()
                pk.write_paged(cache, self.x_chunk, self.chunk_pos, self.chunk_slots)
                n += 1
                if chunk_events is not None:
                    c1.record()
                    chunk_events.append((c0, c1))
            fused = write and not self.simt and self.fused_prologue
            inline = fused and self.inline_absorb and not scores_only
            if inline:                                                # the write alone; attention absorbs the raw queries
                pk.prologue_step(cache, self.x_new[l], self.wpos, self.wslots[l], None, None, ws, v=self.v_new[l])
                n += 1
            elif fused:                                               # newest token's write + absorb: one launch
                pk.prologue_step(cache, self.x_new[l], self.wpos, self.wslots[l], self.q[l], self.qpos, ws, v=self.v_new[l],
                                 signal=self.polled and chained and not self.simt)
                n += 1
            else:
                if write:
                    pk.write_paged(cache, self.x_new[l], self.wpos, self.wslots[l], v=self.v_new[l], scratch=ws.wscratch)
                    n += 2
                pk.absorb_step(self.q[l], self.qpos, ws, operand=not self.simt, signal=self.polled_absorb and chained and not self.simt)
                n += 1
            if events is not None:
                e0 = torch.cuda.Event(enable_timing=True)
                e1 = torch.cuda.Event(enable_timing=True)
                e0.record()
            if inline:
                # the queries of the step exist before the layer's first launch: attention starts with the write,
                # streams pages and absorbs at once, and waits for the write only before the page being written
                pk.attend_q_step(cache, self.q[l], self.qpos, ws, early=chained, tail_written=True, query_ready=True)
            else:
                pk.attend_step(cache, ws, simt=self.simt, scores_only=scores_only, after_absorb=chained and not fused,
                               after_prologue=chained and fused,
                               polled=chained and not self.simt and (self.polled if fused else self.polled_absorb))
            if events is not None:
                e1.record()
                events.append((e0, e1))
            if merge:
                pk.merge_step(ws, out=self.out[l])
            n += 2 if merge else 1
            if post is not None:
                post(l)
        self.launches_per_layer = n // len(self.layers)
        return n

    # bytes one attention launch must move (per layer): NVFP4 codes + scales, and bf16 V
    def bytes_k(self):
        return self.B * self.T * (self.W // 2 + self.W // 16)

    def bytes_v_per_token(self):
        # bf16 rows, or per kv head 64 bytes of codes + one bf16 scale
        return self.n_kv * (66 if self.v_bits else self.d * 2)

    def bytes_full(self):
        return self.bytes_k() + self.B * self.T * self.bytes_v_per_token()


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


def capture(fn):
    """`fn` (kernel launches on the current stream) as a CUDA graph; returns its replay, or None if capture fails."""
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        return g.replay
    except Exception as e:
        sys.stderr.write("graph capture failed: %r\n" % (e,))
        torch.cuda.synchronize()
        return None


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p)), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


def profile_traffic_base():
    """DRAM bytes read per launch and the tokens of that launch, from the ncu summary kept under profiles/
    (the line `dram_bytes_read_per_launch: <bytes> for <tokens> tokens`); None if it is not there."""
    import re
    p = os.path.join(ROOT, "profiles", "pkv_attn_tc__cfg2_b16_t8192.md")
    try:
        m = re.search(r"dram_bytes_read_per_launch:\s*([0-9.e+]+)\s*for\s*(\d+)\s*tokens", open(p).read())
        return (float(m.group(1)), int(m.group(2))) if m else None
    except OSError:
        return None


def read_probe_gbs(device, n_bytes=2 << 30, reps=5):
    """Bandwidth of the library's plain read-only stream kernel over a buffer far larger than L2."""
    from phasorkv_b200 import _lib
    lib = _lib.load()
    buf = torch.empty(n_bytes, dtype=torch.uint8, device=device)
    buf.random_(0, 255)
    sink = torch.zeros(1, dtype=torch.int32, device=device)
    best = 0.0
    for i in range(reps + 2):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        _lib.check(lib.pkv_read_probe(_lib.ptr(buf), n_bytes, _lib.ptr(sink), _lib.current_stream()), "pkv_read_probe")
        e1.record()
        torch.cuda.synchronize()
        if i >= 2:
            best = max(best, n_bytes / (e0.elapsed_time(e1) * 1e-3) / 1e9)
    del buf
    return round(best, 1)


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

    sharded_headline = args.workload == "cfg4"          # the token-sharded step is the line; its pools are cfg2's
    st = Stack("cfg2" if sharded_headline else args.workload, args.layers, device, args.algo, seed=1234 + rank,
               batch=args.batch, context=args.context, n_split=args.splits, chunk_write=not args.no_chunk_write,
               v_bits={"bf16": 0, "q3": 3, "q2": 2}[args.v_format])
    torch.cuda.synchronize()
    pk, src = peaks()
    L = args.layers
    if sharded_headline:
        sampler = ClockSampler(local)
        sampler.start()
        sh = run_sharded(st, args, dist, world, want_e2e=True)
        clocks = sampler.stop()
        line = {
            "metric": "decode tokens/s (token-sharded B=4, T=131072, %d layers)" % L,
            "value": sh["value"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": sh["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "nvfp4 latent (e2m1 x ue4m3) x nvfp4 query, fp32 accumulate; %s"
                     % ("bf16 V" if not st.v_bits else "V as per-token %d-bit codes + bf16 scale per (token, kv head)" % st.v_bits),
            "data": "synthetic",
            "config": {"workload": sh["workload"], "algo": args.algo, "parallelism": "token-sharded x%d" % world,
                       "l2": "inputs larger than L2 (%.2f GB streamed per GPU per layer)" % (sh["bytes_per_gpu_per_layer"] / 1e9)},
            "roofline": sh.pop("roofline"), "e2e": sh.pop("e2e"), "gpu_launches": sh["gpu_launches"], "clocks": clocks,
            "seq_sharded": sh,
        }
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        if rank == 0:
            print(json.dumps(line), flush=True)
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---- device-resident timing of exactly K steps
    sampler = ClockSampler(local)
    sampler.start()
    launches = {"n": 0}

    def full_step():
        launches["n"] += st.step()
    # A step is replayed as ONE CUDA graph (96 launches: the host is out of the loop, and the dependent-launch chain
    # keeps the 2-3 us between kernels that eager launches from Python lose); `--no-graph` times the eager step.
    g_full = None if (args.no_graph or args.algo != "tc") else capture(full_step)
    ms_step = timed(g_full if g_full else full_step, args.steps, args.warmup, dist)
    # ---- the same K steps once more with CUDA events around every attention launch: the per-launch
    # duration the roofline is computed from (the events sit between kernels of the chain, so this pass
    # is kept apart from the one that gives `value`)
    events, chunk_events = [], []
    ms_step_ev = timed(lambda: st.step(events=events, chunk_events=chunk_events), args.steps, 1, dist)
    clocks = sampler.stop()
    timed_events = events[-args.steps * L:]
    attn_ms = sum(a.elapsed_time(b) for a, b in timed_events) / len(timed_events)
    gpu_launches = st.launches_per_layer * L * args.steps

    # ---- K path only (logits + log-sum-exp, V never read): the "K-path us/layer" of the metric. Without the V
    # stream a layer lasts ~25 us, less than the host needs to enqueue its launches, so the K path is replayed
    # as CUDA graphs over all layers (every layer streams its own 75 MB of latent: nothing comes from L2):
    # (1) the scores-only attention launches alone; (2) the whole K path of a step -- absorb, scores-only
    # attention, log-sum-exp merge per layer -- as one dependent-launch chain. The eager figure (events around
    # each launch, cold start included) is kept beside them.
    nk = max(2, args.steps // 2)
    ev_k = []
    timed(lambda: st.step(events=ev_k, scores_only=True, write=False), nk, 2, dist)
    k_events = ev_k[-nk * L:]
    attn_k_eager_ms = sum(a.elapsed_time(b) for a, b in k_events) / len(k_events)

    def k_attention_only():
        for l, (pk_, cache) in enumerate(zip(st.layers, st.caches)):
            pk_.attend_step(cache, st.ws[l & 1], simt=st.simt, scores_only=True)
    st.step(scores_only=True, write=False)                     # operands of the last layers are in both workspaces
    k_step = lambda: st.step(scores_only=True, write=False, merge=False)       # K2 + K3: absorb, then scores + log-sum-exp per split
    g_attn, g_step = capture(k_attention_only), capture(k_step)
    attn_k_ms = timed(g_attn, 4 * nk, 3, dist) / L if g_attn else attn_k_eager_ms
    ms_kstep = timed(g_step, 4 * nk, 3, dist) if g_step else timed(k_step, nk, 2, dist)

    peak_read = read_probe_gbs(device) if args.algo == "tc" else None

    # ---- end to end through the host API: pinned host inputs in, outputs back, every step
    hx = torch.empty(st.x_new.shape, dtype=st.x_new.dtype).pin_memory()
    hv = torch.empty(st.v_new.shape, dtype=st.v_new.dtype).pin_memory()
    hq = torch.empty(st.q.shape, dtype=st.q.dtype).pin_memory()
    ho = torch.empty(st.out.shape, dtype=st.out.dtype).pin_memory()
    hx.copy_(st.x_new); hv.copy_(st.v_new); hq.copy_(st.q)
    hc = None
    if st.chunk:                                        # the chunk's hidden states come from the host as well
        hc = torch.empty(st.x_chunk.shape, dtype=st.x_chunk.dtype).pin_memory()
        hc.copy_(st.x_chunk)

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
            if hc is not None:
                st.x_chunk.copy_(hc, non_blocking=True)
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
    # the copies and the launches of a step replayed as one CUDA graph (three streams, joined before it ends), like `value`
    g_e2e = None if (args.no_graph or args.algo != "tc") else capture(e2e_step)
    ms_e2e = timed(g_e2e if g_e2e else e2e_step, args.steps, args.warmup, dist)
    h2d = hx.numel() * hx.element_size() + hv.numel() * hv.element_size() + hq.numel() * hq.element_size()
    if hc is not None:
        h2d += hc.numel() * hc.element_size()
    d2h = ho.numel() * ho.element_size()

    # ---- token-sharded long context (cfg4): the same pools viewed as B=4, T=131072/world per rank
    sharded = None
    if not args.no_sharded and args.workload == "cfg2" and not args.batch and not args.context and not st.v_bits:
        try:
            sharded = run_sharded(st, args, dist, world)
            sharded.pop("roofline", None)
        except Exception as e:                       # the headline line is still reported
            sys.stderr.write("token-sharded run failed: %r\n" % (e,))
            sharded = {"workload": "cfg4", "error": repr(e)[:300]}

    # DRAM traffic per launch: the reads of an ncu capture of this kernel on a smaller case of the same
    # shape (kept under profiles/) scaled by the tokens streamed -- reads grow in proportion to them -- plus
    # the split partials written (B x n_split x 32 x 130 floats), which do not.
    traffic = None
    base = profile_traffic_base()
    if base and args.algo == "tc" and st.W == 256 and st.n_kv == 8 and not st.v_bits:
        traffic = int(base[0] * (st.B * st.T) / base[1] + st.B * st.n_split * 32 * 130 * 4)
    achieved = st.bytes_full() / (attn_ms * 1e-3) / 1e9
    roof = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
            "frac": round(achieved / pk["hbm_gbs"], 4), "traffic": traffic, "peak_source": src,
            "kernel": "pkv_attn_%s" % args.algo, "bytes_per_launch": st.bytes_full(),
            "us_per_launch": round(attn_ms * 1e3, 2),
            "timed_over": "%d launches of a second pass of the same %d steps with CUDA events around each attention "
                          "launch (%.4f ms per step in that pass)" % (len(timed_events), args.steps, ms_step_ev)}
    if peak_read:
        roof["peak_read_gbs"] = peak_read              # a read-only stream kernel of the library, same run
        roof["frac_of_read_peak"] = round(achieved / peak_read, 4)
    v_desc = "bf16 V" if not st.v_bits else "V as per-token %d-bit codes + bf16 scale per (token, kv head)" % st.v_bits
    line = {
        "metric": "decode tokens/s (B=%d, T=%d, %d layers; K-path us/layer and HBM GB/s beside it)" % (st.B, st.T, L),
        "value": round(world * st.B / (ms_step * 1e-3), 2), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": "nvfp4 latent (e2m1 x ue4m3) x nvfp4 query, fp32 accumulate; %s" % v_desc,
        "data": "synthetic",
        "config": {"workload": "%s: %s layer shape, B=%d per GPU, T=%d, NVFP4 latent W=%d, %s %dx%d, %d layers%s"
                   % (args.workload, "7B multi-head-attention" if st.n_kv == st.n_q else "Llama-3.1-8B", st.B, st.T, st.W,
                      v_desc, st.n_kv, st.d, L, (", plus a %d-token chunk write per sequence per layer" % st.chunk) if st.chunk else ""),
                   "algo": args.algo, "n_split": st.n_split, "cuda_graph": bool(g_full), "parallelism": "batch-parallel x%d" % world,
                   "l2": "inputs larger than L2 (%.2f GB streamed per layer, %.1f GB per step)"
                         % (st.bytes_full() / 1e9, L * st.bytes_full() / 1e9)},
        "k_path_us_per_layer": round(attn_k_ms * 1e3, 2),
        "k_path_gbs": round(st.bytes_k() / (attn_k_ms * 1e-3) / 1e9, 1),
        "k_path_frac_of_hbm_peak": round(st.bytes_k() / (attn_k_ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4),
        "k_path_step_us_per_layer": round(ms_kstep * 1e3 / L, 2),
        "k_path_eager_us_per_launch": round(attn_k_eager_ms * 1e3, 2),
        "k_path_note": "k_path_us_per_layer: scores-only attention, %d layers replayed as one CUDA graph; k_path_step: absorb + "
                       "scores-only attention (logits and log-sum-exp per split) per layer as one dependent-launch chain in a CUDA graph; "
                       "eager: CUDA events around each scores-only launch enqueued from the host" % L,
        "full_us_per_layer": round(ms_step * 1e3 / L, 2),
        "hbm_gbs": round(achieved, 1),
        "roofline": roof,
        "e2e": {"value": round(world * st.B / (ms_e2e * 1e-3), 2), "unit": "tokens/s", "ms_per_step": round(ms_e2e, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "cuda_graph": bool(g_e2e)},
        "gpu_launches": gpu_launches,
        "clocks": clocks,
    }
    if st.chunk and chunk_events:
        ce = chunk_events[-args.steps * L:]
        cw_ms = sum(a.elapsed_time(b) for a, b in ce) / len(ce)
        n_tok = st.B * st.chunk
        Wp = 128 if st.W <= 128 else 256
        useful = 2.0 * n_tok * D_MODEL * st.W
        cw_bytes = n_tok * D_MODEL * 2 + n_tok * (st.W // 2 + st.W // 16) + 3 * Wp * D_MODEL * 2
        line["chunk_write"] = {
            "tokens_per_launch": n_tok, "us_per_launch": round(cw_ms * 1e3, 2),
            "tflops_useful": round(useful / (cw_ms * 1e-3) / 1e12, 1),
            "tflops_mma": round(3 * useful / (cw_ms * 1e-3) / 1e12, 1),        # the factors are three bf16 terms
            "frac_of_bf16_sustained": round(3 * useful / (cw_ms * 1e-3) / 1e12 / pk.get("bf16_tflops_sustained", pk["bf16_tflops"]), 4),
            "gbs": round(cw_bytes / (cw_ms * 1e-3) / 1e9, 1), "frac_of_hbm": round(cw_bytes / (cw_ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4),
            "kernel": "pkv_cache_write_tc (latent of the chunk; V rows are not part of PhasorKey.write)"}
    if sharded is not None:
        line["seq_sharded"] = sharded
    if rank == 0 and not args.no_cpu_baseline and world == 1:
        line["cpu_baseline"] = cpu_baseline(args.workload, budget_s=12.0)
        line["cpu_baseline_cfg1"] = cpu_baseline_cfg1(budget_s=6.0)
    sys.stdout.flush()
    os.dup2(real_stdout, 1)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_sharded(st, args, dist, world, want_e2e=False):
    """cfg4: B=4, T=131072 with the token axis split evenly over the ranks; the partial triples of a layer
    are exchanged once. Timed as one CUDA graph per step, then checked (see `check` in the result)."""
    from phasorkv_b200.sharded import ShardExchange, owner_of
    B4, T4 = 4, 131072
    Tl = T4 // world
    pages = Tl // 128
    dev = st.device
    L = args.layers
    rank = int(os.environ.get("RANK", 0))
    pt = torch.arange(B4 * pages, dtype=torch.int32, device=dev).reshape(B4, pages)
    seqlens = torch.full((B4,), Tl, dtype=torch.int32, device=dev)
    pk0 = st.layers[0]
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    n_split = max(1, min(pages, (sms * (3 if st.simt else 1)) // B4))
    ws = pk0.workspace(B4, n_split)
    gathered = torch.empty((world, B4, st.n_q, st.d + 2), dtype=torch.float32, device=dev)
    out = torch.empty((L, B4, st.n_q, st.d), dtype=torch.float32, device=dev)
    qpos = torch.full((B4,), T4, dtype=torch.int32, device=dev)
    saved = [(c.page_table, c.seqlens, c.max_pages) for c in st.caches]
    ex = None
    if world > 1 and args.collective == "p2p":
        # peer buffers in torch symmetric memory; if any rank cannot set them up, every rank takes the NCCL route
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
    owner = rank == owner_of(T4 - 1, world, T4) and not st.simt
    wpos = torch.full((B4,), T4 - 1, dtype=torch.int32, device=dev)
    wslots = (pt[:, (Tl - 1) // 128] * 128 + (Tl - 1) % 128).to(torch.int32).contiguous()
    inline = st.inline_absorb and not st.simt

    def attend(pk, cache, l, events=None, **out_kw):
        """attention of layer l on this rank's shard: raw queries absorbed in the kernel, or absorb launch + operand"""
        chained = events is None
        if inline:
            if owner:                                       # the write alone; attention waits for it before the last page only
                pk.prologue_step(cache, st.x_new[l, :B4], wpos, wslots, None, None, ws, v=st.v_new[l, :B4])
            pk.attend_q_step(cache, st.q[l, :B4], qpos, ws, early=chained, tail_written=owner, query_ready=True, **out_kw)
            return
        # polling pays behind the prologue (the attention starts while the newest token is still being written); behind
        # the small absorb launch the plain dependent launch is as fast (measured: 45.1 against 44.1 us per layer)
        sig = chained and st.polled and not st.simt and owner
        if owner:
            pk.prologue_step(cache, st.x_new[l, :B4], wpos, wslots, st.q[l, :B4], qpos, ws, v=st.v_new[l, :B4], signal=sig)
        else:
            pk.absorb_step(st.q[l, :B4], qpos, ws, operand=not st.simt, signal=sig)
        early = {} if not chained else (dict(after_prologue=True, polled=sig) if owner else dict(after_absorb=True, polled=sig))
        if events is not None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        pk.attend_step(cache, ws, simt=st.simt, **early, **out_kw)
        if events is not None:
            e1.record()
            events.append((e0, e1))

    def layer(l, route, events=None):
        pk, cache = st.layers[l], st.caches[l]
        if world == 1:
            attend(pk, cache, l, events, out=out[l])
        elif route == "p2p":
            attend(pk, cache, l, events)
            ex.run_parts(ws.partials, ws.n_split, out[l])           # local merge + peer stores + merge, one kernel
        else:
            attend(pk, cache, l, events, packed_out=ws.packed)      # local splits merged by a launch behind
            dist.all_gather_into_tensor(gathered, ws.packed)
            pk.merge_gathered(gathered, out[l])

    route = "p2p" if ex is not None else "nccl"

    def step():
        for l in range(L):
            layer(l, route)
    per_layer_launches = 2 if world == 1 else (3 if route == "p2p" else 4)
    for c in st.caches:
        c.page_table, c.seqlens, c.max_pages = pt, seqlens, pages
    graphed = False
    try:
        fn = step
        if not args.no_graph:
            # at 1/8 of the tokens per GPU a layer lasts tens of microseconds: the step is replayed as one
            # CUDA graph (kernels, exchange and all) so that the host is out of the loop, as the
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
        torch.cuda.synchronize()
        out_timed = out.clone()                                     # what the timed replays left behind
        per_gpu_bytes = B4 * Tl * (st.W // 2 + st.W // 16 + st.bytes_v_per_token())
        res = {"workload": "cfg4: B=4, T=131072, tokens split evenly over %d GPU(s), %d layers" % (world, L),
               "value": round(B4 / (ms * 1e-3), 2), "unit": "tokens/s", "ms_per_step": round(ms, 4), "n_gpus": world,
               "us_per_layer": round(ms * 1e3 / L, 2),
               "scaling": "strong", "cuda_graph": graphed, "newest_token_written_by": "rank %d (fused prologue)" % (world - 1),
               "collective": "none" if world == 1 else ("local merge + exchange + merge in one kernel over NVLink peer memory, [B,H,d+2] fp32 per layer"
                                                        if ex is not None else "NCCL all_gather of [B,H,d+2] fp32 per layer + merge"),
               "allgather_bytes_per_gpu_per_layer": B4 * st.n_q * (st.d + 2) * 4 if world > 1 else 0,
               "bytes_per_gpu_per_layer": per_gpu_bytes,
               "hbm_gbs_per_gpu": round(per_gpu_bytes * L / (ms * 1e-3) / 1e9, 1),
               "gpu_launches": per_layer_launches * L * args.steps}

        # ---- the check: nothing above looked at a result
        chk = {"status_attention": [int(v) for v in ws.status.cpu()],
               "status_exchange": [int(v) for v in ex.status.cpu()] if ex is not None else None}
        ok = not any(chk["status_attention"]) and not (chk["status_exchange"] and any(chk["status_exchange"]))

        def relerr(a, b):
            return float((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-300))
        check_layers = sorted({0, L - 1})
        if world > 1:
            # (1) the exchange routes against each other: peer-store kernel vs NCCL all-gather + merge
            other = "nccl" if route == "p2p" else ("p2p" if ex is not None else None)
            if other is not None:
                worst = 0.0
                for l in check_layers:
                    layer(l, other)
                    torch.cuda.synchronize()
                    worst = max(worst, relerr(out[l], out_timed[l]))
                chk["rel_p2p_vs_nccl"] = worst
                ok = ok and worst <= 1e-5
        if not st.simt:
            # (2) every rank forms its shard's triples with the CUDA-core kernel; gathered, merged, compared with the
            # tensor-core result of the timed step (tolerance of the attention output: 2e-3)
            ws_s = pk0.workspace(B4, max(1, min(pages, (sms * 3) // B4)))
            worst = 0.0
            # (quantised V pages are read by the tensor-core kernel only: the second opinion is then that kernel with
            # another number of token splits, i.e. other reference maxima and another merge)
            by_simt = not st.v_bits
            for l in check_layers:
                pkl, cache = st.layers[l], st.caches[l]
                pkl.absorb_step(st.q[l, :B4], qpos, ws_s, operand=not by_simt)
                o_s = torch.empty((B4, st.n_q, st.d), dtype=torch.float32, device=dev)
                if world == 1:
                    pkl.attend_step(cache, ws_s, simt=by_simt, out=o_s)
                else:
                    pkl.attend_step(cache, ws_s, simt=by_simt, packed_out=ws_s.packed)
                    dist.all_gather_into_tensor(gathered, ws_s.packed)
                    pkl.merge_gathered(gathered, o_s)
                torch.cuda.synchronize()
                worst = max(worst, relerr(out_timed[l], o_s))
            chk["rel_tc_vs_simt" if by_simt else "rel_tc_vs_other_split"] = worst
            ok = ok and worst <= 2e-3
        if dist is not None:                                        # every rank must agree that it is fine
            flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            ok = bool(int(flag.item()))
        chk["ok"] = ok
        chk["bounds"] = {"rel_p2p_vs_nccl": 1e-5, "rel_tc_vs_simt": 2e-3, "rel_tc_vs_other_split": 2e-3, "status": "all zero"}
        res["check"] = chk
        if not ok:
            res["failed"] = "correctness check of the token-sharded step failed: value withdrawn"
            res["value_unchecked"], res["value"] = res["value"], None

        # ---- roofline of the attention launch on this rank's shard, eager with events (for --workload cfg4)
        ev = []
        for _ in range(3):
            for l in range(L):
                layer(l, route, ev)
        torch.cuda.synchronize()
        sel = ev[-L:]
        a_ms = sum(a.elapsed_time(b) for a, b in sel) / len(sel)
        pk_, src = peaks()
        ach = per_gpu_bytes / (a_ms * 1e-3) / 1e9
        res["roofline"] = {"bound": "hbm", "achieved": round(ach, 1), "peak": pk_["hbm_gbs"], "unit": "GB/s",
                           "frac": round(ach / pk_["hbm_gbs"], 4), "traffic": None, "peak_source": src,
                           "kernel": "pkv_attn_%s" % args.algo, "bytes_per_launch": per_gpu_bytes,
                           "us_per_launch": round(a_ms * 1e3, 2), "timed_over": "%d launches, eager, CUDA events" % len(sel)}
        res["attention_us_per_layer"] = round(a_ms * 1e3, 2)

        if want_e2e:
            # through the host API with pinned host buffers: this step's hidden states, value rows and queries
            # in, every layer's output back, inside the timed region
            hx = torch.empty((L, B4, D_MODEL), dtype=st.x_new.dtype).pin_memory()
            hv = torch.empty((L, B4, st.n_kv * st.d), dtype=st.v_new.dtype).pin_memory()
            hq = torch.empty((L, B4, st.n_q, st.d), dtype=st.q.dtype).pin_memory()
            ho = torch.empty(out.shape, dtype=out.dtype).pin_memory()
            hx.copy_(st.x_new[:, :B4]); hv.copy_(st.v_new[:, :B4]); hq.copy_(st.q[:, :B4])

            def e2e_step():
                st.x_new[:, :B4].copy_(hx, non_blocking=True)
                st.v_new[:, :B4].copy_(hv, non_blocking=True)
                st.q[:, :B4].copy_(hq, non_blocking=True)
                fn()
                ho.copy_(out, non_blocking=True)
            ms_e = timed(e2e_step, args.steps, args.warmup, dist)
            res["e2e"] = {"value": round(B4 / (ms_e * 1e-3), 2), "unit": "tokens/s", "ms_per_step": round(ms_e, 4),
                          "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in (hx, hv, hq)),
                          "d2h_bytes_per_step": ho.numel() * ho.element_size()}
    finally:
        for c, s_ in zip(st.caches, saved):
            c.page_table, c.seqlens, c.max_pages = s_
    return res


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


def cpu_baseline_cfg1(budget_s: float = 6.0) -> dict:
    """BASELINE configuration 1 in full on the host cores, nothing scaled: one layer, B=1, T=4096, fp32 latent
    without quantisation -- PhasorKey.write of the whole context, then absorb + scores + softmax + P.V of one
    decode step at position 4096 (phasorkv/latent.py:61-88 through the oracle port)."""
    from oracle import phasor_oracle as po
    from phasorkv_b200 import synth
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    T = synth.CONFIGS["cfg1"]["context"]
    spec = synth.make_layer("cfg1", 0)
    pk = po.PhasorKeyOracle.from_spec(spec)
    gen = torch.Generator().manual_seed(101)
    x = synth.make_hidden(gen, T)
    V = synth.make_values(gen, T, spec.n_kv, spec.head_dim)
    q = synth.make_query(gen, 1, spec.n_q, spec.head_dim)[0]
    ph_k = po.rope_phasors(spec.inv_freq, torch.arange(T))
    ph_q = po.rope_phasors(spec.inv_freq, torch.tensor([T]))

    def unit():
        t0 = time.perf_counter()
        rows = pk.write(x, ph_k)
        t1 = time.perf_counter()
        po.decode_step(pk, q, ph_q, rows, V, spec.head_dim)
        return t1 - t0, time.perf_counter() - t1
    unit(); unit()
    tw, td = [], []
    t_end = time.perf_counter() + budget_s
    while len(tw) < 5 or (time.perf_counter() < t_end and len(tw) < 200):
        a, b = unit()
        tw.append(a); td.append(b)
    tw.sort(); td.sort()
    w_ms, d_ms = tw[len(tw) // 2] * 1e3, td[len(td) // 2] * 1e3
    return {"write_ms": round(w_ms, 3), "decode_ms": round(d_ms, 3), "value": round(1.0 / (d_ms * 1e-3), 2),
            "unit": "tokens/s (one layer, B=1)", "cores": cores, "kind": "port",
            "sample": "cfg1 in full, median of %d runs: write of T=%d tokens %.2f ms; one decode step (absorb + scores + "
                      "softmax + P.V, fp32, no quantisation) %.2f ms; nothing scaled" % (len(tw), T, w_ms, d_ms)}


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
