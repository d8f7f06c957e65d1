"""Decode-attention benchmark over context lengths and batch sizes, with the result file of the
reference's own kernel benchmark so that the numbers line up with its runs.

The reference times its latent kernels per decode step over all layers of the model as one CUDA
graph, on random factors and random caches far larger than the L2, and stores
``results[f"{name}|T{T}|B{B}|{kernel options}"] = dict(ms, kernel_ms, gbs, tflops)``
(scripts/bench_decode.py:29-49,112-160); the per-layer shapes it benchmarks come from a
``kernel_shapes.json`` written by scripts/kernel_shapes.py:21-63. This module does both for the
PhasorKey path of this package:

  python -m phasorkv_b200.bench_decode --configs cfg2,cfg3 --lens 4096,16384,32768 --batches 1,8,16 \
      --out bench_decode.json --shapes-out kernel_shapes.json

* ``kernel_shapes(config, n_layers)``: per layer the rank of every RoPE frequency, R, R_s, n_slow, the
  cached width W and the V row, i.e. what fixes the kernels' shapes and the bytes per token.
* one timed configuration = query absorption + split-T attention on the NVFP4 latent and bf16 V + the
  split merge for every layer, captured as one CUDA graph; ``gbs`` = cache bytes streamed per second,
  ``tflops`` = the scoring and P.V contractions (2*H_q*W + 2*H_q*d flop per token and layer).
* ``--dense`` adds torch's bf16 SDPA on a dense GQA cache as the comparison row ``sdpa-bf16|T..|B..``
  (a library kernel: a yardstick, not part of the path).
A key that is already in the output file is skipped, so an interrupted sweep resumes.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import Dict, List, Optional

from . import synth

N_LAYERS = 32


def kernel_shapes(config: str, n_layers: int = N_LAYERS) -> dict:
    """Shapes of every layer of `config` as the kernels see them (no GPU needed)."""
    c = synth.CONFIGS[config]
    layers = {}
    for i in range(n_layers):
        spec = synth.make_layer(config, i)
        h = spec.head_dim // 2
        ranks = [int((spec.freq == j).sum()) for j in range(h)]
        layers[str(i)] = dict(ranks=ranks, R=spec.R, R_s=spec.R_s, n_slow=0 if spec.slow is None else int(spec.slow.numel()),
                              W=spec.cache_width, n_q=spec.n_q, n_kv=spec.n_kv, head_dim=spec.head_dim,
                              latent="nvfp4", v="bf16")
    return dict(layout=c["layout"], rope_base=c["base"], layers=layers)


def bytes_per_token(shape: dict) -> int:
    """Cache bytes per token over all layers: NVFP4 codes + E4M3 block scales of the padded width, bf16 V."""
    n = 0
    for l in shape["layers"].values():
        wp = 128 if l["W"] <= 128 else 256
        n += wp // 2 + wp // 16 + l["n_kv"] * l["head_dim"] * 2
    return n


def flops_per_token(shape: dict) -> int:
    return sum(2 * l["n_q"] * l["W"] + 2 * l["n_q"] * l["head_dim"] for l in shape["layers"].values())


def result_key(name: str, T: int, B: int, opts: Dict[str, object]) -> str:
    return f"{name}|T{T}|B{B}|" + ",".join(f"{k}={v}" for k, v in opts.items())


class StepGraph:
    """A decode step captured once as a CUDA graph, replayed for timing: the host is out of the loop, which
    is how the reference times its kernels too (one graph over all layers, scripts/bench_decode.py:29-49)."""

    def __init__(self, step_fn, eager_calls: int = 2):
        import torch
        self._torch = torch
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(eager_calls):                # lazy initialisation happens outside the capture
                step_fn()
        side.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=side):
            step_fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()

    def median_ms(self, replays: int = 20, rounds: int = 5) -> float:
        """Median over `rounds` event pairs, each around replays / rounds back-to-back replays."""
        torch = self._torch
        per = max(1, replays // rounds)
        self.graph.replay()
        self.graph.replay()
        pairs = []
        for _ in range(rounds):
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(per):
                self.graph.replay()
            t1.record()
            pairs.append((t0, t1))
        torch.cuda.synchronize()
        ms = sorted(a.elapsed_time(b) / per for a, b in pairs)
        return ms[len(ms) // 2]


def bench_latent(config: str, n_layers: int, B: int, T: int, algo: str, n_split: int = 0, iters: int = 20):
    """-> (ms per step over all layers, options used). Random cache contents: timing does not depend on them."""
    import torch
    from .latent import PhasorKey
    dev = torch.device("cuda")
    simt = algo == "simt"
    pks = [PhasorKey.from_spec(synth.make_layer(config, l), device=dev) for l in range(n_layers)]
    caches = []
    for pk in pks:
        pk.set_second(0.01)
        c = pk.new_cache(B, T)
        c.latent.random_(0, 120)                       # any code; scale bytes stay finite E4M3
        c.v.normal_()
        c.seqlens.fill_(T)
        caches.append(c)
    ns = n_split or pks[0].default_splits(B, T, simt)
    ws = [pks[0].workspace(B, ns) for _ in range(2)]
    q = torch.randn((n_layers, B, pks[0].n_q, pks[0].head_dim), device=dev)
    pos = torch.full((B,), T, dtype=torch.int32, device=dev)
    outs = torch.empty((n_layers, B, pks[0].n_q, pks[0].head_dim), device=dev)

    def step():
        for l, (pk, c) in enumerate(zip(pks, caches)):
            w = ws[l & 1]
            pk.absorb_step(q[l], pos, w, operand=not simt)
            pk.attend_step(c, w, simt=simt, out=outs[l], after_absorb=True)
    ms = StepGraph(step).median_ms(replays=iters)
    assert all(int(w.status.abs().sum()) == 0 for w in ws), "a kernel reported a give-up"
    del caches
    torch.cuda.empty_cache()
    return ms, dict(algo=algo, n_split=ns)


def dense_sdpa_ms(B: int, T: int, n_layers: int, n_q: int, n_kv: int, d: int, budget_bytes: float) -> Optional[float]:
    """Yardstick: torch's bf16 scaled-dot-product attention (a library kernel) decoding over a dense grouped-query
    cache of the same shape. One allocation holds as many layers as the budget allows; the time is scaled to
    the full depth. None when not even one layer fits or the backend refuses the call."""
    import torch
    layer_bytes = 2 * 2 * B * T * n_kv * d                 # keys and values, two bytes each
    fit = min(n_layers, int(budget_bytes // layer_bytes))
    if fit <= 0:
        return None
    dense = torch.empty((fit, 2, B, n_kv, T, d), dtype=torch.bfloat16, device="cuda").normal_()
    query = torch.empty((B, n_q, 1, d), dtype=torch.bfloat16, device="cuda").normal_()

    def step():
        for layer in dense:
            torch.nn.functional.scaled_dot_product_attention(query, layer[0], layer[1], enable_gqa=True)
    ms = None
    try:
        ms = StepGraph(step).median_ms() * n_layers / fit
    except RuntimeError as err:
        print(f"  dense SDPA yardstick skipped ({type(err).__name__}: {str(err)[:100]})", flush=True)
    del dense
    torch.cuda.empty_cache()
    return ms


def parse_args(argv: Optional[List[str]] = None) -> argparse.Namespace:
    p = argparse.ArgumentParser(prog="python -m phasorkv_b200.bench_decode", description=__doc__.split("\n\n")[0])
    p.add_argument("--configs", default="cfg2", help="comma-separated names from phasorkv_b200.synth.CONFIGS")
    p.add_argument("--lens", default="4096,16384,32768,65536")
    p.add_argument("--batches", default="1,8,32")
    p.add_argument("--layers", type=int, default=N_LAYERS)
    p.add_argument("--algo", default="tc", choices=["tc", "simt"])
    p.add_argument("--splits", type=int, default=0, help="token splits per sequence (default: fill the GPU once)")
    p.add_argument("--budget-gb", type=float, default=70.0, help="cache memory the benchmark may use")
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--dense", action="store_true", help="also time torch's bf16 SDPA on a dense cache")
    p.add_argument("--out", default="bench_decode.json")
    p.add_argument("--shapes-out", default="kernel_shapes.json")
    p.add_argument("--shapes-only", action="store_true", help="write the shapes file and stop (no GPU needed)")
    return p.parse_args(argv)


def main(argv: Optional[List[str]] = None) -> int:
    args = parse_args(argv)
    names = [c for c in args.configs.split(",") if c]
    for n in names:
        if n not in synth.CONFIGS:
            raise SystemExit(f"unknown config {n!r}; known: {', '.join(synth.CONFIGS)}")
    shapes = json.load(open(args.shapes_out)) if os.path.exists(args.shapes_out) else {}
    for n in names:
        shapes[n] = kernel_shapes(n, args.layers)
    json.dump(shapes, open(args.shapes_out, "w"), indent=1)
    if args.shapes_only:
        print("wrote", args.shapes_out)
        return 0
    import torch
    torch.set_grad_enabled(False)
    if not torch.cuda.is_available():
        raise SystemExit("bench_decode needs a CUDA device: this package has no CPU path")
    res = json.load(open(args.out)) if os.path.exists(args.out) else {}
    lens = [int(x) for x in args.lens.split(",")]
    batches = [int(x) for x in args.batches.split(",")]
    budget = args.budget_gb * 2 ** 30
    print(torch.cuda.get_device_name(), "algo", args.algo, flush=True)
    for name in names:
        shape = shapes[name]
        bpt, flops = bytes_per_token(shape), flops_per_token(shape)
        l0 = shape["layers"]["0"]
        # the tensor-core attention kernel takes 1, 4 or 8 query heads per kv head; other groupings run the CUDA-core kernel
        rep = l0["n_q"] // l0["n_kv"]
        algo = args.algo if rep in (1, 4, 8) else "simt"
        groups = 4 if (rep == 1 and algo == "tc") else 1       # one query head per kv head: 4 CTAs per (sequence, split)
        print(f"{name}: {bpt / 1024:.1f} KiB/token (NVFP4 latent + bf16 V, {args.layers} layers), "
              f"{flops / 1e6:.2f} MFLOP/token", flush=True)
        for T in lens:
            for B in batches:
                if B * T * bpt > budget:
                    print(f"  T={T} B={B}: over budget", flush=True)
                    continue
                ns = args.splits
                if not ns:                                # the key must be known before the run: same rule as default_splits
                    sms = torch.cuda.get_device_properties(0).multi_processor_count
                    ns = max(1, min((T + 127) // 128, (sms * (3 if algo == "simt" else 1)) // (B * groups)))
                key = result_key(name, T, B, dict(algo=algo, n_split=ns))
                if key in res:
                    continue
                t0 = time.time()
                ms, _ = bench_latent(name, args.layers, B, T, algo, ns, args.iters)
                res[key] = dict(ms=ms, kernel_ms=ms, gbs=B * T * bpt / (ms * 1e-3) / 1e9,
                                tflops=B * T * flops / (ms * 1e-3) / 1e12)
                print(f"  T={T:6d} B={B:3d}: {ms:8.3f} ms/step  {res[key]['gbs']:6.0f} GB/s  "
                      f"{res[key]['tflops']:6.1f} TFLOP/s  [{time.time() - t0:.0f}s]", flush=True)
                json.dump(res, open(args.out, "w"), indent=1)
        if args.dense:
            for T in lens:
                for B in batches:
                    key = f"sdpa-bf16|T{T}|B{B}"
                    if key in res:
                        continue
                    t = dense_sdpa_ms(B, T, args.layers, l0["n_q"], l0["n_kv"], l0["head_dim"], budget)
                    if t is None:
                        continue
                    dense_bpt = args.layers * 2 * l0["n_kv"] * l0["head_dim"] * 2
                    res[key] = dict(ms=t, gbs=B * T * dense_bpt / (t * 1e-3) / 1e9)
                    print(f"  sdpa-bf16 T={T:6d} B={B:3d}: {t:8.3f} ms/step  {res[key]['gbs']:6.0f} GB/s", flush=True)
                    json.dump(res, open(args.out, "w"), indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
