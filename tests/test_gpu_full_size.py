"""The benchmark configurations at their full sizes, checked through properties that do not need the
CPU oracle on all of the data: invariance under the number of token splits, agreement of the two
attention kernels, token-sharded merge == unsharded, bit-exact re-quantisation of the stored rows, and
one sequence compared with the oracle on the dequantised cache (logits 1e-3, outputs 2e-3)."""
import pytest
import torch

from oracle import phasor_oracle as po
from phasorkv_b200 import synth
from phasorkv_b200.latent import PhasorKey

from helpers import rel

pytestmark = pytest.mark.gpu

#            config  batch  context  tensor-core kernel (cfg5: one query head per kv head, 4 head-group CTAs)
CASES = [("cfg2", 16, 32768, True), ("cfg3", 32, 16384, True), ("cfg4", 4, 131072, True), ("cfg5", 8, 32768, True)]


def _fill(pk, cache, B, T, gen):
    n_out = max(1, round(0.01 * pk.d_model))
    ch = torch.randperm(pk.d_model, generator=gen, device="cuda")[:n_out]
    chunk = 16384
    for b in range(B):
        for t0 in range(0, T, chunk):
            n = min(chunk, T - t0)
            x = torch.randn((n, pk.d_model), generator=gen, device="cuda")
            x[:, ch] *= 20.0
            lp = torch.arange(t0, t0 + n, dtype=torch.int32, device="cuda")
            slots = cache.slots(torch.full((n,), b, dtype=torch.int32, device="cuda"), lp)
            v = torch.randn((n, pk.n_kv, pk.head_dim), generator=gen, device="cuda").to(torch.bfloat16)
            pk.write_paged(cache, x.to(torch.bfloat16), lp, slots, v=v)
    cache.seqlens.fill_(T)


@pytest.mark.parametrize("config,B,T,tc", CASES)
def test_full_size_properties(config, B, T, tc):
    spec = synth.make_layer(config, 0, factor_gain=64.0)              # peaked softmax: rescaling is exercised
    pk = PhasorKey.from_spec(spec)
    gen = torch.Generator(device="cuda").manual_seed(77)
    xc = torch.randn((2048, pk.d_model), generator=gen, device="cuda")
    rows = torch.empty((2048, pk.cache_width), device="cuda")
    pk.write_paged(None, xc, torch.arange(2048, dtype=torch.int32, device="cuda"), None, latent_out=rows)
    second = pk.calibrate_second(rows)
    cache = pk.new_cache(B, T)
    _fill(pk, cache, B, T, gen)
    q = torch.randn((B, pk.n_q, pk.head_dim), generator=gen, device="cuda")
    qpos = torch.full((B,), T, dtype=torch.int32, device="cuda")

    def run(n_split, simt, c=cache, packed=False):
        ws = pk.workspace(B, n_split)
        pk.absorb_step(q, qpos, ws, operand=not simt)
        if packed:
            pk.attend_step(c, ws, simt=simt, packed_out=ws.packed, after_absorb=True)
            return ws.packed.clone()
        pk.attend_step(c, ws, simt=simt, out=ws.out, after_absorb=True)
        torch.cuda.synchronize()
        assert int(ws.status.abs().sum()) == 0
        return ws.out.clone()

    simt_only = not tc
    base = run(pk.default_splits(B, T, simt_only), simt_only)
    assert torch.isfinite(base).all()
    # 1. the result does not depend on how the tokens are split (the tensor-core kernel rounds the softmax
    #    weights to bf16 relative to a split-dependent reference maximum: agreement to that rounding)
    for ns in (1, 7, 40):
        e = rel(run(ns, simt_only).cpu(), base.cpu())
        print(f"{config}: n_split {ns} vs default: {e:.2e}")
        assert e < (2e-3 if tc else 2e-5), ns
    # 2. the tensor-core and the CUDA-core kernels agree
    if tc:
        assert rel(run(12, True).cpu(), base.cpu()) < 2e-3
    # 3. token sharding over 8 ranks (page-table views of the same pools) merges to the same result
    G, P = 8, cache.max_pages
    gathered = torch.empty((G, B, pk.n_q, pk.head_dim + 2), device="cuda")
    full_pt, full_len, full_mp = cache.page_table, cache.seqlens, cache.max_pages
    for r in range(G):
        cache.page_table = full_pt[:, r * P // G:(r + 1) * P // G].contiguous()
        cache.max_pages = P // G
        cache.seqlens = torch.full((B,), T // G, dtype=torch.int32, device="cuda")
        gathered[r] = run(5, simt_only, packed=True)
    cache.page_table, cache.seqlens, cache.max_pages = full_pt, full_len, full_mp
    out = torch.empty_like(base)
    pk.merge_gathered(gathered, out)
    e = rel(out.cpu(), base.cpu())
    print(f"{config}: 8 token shards vs one: {e:.2e}")
    assert e < (2e-3 if tc else 2e-5)
    # 4. what is stored re-quantises to itself bit for bit (idempotence of the NVFP4 quantiser)
    b = B - 1
    lp = torch.arange(T, dtype=torch.int32, device="cuda")
    slots = cache.slots(torch.full((T,), b, dtype=torch.int32, device="cuda"), lp)
    deq, codes, scales = cache.read(slots, second)
    again = pk.new_cache(1, T, with_v=False)
    s2 = again.slots(torch.zeros_like(lp), lp)
    again.quantize_rows(deq, s2, second)
    deq2, codes2, scales2 = again.read(s2, second)
    assert torch.equal(deq2, deq)
    live = scales.repeat_interleave(8, dim=1) != 0                      # codes of a zero-scale block carry no information
    assert torch.equal(codes2[live], codes[live]) and torch.equal(scales2, scales)
    # 5. one whole sequence against the oracle on the dequantised cache
    opk = po.PhasorKeyOracle.from_spec(spec)
    ph = po.rope_phasors(spec.inv_freq, qpos[b:b + 1].cpu(), spec.attn_scale)
    qa = opk.absorb(q[b].cpu()[:, None, :], ph)[:, 0]
    S_ref = opk.scores(qa, deq.cpu())
    O_ref = po.attend(S_ref, cache.v_rows(slots).cpu(), spec.n_kv, spec.head_dim)
    ws = pk.workspace(B, 9)
    S = torch.zeros((B, pk.n_q, T), device="cuda")
    pk.absorb_step(q, qpos, ws, operand=not simt_only)
    pk.attend_step(cache, ws, simt=simt_only, scores_out=S, out=ws.out)
    es, eo = rel(S[b].cpu(), S_ref), rel(ws.out[b].cpu(), O_ref)
    print(f"{config}: sequence {b} against the oracle: logits {es:.2e}, outputs {eo:.2e}")
    assert es < 1e-3 and eo < 2e-3


@pytest.mark.parametrize("config,B,T,bits", [("cfg2", 16, 32768, 3), ("cfg5", 8, 32768, 2)])
def test_full_size_quantised_v(config, B, T, bits):
    """The same sizes with V stored as per-token low-bit codes: split invariance, and one whole sequence against
    the oracle's softmax . V on the dequantised value rows (2e-3)."""
    spec = synth.make_layer(config, 0, factor_gain=64.0)
    pk = PhasorKey.from_spec(spec)
    gen = torch.Generator(device="cuda").manual_seed(78)
    xc = torch.randn((2048, pk.d_model), generator=gen, device="cuda")
    rows = torch.empty((2048, pk.cache_width), device="cuda")
    pk.write_paged(None, xc, torch.arange(2048, dtype=torch.int32, device="cuda"), None, latent_out=rows)
    second = pk.calibrate_second(rows)
    cache = pk.new_cache(B, T, v_bits=bits)
    _fill(pk, cache, B, T, gen)
    q = torch.randn((B, pk.n_q, pk.head_dim), generator=gen, device="cuda")
    qpos = torch.full((B,), T, dtype=torch.int32, device="cuda")

    def run(n_split):
        ws = pk.workspace(B, n_split)
        pk.absorb_step(q, qpos, ws)
        pk.attend_step(cache, ws, out=ws.out, after_absorb=True)
        torch.cuda.synchronize()
        assert int(ws.status.abs().sum()) == 0
        return ws.out.clone()

    base = run(pk.default_splits(B, T))
    assert torch.isfinite(base).all()
    for ns in (1, 7, 40):
        e = rel(run(ns).cpu(), base.cpu())
        print(f"{config} q{bits}: n_split {ns} vs default: {e:.2e}")
        assert e < 2e-3, ns
    b = B - 1
    lp = torch.arange(T, dtype=torch.int32, device="cuda")
    slots = cache.slots(torch.full((T,), b, dtype=torch.int32, device="cuda"), lp)
    deq, _, _ = cache.read(slots, second)
    v_hat, _, _ = cache.read_vq(slots)
    opk = po.PhasorKeyOracle.from_spec(spec)
    ph = po.rope_phasors(spec.inv_freq, qpos[b:b + 1].cpu(), spec.attn_scale)
    qa = opk.absorb(q[b].cpu()[:, None, :], ph)[:, 0]
    O_ref = po.attend(opk.scores(qa, deq.cpu()), v_hat.cpu(), spec.n_kv, spec.head_dim)
    eo = rel(base[b].cpu(), O_ref)
    print(f"{config} q{bits}: sequence {b} against the oracle: outputs {eo:.2e}")
    assert eo < 2e-3
