"""Host-side logic that needs no GPU: the library loads and exports the declared ABI, the layout
index maps are consistent, the PhasorKey constructor matches the reference's attribute arrays,
and the patch protocol behaves like the reference's patch objects."""
import ctypes
import os
import re
import types

import numpy as np
import pytest
import torch

from phasorkv_b200 import _lib, build, synth
from phasorkv_b200.latent import PhasorKey
from phasorkv_b200.patch import PhasorKeyPatch

from conftest import GOLDEN, ROOT
from helpers import Blk as _Blk, fac_from_golden as _fac_from_golden


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def test_library_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "phasorkv_b200.h")).read()
    declared = set(re.findall(r"\b(pkv_[a-z0-9_]+)\s*\(", header))
    declared -= {"pkv_status"}
    assert declared, "no declarations found"
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert declared == set(_lib.SIGNATURES), "ctypes table and header disagree"
    assert lib.pkv_abi_version() == 2          # 2: pkv_cache_t grew vq_dev, v_bits


def test_sizes_and_status_strings(lib):
    assert lib.pkv_latent_page_bytes(256) == 128 * 128 + 4 * 512
    assert lib.pkv_latent_page_bytes(128) == 128 * 64 + 2 * 512
    assert lib.pkv_latent_page_bytes(240) == lib.pkv_latent_page_bytes(256)
    assert lib.pkv_latent_page_bytes(272) == -2 and lib.pkv_latent_page_bytes(100) == -2
    assert lib.pkv_v_page_bytes(8, 128) == 128 * 8 * 128 * 2
    assert lib.pkv_query_operand_bytes(256) == 18432 + 512
    assert lib.pkv_query_operand_bytes(128) == 9216 + 512
    assert lib.pkv_status_string(0) == b"ok" and lib.pkv_status_string(-2) == b"unsupported shape"


def test_argument_checks_without_a_device(lib):
    """Invalid arguments are rejected before any CUDA call is made."""
    assert lib.pkv_quantize_rows(None, None, None, 0, ctypes.c_float(1.0), None) == -1
    c = _lib.Cache(4096, 0, 1, 300, 8, 128)
    assert lib.pkv_quantize_rows(ctypes.byref(c), 1024, 1024, 1, ctypes.c_float(1.0), None) == -2   # W = 300
    c = _lib.Cache(4096 + 8, 0, 1, 256, 8, 128)
    assert lib.pkv_quantize_rows(ctypes.byref(c), 1024, 1024, 1, ctypes.c_float(1.0), None) == -1   # misaligned pool
    assert lib.pkv_merge(None, 0, 0, 1, 1, 32, 128, None, None, None) == -1


def test_synth_layers_have_benchmark_shapes():
    s2 = synth.make_layer("cfg2", 0)
    assert (s2.R, s2.R_s, s2.cache_width, s2.n_kv) == (128, 0, 256, 8)
    s3 = synth.make_layer("cfg3", 0)
    assert (s3.R, s3.R_s, s3.cache_width) == (120, 16, 256)
    counts = torch.bincount(s3.freq, minlength=64)
    assert counts[:56].max() <= 6 and counts[56:].sum() == 0 and list(s3.slow) == list(range(56, 64))
    s5 = synth.make_layer("cfg5", 3)
    assert (s5.R, s5.cache_width, s5.n_kv) == (64, 128, 32)
    assert abs(float(s5.inv_freq[1]) - 10000.0 ** (-2 / 128)) < 1e-15
    again = synth.make_layer("cfg3", 0)
    assert torch.equal(again.A, s3.A) and torch.equal(again.B_s, s3.B_s)
    assert not torch.equal(synth.make_layer("cfg2", 1).B, s2.B)


@pytest.mark.parametrize("tag", ["freq", "band"])
def test_constructor_matches_reference_attribute_arrays(tag):
    """PhasorKey(fac, ranks, n_q) fed with the block data of a reference Factorization (eigenvectors,
    energies, row weights, weighted rows; stored in the golden file) reproduces the arrays the
    reference's own constructor built from them: A, B, freq, energy, slow, A_s, B_s."""
    g = np.load(os.path.join(GOLDEN, "phasorkey_factorized.npz"))
    fac, n_q = _fac_from_golden(g, tag)
    pk = PhasorKey(fac, g[f"{tag}_ranks"].tolist(), n_q, inv_freq=torch.from_numpy(g["inv_freq"]), device="cpu")
    assert torch.equal(pk.freq, torch.from_numpy(g[f"{tag}_freq"]))
    for name in ("A", "B", "energy"):
        ref = torch.from_numpy(g[f"{tag}_{name}"])
        assert torch.allclose(getattr(pk, name), ref, rtol=1e-13, atol=1e-15), name
    assert torch.equal(pk.slow, torch.from_numpy(g[f"{tag}_slow"]))
    assert pk.cache_width == g[f"{tag}_rows"].shape[1]
    if f"{tag}_A_s" in g:
        assert torch.allclose(pk.A_s, torch.from_numpy(g[f"{tag}_A_s"]), rtol=1e-13, atol=1e-15)
        assert torch.allclose(pk.B_s, torch.from_numpy(g[f"{tag}_B_s"]), rtol=1e-13, atol=1e-15)
    else:
        assert pk.A_s is None and pk.R_s == 0


def test_constructor_orders_latent_dims_by_energy():
    gen = torch.Generator().manual_seed(3)
    n_kv, D, h = 2, 12, 4
    blocks, ranks = [], [2, 0, 1, 2]
    for j in range(h):
        U, _ = torch.linalg.qr(torch.complex(torch.randn(n_kv, n_kv, generator=gen), torch.randn(n_kv, n_kv, generator=gen)))
        blocks.append(_Blk(U=U, s2=torch.tensor([3.0 - j * 0.5, 1.0 + j]), sq=torch.rand(n_kv, generator=gen) + 0.5,
                           Mw=torch.complex(torch.randn(n_kv, D, generator=gen), torch.randn(n_kv, D, generator=gen)),
                           where=j, cost=2))
    fac = types.SimpleNamespace(blocks=blocks, n_kv=n_kv, d=2 * h, absorbed=True, nope=torch.zeros(h, dtype=torch.bool))
    pk = PhasorKey(fac, ranks, 4, inv_freq=torch.ones(h, dtype=torch.float64), device="cpu")
    assert pk.R == 5 and pk.cache_width == 10 and pk.R_s == 0
    assert list(pk.energy) == sorted(pk.energy.tolist(), reverse=True)
    assert pk.freq.tolist() == [3, 0, 2, 3, 0]
    assert torch.allclose(pk.A[:, 0], blocks[3].U[:, 1] / blocks[3].sq)
    assert torch.allclose(pk.B[0], blocks[3].U[:, 1].conj() @ blocks[3].Mw)


def test_patch_protocol_install_and_undo():
    spec = synth.make_layer("cfg2", 0, d_model=64)
    layer = types.SimpleNamespace(self_attn=types.SimpleNamespace())
    p = PhasorKeyPatch()
    undo = p.patch(5, layer, spec, spec.n_kv, spec.head_dim, spec.n_q, "cpu")
    assert p.name == "phasor.nvfp4"
    assert layer.self_attn.phasor_key.cache_width == 256 and layer.self_attn.phasor_layer == 5
    assert p.layer_stats[5]["bits_k"] == 4.5 * 256 and p.layer_stats[5]["bits_v"] == 16.0 * 8 * 128
    undo()
    assert not hasattr(layer.self_attn, "phasor_key")
    with pytest.raises(ValueError):
        p.patch(6, layer, spec, 4, spec.head_dim, spec.n_q, "cpu")


def test_no_cpu_path():
    """Without a GPU the product path refuses to run instead of falling back."""
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    spec = synth.make_layer("cfg2", 0, d_model=64)
    pk = PhasorKey.from_spec(spec, device="cpu")
    with pytest.raises(_lib.PhasorKVError):
        pk.write(torch.zeros(2, 64), torch.ones(2, 64, dtype=torch.complex64))


def test_bench_decode_shapes_and_result_keys(tmp_path):
    """The decode-benchmark CLI: per-layer shapes export (no GPU) and the reference's result-key form
    `name|T..|B..|options` (scripts/bench_decode.py:141)."""
    import json
    from phasorkv_b200 import bench_decode as bd
    shapes = bd.kernel_shapes("cfg3", 2)
    l0 = shapes["layers"]["0"]
    assert l0["R"] == 120 and l0["R_s"] == 16 and l0["n_slow"] == 8 and l0["W"] == 256
    assert sum(l0["ranks"]) == 120 and len(l0["ranks"]) == 64 and l0["ranks"][-8:] == [0] * 8
    s2 = bd.kernel_shapes("cfg2", 32)
    assert bd.bytes_per_token(s2) == 32 * (144 + 2048)                   # per token: 144 B latent + 2048 B V per layer
    assert bd.flops_per_token(s2) == 32 * (16384 + 8192)
    s5 = bd.kernel_shapes("cfg5", 1)
    assert bd.bytes_per_token(s5) == 72 + 8192
    assert bd.result_key("cfg2", 4096, 8, dict(algo="tc", n_split=18)) == "cfg2|T4096|B8|algo=tc,n_split=18"
    out = tmp_path / "shapes.json"
    assert bd.main(["--configs", "cfg2,cfg5", "--layers", "2", "--shapes-only", "--shapes-out", str(out)]) == 0
    got = json.load(open(out))
    assert set(got) == {"cfg2", "cfg5"} and got["cfg5"]["layers"]["1"]["n_kv"] == 32


def test_token_sharded_merge_two_cpu_ranks_gloo():
    """world_size 2 over gloo on the CPU: each rank takes its token range (the package's sharding rule),
    computes its partial triple with the oracle, all-gathers, merges: equal to the unsharded result."""
    import socket
    import subprocess
    import sys
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, os.path.join(os.path.dirname(__file__), "gloo_worker.py")],
                                      env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=300)[0] for p in procs]
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, out[-2000:]
        assert f"rank {r}: tokens" in out


def test_token_ranges():
    from phasorkv_b200.sharded import owner_of, token_range
    for world in (1, 2, 3, 8):
        for T in (1, 7, 128, 131072):
            rs = [token_range(r, world, T) for r in range(world)]
            assert rs[0][0] == 0 and rs[-1][1] == T
            assert all(a[1] == b[0] for a, b in zip(rs, rs[1:]))
            assert max(hi - lo for lo, hi in rs) - min(hi - lo for lo, hi in rs) <= 1
            assert owner_of(T - 1, world, T) == world - 1
    with pytest.raises(ValueError):
        token_range(2, 2, 10)


def test_mean_direction_split_is_a_factor_augmentation():
    """k = A (B_perp x) + alpha * kbar (phasorkv/kvmethods.py:895-899) equals the dense keys of the PhasorKey
    that `with_mean_direction` builds: its W_hat applied to x gives W_hat(A, B_perp) x + alpha kbar, for every
    token, before any rotation (rotation then acts on both alike)."""
    from oracle import phasor_oracle as po
    g = torch.Generator().manual_seed(8)
    n_kv, d, D, n_q, r = 2, 16, 40, 4, 2
    h = d // 2
    freq = torch.arange(h).repeat_interleave(r)
    A = torch.complex(torch.randn(n_kv, h * r, generator=g, dtype=torch.float64), torch.randn(n_kv, h * r, generator=g, dtype=torch.float64))
    B = torch.complex(torch.randn(h * r, D, generator=g, dtype=torch.float64), torch.randn(h * r, D, generator=g, dtype=torch.float64))
    mu = torch.randn(D, generator=g, dtype=torch.float64) + 2.0
    kbar = torch.randn(n_kv * d, generator=g, dtype=torch.float64)
    pk = PhasorKey.with_mean_direction(A, B, freq, mu, kbar, n_q, n_kv, d, torch.ones(h, dtype=torch.float64), device="cpu")
    assert pk.R == h * r + h and pk.cache_width == 2 * (h * r + h)
    x = torch.randn(7, D, generator=g, dtype=torch.float64)
    alpha = x @ mu / mu.dot(mu)
    mu_scaled = mu / mu.dot(mu)
    B_perp = B - (B @ mu.to(B.dtype))[:, None] * mu_scaled.to(B.dtype)[None, :]
    assert float((B_perp @ mu.to(B.dtype)).abs().max()) < 1e-12                       # blind to the mean direction
    k_split = x @ po.w_hat(A, B_perp, freq, n_kv, d).T + alpha[:, None] * kbar[None, :]
    k_aug = x @ po.w_hat(pk.A, pk.B, pk.freq, n_kv, d).T
    assert torch.allclose(k_aug, k_split, rtol=1e-12, atol=1e-12)
