"""CPU-only checks around the layer-list model path: the safetensors container, the model registry's reading of a Nufusun
configuration, the host-side distance-bucket table against the oracle's formula, and the oracle's own invariants (it is
what the GPU tests compare with, so it is checked against hand-computed cases here)."""
import ctypes as C
import json
import os

import numpy as np
import pytest

from powerserve_b200 import arch, arch_synth, build, capi, safetensors
from tests import _nufusun_ref as R


@pytest.fixture(scope="module")
def lib():
    build.build()
    return capi.load_library()


def test_safetensors_round_trip(tmp_path):
    rng = np.random.default_rng(1)
    a = rng.standard_normal((5, 7)).astype(np.float32)
    idx = np.arange(6, dtype=np.int32).reshape(2, 3)
    p = str(tmp_path / "m.safetensors")
    safetensors.write_file(p, {"a": a, "idx": idx})
    f = safetensors.SafeTensorsFile(p)
    assert f["a"].ps_type == safetensors.PS_BF16 and f["a"].shape == (5, 7)
    np.testing.assert_array_equal(f["a"].to_float32(), R.bf16_round(a))
    np.testing.assert_array_equal(f["idx"].data, idx)
    assert f["a"].host_ptr % 2 == 0


def test_bf16_rounding_is_nearest_even():
    x = np.array([1.0, 1.00390625, 1.005859375, 1.01171875, -3.0e-5, 65504.0], np.float32)
    # 1 + 2^-8 is a tie between 1.0 and 1 + 2^-7: the even mantissa wins (1.0); 1 + 3 * 2^-9 rounds up to 1 + 2^-7;
    # 1 + 3 * 2^-8 is a tie between 1 + 2^-7 and 1 + 2^-6: even again (1 + 2^-6)
    got = R.bf16_round(x)
    assert got[0] == 1.0 and got[1] == 1.0 and got[2] == 1.0078125 and got[3] == 1.015625
    bits = safetensors.float32_to_bf16_bits(x)
    np.testing.assert_array_equal((bits.astype(np.uint32) << 16).view(np.float32), got)


@pytest.mark.parametrize("rows,dmax", [(32, 200.0), (16, 100.0), (8, 64.0), (10, 33.0), (9, 50.0), (4, 3.5), (64, 1000.0)])
def test_host_bucket_table_matches_formula(lib, rows, dmax):
    half = rows // 2
    prev = -1
    for n in range(0, 2200):
        b = lib.ps_cuda_host_rel_bucket(n, rows, dmax)
        assert b == R.distance_bucket(n, rows, dmax), (n, rows, dmax)
        assert 0 <= b < rows and b >= prev          # monotone, inside the table
        prev = b
        if n < half:
            assert b == n
    assert lib.ps_cuda_host_rel_bucket(int(np.ceil(dmax)) + 1, rows, dmax) == rows - 1


def test_bucket_edges_by_hand():
    # 8 rows up to distance 64: identity below 4, then 4 logarithmic rows over [4, 64): edges at 4 * 16^(k/4) = 4, 8, 16, 32
    expect = {0: 0, 3: 3, 4: 4, 7: 4, 8: 5, 15: 5, 16: 6, 31: 6, 32: 7, 63: 7, 64: 7, 500: 7}
    for n, b in expect.items():
        assert R.distance_bucket(n, 8, 64.0) == b, n


def test_registry_reads_every_size_from_the_configuration(tmp_path):
    layers = [arch_synth.nufusun_layer(6, 3, 24, 20, bias_max=40.0, experts=5, top=2, ff=48, limit=0.75),
              arch_synth.nufusun_layer(4, 4, 16, 8, scale=0.3, bias_max=9.0)]
    cfg = arch_synth.nufusun_config(72, 130, layers, eps=3e-6, embed_scale=0.25)
    t = arch_synth.nufusun_weights(cfg, seed=3, rel_rows=10)
    arch_synth.write_model_dir(str(tmp_path), cfg, t)
    f = safetensors.SafeTensorsFile(str(tmp_path / "model.safetensors"))
    descs, top = arch.ARCHITECTURES["Nufusun"][0](json.load(open(tmp_path / "config.json")), f.tensors)
    assert top == {"dim": 72, "vocab_size": 130, "norm_eps": 3e-6, "embed_scale": 0.25, "norm_unit_offset": 1}
    a, b = descs
    assert (a.n_heads, a.n_kv_heads, a.qk_dim, a.v_dim, a.rel_buckets) == (6, 3, 24, 20, 10)
    assert (a.mlp_kind, a.n_experts, a.top_k, a.expert_ff) == (capi.MLP_ROUTED, 5, 2, 48)
    assert abs(a.act_limit - 0.75) < 1e-7 and abs(a.rel_max_dist - 40.0) < 1e-6 and abs(a.act_alpha - 1.702) < 1e-6
    assert (a.route_on_input, a.route_renorm, a.sink, a.head_mix, a.head_temp, a.proj_bias) == (1, 0, 1, 1, 1, 1)
    assert b.mlp_kind == capi.MLP_NONE and abs(b.score_scale - 0.3) < 1e-7 and b.n_heads == b.n_kv_heads == 4
    names = arch.ARCHITECTURES["Nufusun"][1](cfg)
    assert names["layers"][0]["gate"][4] == "l0.mlp.e4.gate" and "router" not in names["layers"][1]
    for n in [names["embed"], names["head"], names["final_norm"]] + [v for l in names["layers"] for v in l.values() if isinstance(v, str)]:
        assert n in f


def test_unknown_architecture_is_refused(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "NoSuchDesign"}))
    with pytest.raises(capi.PsCudaError):
        arch.load_model(str(tmp_path))
    with pytest.raises(capi.PsCudaError):
        arch.load_model(str(tmp_path / "nothing-here"))


def test_layer_list_context_needs_a_device(lib):
    if lib.ps_cuda_device_count() > 0:
        pytest.skip("a CUDA device is present")
    ld = (capi.LayerDesc * 1)()
    d = capi.ArchDesc(64, 100, 1, 32, 8, 1e-5, 1.0, 1, 0, ld)
    h = C.c_void_p()
    assert lib.ps_cuda_create_arch(C.byref(h), 0, C.byref(d)) == 1      # PS_CUDA_ERR_NO_DEVICE: no CPU fallback


# ---- the oracle's mechanisms against cases small enough to do by hand
def test_oracle_sink_softmax_first_token():
    # one token, one head, q.k = 0 and no bias: the weight of the only key is e^0 / (1 + e^0) = 1/2
    w = {"q": np.zeros((2, 3)), "k": np.zeros((2, 3)), "v": np.eye(2, 3), "q.b": np.zeros(2), "k.b": np.zeros(2), "v.b": np.array([4.0, 6.0]),
         "o": np.eye(3, 2), "o.b": np.zeros(3), "rel": np.zeros((4, 1)), "talk": np.ones((1, 1)), "temp": np.ones(1)}
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 1.0, "bias_max": 8.0}
    out = R.biased_attention(np.zeros((1, 3)), w, m)
    np.testing.assert_allclose(out, [[2.0, 3.0, 0.0]])
    # a bias of ln 3 on distance 0 makes it 3 / 4
    w["rel"] = np.array([[np.log(3.0)], [0.0], [0.0], [0.0]])
    np.testing.assert_allclose(R.biased_attention(np.zeros((1, 3)), w, m), [[3.0, 4.5, 0.0]])


def test_oracle_head_mixing_and_temperature():
    # two heads, one position: scores (a0, a1) -> T @ (a0 * t0, a1 * t1); pick T that swaps the heads
    h = np.array([[1.0, 2.0]])
    w = {"q": np.array([[1.0, 0.0], [0.0, 1.0]]), "k": np.array([[1.0, 0.0], [0.0, 1.0]]), "v": np.array([[1.0, 0.0], [0.0, 1.0]]),
         "q.b": np.zeros(2), "k.b": np.zeros(2), "v.b": np.zeros(2), "o": np.eye(2), "o.b": np.zeros(2), "rel": np.zeros((2, 2)),
         "talk": np.array([[0.0, 1.0], [1.0, 0.0]]), "temp": np.array([2.0, 0.5])}
    m = {"heads": 2, "kv_heads": 2, "dim": 1, "vdim": 1, "scale": 0.5, "bias_max": 4.0}
    a0, a1 = 1.0 * 1.0 * 0.5 * 2.0, 2.0 * 2.0 * 0.5 * 0.5
    p0, p1 = np.exp(a1) / (1 + np.exp(a1)), np.exp(a0) / (1 + np.exp(a0))
    np.testing.assert_allclose(R.biased_attention(h, w, m), [[p0 * 1.0, p1 * 2.0]])


def test_oracle_routed_ff_weighs_the_input():
    # one expert chosen out of two; gate = up = identity rows, down = identity: y = g * sigmoid(1.702 g) * (u + 1) on s * h
    h = np.array([[0.4, -0.2]])
    w = {"router": np.array([[5.0, 0.0], [-5.0, 0.0]]), "e0.gate": np.eye(2), "e0.up": np.eye(2), "e0.down": np.eye(2),
         "e1.gate": 100 * np.eye(2), "e1.up": np.eye(2), "e1.down": np.eye(2)}
    mlp = {"router": {"experts": 2, "top": 1}, "expert": {"ff": 2, "limit": 0.3}}
    s = 1 / (1 + np.exp(-2.0))
    z = s * h[0]
    g = np.minimum(z, 0.3)
    u = np.clip(z, -0.3, 0.3)
    np.testing.assert_allclose(R.routed_ff(h, w, mlp)[0], g / (1 + np.exp(-1.702 * g)) * (u + 1))
    # both experts: the second one saturates at the limit
    mlp["router"]["top"] = 2
    s1 = 1 / (1 + np.exp(2.0))
    g1 = np.minimum(100 * s1 * h[0], 0.3)
    u1 = np.clip(s1 * h[0], -0.3, 0.3)
    want = g / (1 + np.exp(-1.702 * g)) * (u + 1) + g1 / (1 + np.exp(-1.702 * g1)) * (u1 + 1)
    np.testing.assert_allclose(R.routed_ff(h, w, mlp)[0], want)


def test_oracle_norm_and_prefix_invariance():
    x = np.array([[3.0, -4.0]])
    np.testing.assert_allclose(R.unit_offset_norm(x, np.array([0.5, -0.5]), 0.0), [[3 / np.sqrt(12.5) * 1.5, -4 / np.sqrt(12.5) * 0.5]])
    cfg = arch_synth.nufusun_config(32, 50, [arch_synth.nufusun_layer(4, 2, 8, 4, bias_max=12.0, experts=3, top=2, ff=16)], embed_scale=0.5)
    t = arch_synth.nufusun_weights(cfg, seed=5, rel_rows=8)
    toks = list(np.random.default_rng(0).integers(0, 50, 20))
    full = R.forward(cfg, t, toks)
    np.testing.assert_allclose(R.forward(cfg, t, toks[:11]), full[:11], rtol=1e-10, atol=1e-10)   # causal: a prefix does not see what follows
