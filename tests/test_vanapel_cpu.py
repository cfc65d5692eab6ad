"""CPU-only checks around the Vanapel design: the registry's reading of a configuration (every size and constant comes from
the file), the tensor names, the host-side rotation-frequency table against the oracle's formula, and the oracle's own
invariants (it is what the GPU tests compare with, so it is checked against hand-computed cases and a second formulation here)."""
import ctypes as C
import math

import numpy as np
import pytest

from powerserve_b200 import arch, arch_synth, build, capi
from tests import _vanapel_ref as R

A, LA = arch_synth.vanapel_attention_layer, arch_synth.vanapel_latent_layer
YARN = {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}


@pytest.fixture(scope="module")
def lib():
    build.build()
    return capi.load_library()


def test_registry_reads_every_size_from_the_configuration():
    layers = [LA(3, 10, 6, 14, 20, 24, scale=0.3, rope_base=500.0, rope_dims=4, scaling=YARN, ff=44, limit=0.7),
              A(6, 3, 12, 20, window=9, scale=0.21, ff=0),
              A(4, 2, 8, 15, window=33, v_mix=True, ff=52, limit=2.5),
              A(8, 2, 16, 15, window=5, v_mix=True)]
    cfg = arch_synth.vanapel_config(60, 99, layers, eps=3e-5, groups=3)
    descs, top = arch.ARCHITECTURES["Vanapel"][0](cfg, {})
    assert top == {"dim": 60, "vocab_size": 99, "norm_eps": 3e-5, "embed_scale": 1.0, "norm_unit_offset": 0, "norm_groups": 3}
    d = descs[0]
    assert (d.mixer_kind, d.n_heads, d.n_kv_heads, d.qk_dim, d.rot_dim, d.v_dim, d.q_rank, d.kv_rank) == (capi.MIXER_LATENT, 3, 1, 10, 6, 14, 20, 24)
    assert (d.rope_dims, d.rope_original, d.window, d.qk_norm, d.log_bias, d.v_mix) == (4, 64, 0, 0, 0, 0)
    assert d.rope_base == 500.0 and d.rope_factor == 4.0 and d.rope_fast == 16.0 and d.rope_slow == 2.0
    assert abs(d.score_scale - 0.3) < 1e-7 and d.sink == capi.SINK_LEARNED
    assert (d.mlp_kind, d.expert_ff) == (capi.MLP_DENSE, 44) and abs(d.act_limit - 0.7) < 1e-7 and abs(d.act_alpha - 1.702) < 1e-6 and d.up_shift == 1.0
    d = descs[1]
    assert (d.mixer_kind, d.n_heads, d.n_kv_heads, d.qk_dim, d.v_dim, d.window, d.mlp_kind) == (capi.MIXER_ATTENTION, 6, 3, 12, 20, 9, capi.MLP_NONE)
    assert (d.qk_norm, d.log_bias, d.v_mix, d.block_kind, d.post_norm) == (1, 1, capi.VMIX_NONE, capi.BLOCK_SEQUENTIAL, 1)
    # the first layer marked v_mix supplies the values, every later one blends with them
    assert descs[2].v_mix == capi.VMIX_SOURCE and descs[3].v_mix == capi.VMIX_BLEND
    assert descs[2].window == 33 and descs[3].window == 5 and abs(descs[2].act_limit - 2.5) < 1e-7


def test_plain_rotation_without_scaling():
    cfg = arch_synth.vanapel_config(16, 8, [LA(2, 4, 4, 4, 6, 6, rope_base=77.0)])
    d = arch.ARCHITECTURES["Vanapel"][0](cfg, {})[0][0]
    assert d.rope_factor == 0.0 and d.rope_dims == 4 and d.rope_base == 77.0


def test_tensor_names_follow_the_layer_types():
    cfg = arch_synth.vanapel_config(16, 8, [A(2, 1, 4, 4, window=3, v_mix=True, ff=8), LA(2, 4, 2, 4, 6, 6), A(2, 2, 4, 4, window=3)])
    n = arch.ARCHITECTURES["Vanapel"][1](cfg)
    assert (n["embed"], n["final_norm"], n["head"]) == ("embed", "final.norm", "head")
    l0, l1, l2 = n["layers"]
    assert l0["norm"] == "l0.norm1" and l0["norm_mix_out"] == "l0.norm1b" and l0["norm_ff"] == "l0.norm2" and l0["norm_ff_out"] == "l0.norm2b"
    assert l0["vmix"] == "l0.mix.vmix" and l0["r1"] == "l0.mix.r1" and l0["gate"] == ["l0.mlp.gate"] and l0["down"] == ["l0.mlp.down"]
    assert l1["dq_norm"] == "l1.mix.dq.norm" and l1["dkv"] == "l1.mix.dkv" and l1["uk"] == "l1.mix.uk" and "q" not in l1 and "norm_ff" not in l1
    assert "vmix" not in l2 and l2["sink"] == "l2.mix.sink"
    t = arch_synth.vanapel_weights(cfg, seed=1)
    used = {v for l in n["layers"] for v in l.values() if isinstance(v, str)} | {x for l in n["layers"] for v in l.values() if isinstance(v, list) for x in v}
    assert used | {"embed", "final.norm", "head"} == set(t)


def test_unknown_types_are_refused():
    cfg = arch_synth.vanapel_config(16, 8, [A(2, 1, 4, 4, window=3)])
    cfg["layers"][0]["type"] = "convolution"
    with pytest.raises(capi.PsCudaError):
        arch.ARCHITECTURES["Vanapel"][0](cfg, {})
    cfg = arch_synth.vanapel_config(16, 8, [A(2, 1, 4, 4, window=3, ff=8)])
    cfg["layers"][0]["mlp"]["kind"] = "moe"
    with pytest.raises(capi.PsCudaError):
        arch.ARCHITECTURES["Vanapel"][0](cfg, {})


@pytest.mark.parametrize("dims,base,scaling", [(8, 10000.0, None), (32, 500.0, YARN), (6, 123.0, {"factor": 16.0, "original": 200, "fast": 8.0, "slow": 0.5}),
                                               (64, 1e6, {"factor": 2.0, "original": 4096, "fast": 32.0, "slow": 1.0}), (2, 9.0, YARN)])
def test_host_rotation_table_matches_the_formula(lib, dims, base, scaling):
    rot = {"dims": dims, "base": base}
    if scaling:
        rot["scaling"] = scaling
    f, mag = R.rotation_frequencies(rot)
    out = (C.c_float * (dims // 2))()
    sc = scaling or {"factor": 0.0, "original": 0, "fast": 0.0, "slow": 0.0}
    m = lib.ps_cuda_host_rope_freq(dims, base, sc["factor"], sc["original"], sc["fast"], sc["slow"], out)
    np.testing.assert_allclose(np.array(out[:]), f, rtol=1e-6)
    assert abs(m - mag) < 1e-6


def test_rotation_table_by_hand():
    # 8 rotated dims, base 16: f = 16^(-i/4) = 1, 1/2, 1/4, 1/8.  original 32: c(r) = 8 ln(32 / (2 pi r)) / (2 ln 16);
    # fast 4 -> c = 0.348 -> lo 0; slow 1 -> c = 2.348 -> hi 3: t = 0, 1/3, 2/3, 1; factor 2
    f, mag = R.rotation_frequencies({"dims": 8, "base": 16.0, "scaling": {"factor": 2.0, "original": 32, "fast": 4.0, "slow": 1.0}})
    np.testing.assert_allclose(f, [1.0, 0.5 * (1 - 1 / 6), 0.25 * (1 - 1 / 3), 0.125 / 2], rtol=1e-12)
    assert abs(mag - (0.1 * math.log(2.0) + 1.0)) < 1e-12


def test_oracle_group_norm_and_softmax_by_hand():
    x = np.array([[3.0, 4.0, 0.0, 2.0]])
    w = np.array([1.0, 2.0, 3.0, 0.5])
    np.testing.assert_allclose(R.group_norm(x, w, 0.0, 1), x / math.sqrt(29 / 4) * w)
    np.testing.assert_allclose(R.group_norm(x, w, 0.0, 2), [[3 / math.sqrt(12.5), 8 / math.sqrt(12.5), 0.0, 0.5 * 2 / math.sqrt(2.0)]])
    # two visible keys with scores ln 1 and ln 3, sink ln 4: weights 1/8 and 3/8, the rest is the sink's
    s = np.array([[0.0, -50.0, 7.0], [math.log(1.0), math.log(3.0), 9.0]])
    ok = np.array([[True, False, False], [True, True, False]])
    p = R.sink_softmax(s, ok, math.log(4.0))
    np.testing.assert_allclose(p, [[0.2, 0.0, 0.0], [0.125, 0.375, 0.0]], atol=1e-15)
    np.testing.assert_array_equal(R.visible(4, 2), np.array([[1, 0, 0, 0], [1, 1, 0, 0], [0, 1, 1, 0], [0, 0, 1, 1]], bool))
    np.testing.assert_array_equal(R.visible(3, None), np.tril(np.ones((3, 3), bool)))
    np.testing.assert_allclose(R.distance_penalty(2.0, 0.5, 3), [[0, 0, 0], [2 * math.log(1.5), 0, 0], [2 * math.log(2.0), 2 * math.log(1.5), 0]])


def test_oracle_rotation_properties():
    rng = np.random.default_rng(2)
    rot = {"dims": 6, "base": 50.0, "scaling": YARN}
    x = rng.standard_normal((5, 2, 8))
    y = R.rotate(x, np.arange(5), rot)
    _, mag = R.rotation_frequencies(rot)
    np.testing.assert_allclose(y[..., 6:], x[..., 6:])                                        # dims beyond the rotated ones pass
    np.testing.assert_allclose(np.linalg.norm(y[..., :6], axis=-1), mag * np.linalg.norm(x[..., :6], axis=-1))
    np.testing.assert_allclose(y[0, :, :6], mag * x[0, :, :6])                                # position 0: no turn
    # the product of a turned query and a turned key depends on the distance only
    q, k = rng.standard_normal((1, 1, 6)), rng.standard_normal((1, 1, 6))
    a = (R.rotate(q, [9], rot) * R.rotate(k, [4], rot)).sum()
    b = (R.rotate(q, [25], rot) * R.rotate(k, [20], rot)).sum()
    assert abs(a - b) < 1e-12


def test_oracle_latent_attention_equals_the_folded_form():
    """the latent attention written the other way round - W_uk folded into the query, W_uv applied to the weighted sum of latents -
    gives the same output: what a cache of latents relies on"""
    rng = np.random.default_rng(3)
    layer = LA(3, 5, 4, 7, 9, 11, scaling=YARN, rope_base=300.0)
    cfg = arch_synth.vanapel_config(20, 30, [layer])
    t = {k: v.astype(np.float64) for k, v in arch_synth.vanapel_weights(cfg, seed=3).items()}
    w = {k[7:]: v for k, v in t.items() if k.startswith("l0.mix.")}
    m, eps, n = layer["mixer"], 1e-6, 13
    h = rng.standard_normal((n, 20))
    ref = R.latent_attention(h, w, m, eps)
    H, dn, dr, dv, rk = 3, 5, 4, 7, 11
    cq = R.unit_rms(h @ w["dq"].T, eps) * w["dq.norm"]
    q = (cq @ w["uq"].T).reshape(n, H, dn + dr)
    tt = h @ w["dkv"].T
    c = R.unit_rms(tt[:, :rk], eps) * w["dkv.norm"]
    kr = R.rotate(tt[:, rk:].reshape(n, 1, dr), np.arange(n), m["rot"])[:, 0]
    qr = R.rotate(q[..., dn:], np.arange(n), m["rot"])
    out = np.zeros((n, H, dv))
    for hh in range(H):
        uk, uv = w["uk"][hh * dn:(hh + 1) * dn], w["uv"][hh * dv:(hh + 1) * dv]
        s = ((q[:, hh, :dn] @ uk) @ c.T + qr[:, hh] @ kr.T) * m["scale"]
        out[:, hh] = (R.sink_softmax(s, R.visible(n, None), float(w["sink"][hh])) @ c) @ uv.T
    np.testing.assert_allclose(out.reshape(n, H * dv) @ w["o"].T, ref, rtol=1e-9, atol=1e-9)


def test_oracle_value_blending_and_window():
    cfg = arch_synth.vanapel_config(16, 20, [A(2, 1, 4, 6, window=3, v_mix=True), A(3, 1, 8, 6, window=2, v_mix=True)])
    t = arch_synth.vanapel_weights(cfg, seed=4)
    toks = [1, 5, 5, 2, 9, 3, 3, 7]
    a = R.forward(cfg, t, toks)
    # a token further back than every window cannot matter: two layers of windows 3 and 2 reach 3 positions back
    alt = list(toks)
    alt[0] = 11
    b = R.forward(cfg, t, alt)
    assert np.abs(a[4:] - b[4:]).max() < 1e-12 and np.abs(a[:4] - b[:4]).max() > 1e-3
    # the second layer's blend weight matters, the first layer's own is never read
    t2 = dict(t)
    t2["l1.mix.vmix"] = np.array(0.0, np.float32)
    assert np.abs(R.forward(cfg, t2, toks) - a).max() > 1e-3
    t3 = dict(t)
    t3["l0.mix.vmix"] = np.array(0.9, np.float32)
    np.testing.assert_array_equal(R.forward(cfg, t3, toks), a)
