"""GPU tests of the Vanapel design on the layer-list path: the CUDA backend (forward / sessions / decode_greedy behind
arch.load_model) against the plain numpy oracle in tests/_vanapel_ref.py, on small random models made here.

float32 mode is compared tightly with the oracle; bfloat16 mode loosely with the oracle and tightly with itself (the
same positions reached through different schedules)."""
import json
import os
import subprocess

import numpy as np
import pytest

from powerserve_b200 import arch, arch_synth, capi
from tests import _vanapel_ref as R

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
A, LA = arch_synth.vanapel_attention_layer, arch_synth.vanapel_latent_layer
YARN = {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}


def make(tmp_path, layers, width=48, vocab=96, seed=0, eps=1e-6, groups=1, edit=None, name="m"):
    cfg = arch_synth.vanapel_config(width, vocab, layers, eps=eps, groups=groups)
    t = arch_synth.vanapel_weights(cfg, seed=seed)
    if edit:
        edit(t)
        t = {k: R.bf16_round(v) for k, v in t.items()}
    d = str(tmp_path / name)
    arch_synth.write_model_dir(d, cfg, t)
    return d, cfg, t


def tokens(vocab, n, seed=0):
    return [int(v) for v in np.random.default_rng(seed).integers(0, vocab, n)]


def run(model, toks, cuts=None):
    """logits of every position, the sequence fed in portions of the given sizes (cycled); None = one portion per batch cap"""
    model.reset()
    cap, out, lo, k = model.desc.max_batch, [], 0, 0
    while lo < len(toks):
        s = min(cap if cuts is None else min(cuts[k % len(cuts)], cap), len(toks) - lo)
        out.append(model.forward(toks[lo:lo + s]))
        lo, k = lo + s, k + 1
    return np.concatenate(out)


def rel_err(got, ref):
    """per position: rms of the difference over rms of the reference"""
    return np.sqrt(((got - ref) ** 2).mean(-1)) / np.maximum(np.sqrt((ref ** 2).mean(-1)), 1e-6)


TOL = {"float32": 4e-5, "bfloat16": 5e-2}


def check(got, ref, dtype, what=""):
    e = rel_err(got, ref)
    assert e.max() < TOL[dtype], f"{what}: worst relative error {e.max():.3g} at position {int(e.argmax())} ({dtype})"
    if dtype == "bfloat16":
        assert np.median(e) < 1.5e-2, f"{what}: median relative error {np.median(e):.3g}"


def both_paths(d, toks, ref, what, n_ctx, cap=64, cuts=([7, 2, 33, 1],), decode_from=None):
    """float32: portions of the batch cap, ragged portions, and the tail decoded token by token, all against the oracle"""
    m = arch.load_model(d, dtype="float32", max_batch=cap, n_ctx=n_ctx)
    check(run(m, toks), ref, "float32", what + ", portions of the batch cap")
    for c in cuts:
        check(run(m, toks, list(c)), ref, "float32", what + f", portions {list(c)}")
    k = decode_from if decode_from is not None else len(toks) // 2
    m.reset()
    for lo in range(0, k, cap):
        m.forward(toks[lo:min(k, lo + cap)], lm_head=False)
    dec = np.concatenate([m.forward(toks[i:i + 1]) for i in range(k, len(toks))])
    check(dec, ref[k:], "float32", what + ", decoded alone")
    m.close()


# ------------------------------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("groups", [1, 2, 4])
def test_windowed_attention_layer_alone(tmp_path, groups):
    d, cfg, t = make(tmp_path, [A(4, 2, 16, 12, window=11)], seed=1, groups=groups)
    toks = tokens(96, 45, 1)
    taps = []
    ref = R.forward(cfg, t, toks, taps=taps)
    m = arch.load_model(d, dtype="float32", max_batch=64, n_ctx=64)
    m.be.set_option("arch_taps", 1)
    check(run(m, toks), ref, "float32", "attention-only layer")
    check(m.layer_tap(0, len(toks)), taps[0], "float32", "residual after the layer")
    m.close()
    both_paths(d, toks, ref, "attention-only layer", 64)


@pytest.mark.parametrize("scaling,rope_dims", [(YARN, None), (None, None), (YARN, 4)])
def test_latent_attention_layer_alone(tmp_path, scaling, rope_dims):
    d, cfg, t = make(tmp_path, [LA(3, 10, 8, 14, 20, 24, rope_base=300.0, rope_dims=rope_dims, scaling=scaling)], seed=2, groups=2)
    toks = tokens(96, 90, 2)
    taps = []
    ref = R.forward(cfg, t, toks, taps=taps)
    m = arch.load_model(d, dtype="float32", max_batch=96, n_ctx=96)
    m.be.set_option("arch_taps", 1)
    check(run(m, toks), ref, "float32", "latent-attention-only layer")
    check(m.layer_tap(0, len(toks)), taps[0], "float32", "residual after the layer")
    m.close()
    both_paths(d, toks, ref, "latent-attention-only layer", 96, cap=32)


def test_gated_feed_forward_limits(tmp_path):
    """large gate / up rows so that min(g, L) and clip(u, -L, L) bite for most entries; a second model with a limit nothing reaches"""
    def edit(t):
        t["l0.mlp.gate"] = t["l0.mlp.gate"] * 4.0
        t["l0.mlp.up"] = t["l0.mlp.up"] * 4.0
    for limit in (0.4, 50.0):
        d, cfg, t = make(tmp_path, [A(2, 1, 8, 8, window=6, ff=72, limit=limit)], seed=3, groups=3, edit=edit, name=f"m{limit}")
        toks = tokens(96, 40, 3)
        taps = []
        ref = R.forward(cfg, t, toks, taps=taps)
        m = arch.load_model(d, dtype="float32", max_batch=64, n_ctx=64)
        m.be.set_option("arch_taps", 1)
        check(run(m, toks), ref, "float32", f"feed-forward, limit {limit}")
        check(m.layer_tap(0, len(toks)), taps[0], "float32", "residual after the layer")
        m.close()
        both_paths(d, toks, ref, f"feed-forward, limit {limit}", 64, cuts=([2],))
    t2 = dict(t)
    t2["l0.mlp.gate"] = t["l0.mlp.gate"] * 0.5
    assert rel_err(R.forward(cfg, t2, toks), ref).max() > 1e-3          # (with the wide limit the gate's size matters)


def test_sinks_shift_the_heads(tmp_path):
    """head 0's sink takes most of its mass, head 1's next to none: leaving the sink out, or scaling / biasing it like a key, shows"""
    def edit(t):
        t["l0.mix.sink"] = np.array([4.0, -6.0, 1.0], np.float32)
    d, cfg, t = make(tmp_path, [A(3, 3, 8, 8, window=20, scale=0.5)], seed=4, edit=edit)
    toks = tokens(96, 50, 4)
    ref = R.forward(cfg, t, toks)
    t2 = dict(t)
    t2["l0.mix.sink"] = np.full(3, -40.0, np.float32)
    assert rel_err(R.forward(cfg, t2, toks), ref).max() > 1e-2          # the oracle itself: the sinks matter
    both_paths(d, toks, ref, "sinks", 64)


@pytest.mark.parametrize("window", [1, 2, 12, 16, 17, 33, 64, 65])
def test_window_edges(tmp_path, window):
    """q = k = 0 and r1 < 0 for head 0: its scores GROW with distance as 8 ln(1 + d), so the furthest key in sight (distance
    window - 1) holds the largest weight; a window one key too wide or too narrow, in a prompt portion or for a token decoded
    alone, at any place relative to the 16-key blocks and 64-key tiles of the kernels, moves the output by O(1)"""
    def edit(t):
        for n in ("q", "k"):
            t[f"l0.mix.{n}"] = np.zeros_like(t[f"l0.mix.{n}"])
        t["l0.mix.r1"] = np.array([-8.0, 0.5], np.float32)
        t["l0.mix.r2"] = np.array([1.0, 0.25], np.float32)
        t["l0.mix.sink"] = np.array([-2.0, 0.5], np.float32)
    d, cfg, t = make(tmp_path, [A(2, 1, 8, 16, window=window)], seed=5, edit=edit)
    n = 150
    toks = tokens(96, n, 5)
    ref = R.forward(cfg, t, toks)
    if window > 1:
        wider = json.loads(json.dumps(cfg))
        wider["layers"][0]["mixer"]["mask"]["size"] = window + 1
        assert rel_err(R.forward(wider, t, toks)[window:], ref[window:]).min() > 1e-3   # the oracle itself: one more key shows everywhere
    both_paths(d, toks, ref, f"window {window}", 160, decode_from=60)


def test_far_key_stands_out_in_the_latent_layer(tmp_path):
    """one early token's latent is made to stand out along a direction every later query shares: hundreds of positions later the
    causal soft-max still has to find it (prompt portions, and tokens decoded alone, across the portion edges)"""
    far_at, H, dn, dr = 5, 2, 8, 4

    def edit(t):
        t["embed"][:, 0], t["embed"][:, 1] = 2.0, 0.0
        t["embed"][39, 1] = 6.0                                     # a token that occurs once
        t["l0.norm1"] = np.ones_like(t["l0.norm1"])
        t["l0.mix.dq"][0], t["l0.mix.dkv"][0] = 0.0, 0.0
        t["l0.mix.dq"][0, 0] = 4.0                                  # query latent 0: positive for every token
        t["l0.mix.dkv"][0, 1] = 4.0                                 # kv latent 0: large for that token only
        t["l0.mix.dq.norm"], t["l0.mix.dkv.norm"] = np.ones_like(t["l0.mix.dq.norm"]), np.ones_like(t["l0.mix.dkv.norm"])
        for hh in range(H):
            t["l0.mix.uq"][hh * (dn + dr):hh * (dn + dr) + dn, 0] = 0.5
            t["l0.mix.uk"][hh * dn:(hh + 1) * dn, 0] = 3.0
    d, cfg, t = make(tmp_path, [LA(H, dn, dr, 8, 12, 16, scaling=YARN, rope_base=100.0)], width=32, vocab=40, seed=6, edit=edit)
    toks = tokens(39, 330, 6)
    toks[far_at] = 39
    ref = R.forward(cfg, t, toks)
    alt = list(toks)
    alt[far_at] = 1
    assert rel_err(R.forward(cfg, t, alt)[300:], ref[300:]).min() > 1e-2        # the far key matters to every late position
    m = arch.load_model(d, dtype="float32", max_batch=128, n_ctx=336)
    check(run(m, toks), ref, "float32", "far key, portions of 128")
    m.reset()
    m.forward(toks[:128], lm_head=False)
    for i in range(128, 290, 54):
        m.forward(toks[i:i + 54], lm_head=False)
    dec = np.concatenate([m.forward(toks[i:i + 1]) for i in range(290, 330)])
    check(dec, ref[290:], "float32", "far key, decoded alone")
    m.close()


def test_value_blending_across_layers(tmp_path):
    """the source of the blended values is the FIRST marked layer, which is not the first layer here; an unmarked layer sits between"""
    layers = [A(2, 2, 8, 6, window=9, ff=24), A(4, 2, 12, 10, window=7, v_mix=True), A(3, 3, 8, 5, window=30),
              A(6, 2, 4, 10, window=13, v_mix=True, ff=40), A(2, 2, 16, 10, window=4, v_mix=True)]
    def edit(t):
        t["l3.mix.vmix"] = np.array(0.75, np.float32)
        t["l4.mix.vmix"] = np.array(0.3125, np.float32)
        t["l1.mix.vmix"] = np.array(0.9, np.float32)                # never read
    d, cfg, t = make(tmp_path, layers, seed=7, groups=2, edit=edit)
    toks = tokens(96, 70, 7)
    ref = R.forward(cfg, t, toks)
    t2 = dict(t)
    t2["l4.mix.vmix"] = np.array(0.0, np.float32)
    assert rel_err(R.forward(cfg, t2, toks), ref).max() > 1e-3
    both_paths(d, toks, ref, "value blending", 80, cap=32, cuts=([2], [5, 1, 31]))


# ------------------------------------------------------------------------------------------------- schedules
MIXED = [A(4, 1, 16, 12, window=24, v_mix=True, ff=40, limit=1.5),
         LA(3, 8, 8, 10, 20, 16, scaling=YARN, rope_base=1000.0, ff=56, limit=0.8),
         A(6, 1, 8, 12, window=9, v_mix=True),
         A(2, 2, 24, 20, window=40, ff=32, limit=2.0),
         LA(2, 12, 4, 6, 10, 28, rope_dims=2, ff=24)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_decode_and_portions_agree(tmp_path, dtype):
    d, cfg, t = make(tmp_path, MIXED, width=72, vocab=130, seed=8, groups=3)
    toks = tokens(130, 140, 8)
    ref = R.forward(cfg, t, toks)
    m = arch.load_model(d, dtype=dtype, max_batch=64, n_ctx=144)
    whole = run(m, toks)
    check(whole, ref, dtype, "whole prompt")
    one = run(m, toks, [1])
    check(one, ref, dtype, "token by token")
    for cuts in ([2], [3, 2, 64, 1, 5], [37, 2, 2, 28, 1, 1, 9], [63, 64, 13]):
        got = run(m, toks, cuts)
        check(got, ref, dtype, f"portions {cuts}")
        assert rel_err(got, whole).max() < (1e-5 if dtype == "float32" else 3e-2), cuts   # the schedule changes rounding only
    assert rel_err(one, whole).max() < (1e-5 if dtype == "float32" else 3e-2)
    m.close()


def test_single_token_kernels_match_the_tiled_ones(tmp_path):
    d, cfg, t = make(tmp_path, MIXED, width=72, vocab=130, seed=9, groups=3)
    toks = tokens(130, 60, 9)
    for dtype in ("float32", "bfloat16"):
        m = arch.load_model(d, dtype=dtype, max_batch=32, n_ctx=64)
        n0 = m.be.counter("kernel_launches")
        a = run(m, toks, [1])
        n1 = m.be.counter("kernel_launches")
        m.be.set_option("arch_simple", 1)
        b = run(m, toks, [1])
        n2 = m.be.counter("kernel_launches")
        assert n1 - n0 != n2 - n1                                   # two different launch sequences did run
        # same operands, same roundings: only the summation order differs.  In bfloat16 mode a last-bit difference of an fp32
        # activation now and then lands on the other side of a bfloat16 rounding, the cached rows of a position then differ by
        # that much for every later query, and the norms of the sublayer outputs carry it on: 1e-3 .. 1e-2 after five layers
        assert rel_err(a, b).max() < (1e-5 if dtype == "float32" else 2e-2), dtype
        m.close()


def test_replayed_step_matches_the_plain_launches(tmp_path):
    """token-by-token decoding through the captured-and-replayed step (the default) against the same kernels launched one by one"""
    d, cfg, t = make(tmp_path, MIXED, width=72, vocab=130, seed=10, groups=3)
    toks = tokens(130, 90, 10)
    for dtype in ("float32", "bfloat16"):
        m = arch.load_model(d, dtype=dtype, max_batch=40, n_ctx=96)
        g0 = m.be.counter("graph_replays")
        a = run(m, toks, [1])
        assert m.be.counter("graph_replays") - g0 == len(toks)
        m.reset()
        m.forward(toks[:40], lm_head=False)
        ids_a = list(m.decode_greedy(toks[40], 20))
        m.be.set_option("graph", 0)
        b = run(m, toks, [1])
        m.reset()
        m.forward(toks[:40], lm_head=False)
        ids_b = list(m.decode_greedy(toks[40], 20))
        np.testing.assert_array_equal(a, b)                         # the same kernels on the same data
        assert ids_a == ids_b
        m.be.set_option("graph", 1)
        m.be.set_option("arch_pdl", 0)                              # every launch waits for the whole kernel before it
        np.testing.assert_array_equal(run(m, toks, [1]), a)
        m.close()


def test_tensor_core_gemm_matches_the_tile_kernels(tmp_path):
    """bfloat16 batches: the tcgen05 GEMM (projections, fused gate|up with the activation, down) against the fp32-FMA tile kernels on
    the same rounded operands - several row tiles, several column tiles, K not a multiple of the k block"""
    layers = [A(6, 3, 24, 20, window=50, v_mix=True, ff=200, limit=1.2), LA(4, 24, 8, 40, 72, 40, scaling=YARN, ff=136), A(6, 3, 40, 20, window=200, v_mix=True, ff=72)]
    d, cfg, t = make(tmp_path, layers, width=136, vocab=300, seed=11, groups=2)
    toks = tokens(300, 300, 11)
    m = arch.load_model(d, dtype="bfloat16", max_batch=160, n_ctx=304)
    n0 = m.be.counter("kernel_launches")
    a = run(m, toks)
    n1 = m.be.counter("kernel_launches")
    m.be.set_option("arch_tc", 0)
    b = run(m, toks)
    n2 = m.be.counter("kernel_launches")
    assert n1 - n0 > n2 - n1                                        # the tensor-core path adds its operand-tiling launches: it did run
    e = rel_err(a, b)
    # same rounded operands, another summation order: bfloat16 roundings that fall the other way (see above); a wrong tile shows as O(1)
    assert e[:4].max() < 1e-5 and np.median(e) < 5e-3 and e.max() < 2e-2, (np.median(e), e.max())
    check(a, R.forward(cfg, t, toks), "bfloat16", "tensor-core path against the oracle")
    m.close()


def test_sessions_interleaved_and_slots_reused(tmp_path):
    d, cfg, t = make(tmp_path, MIXED, width=72, vocab=130, seed=12, groups=3)
    reqs = [tokens(130, n, 20 + i) for i, n in enumerate((50, 9, 33, 64))]
    refs = [R.forward(cfg, t, r) for r in reqs]
    m = arch.load_model(d, dtype="float32", max_batch=16, n_ctx=64)
    sid = [m.session_create() for _ in range(3)]
    got = [[] for _ in reqs]
    at = [0, 0, 0, 0]
    sizes = [5, 2, 16, 1, 7]
    live, k = [0, 1, 2], 0
    while live:
        for r in list(live):
            s = min(sizes[k % len(sizes)], len(reqs[r]) - at[r])
            k += 1
            m.session_select(sid[r])
            assert m.position == at[r]
            got[r].append(m.forward(reqs[r][at[r]:at[r] + s]))
            at[r] += s
            if at[r] == len(reqs[r]):
                live.remove(r)
                if r == 1:              # the short request ends first: its cache set is freed and a new request takes a new one
                    m.session_select(0)
                    m.session_destroy(sid[1])
                    sid.append(m.session_create())
                    live.append(3)
    for r in range(4):
        check(np.concatenate(got[r]), refs[r], "float32", f"request {r} among others")
    # the same cache set used again from position 0 (stale rows of a longer request behind it), and after a rollback
    m.session_select(sid[0])
    m.reset()
    check(run(m, reqs[2], [16]), refs[2], "float32", "cache set reused after reset")
    m.be.kv_rollback(13)
    assert m.position == 20
    tail = np.concatenate([m.forward(reqs[2][20:27]), m.forward(reqs[2][27:])])
    check(tail, refs[2][20:], "float32", "continued after a rollback")
    m.close()


def test_long_decoding_past_every_window(tmp_path):
    layers = [A(4, 1, 8, 8, window=37, v_mix=True, ff=16), LA(2, 8, 4, 4, 8, 12, scaling=YARN, rope_base=200.0), A(2, 1, 8, 8, window=130, v_mix=True)]
    d, cfg, t = make(tmp_path, layers, width=32, vocab=50, seed=13, groups=2)
    toks = tokens(50, 400, 13)
    ref = R.forward(cfg, t, toks)
    for dtype in ("float32", "bfloat16"):
        m = arch.load_model(d, dtype=dtype, max_batch=8, n_ctx=400)
        m.reset()
        m.forward(toks[:6], lm_head=False)
        dec = np.concatenate([m.forward(toks[i:i + 1]) for i in range(6, 400)])
        check(dec, ref[6:], dtype, "394 tokens decoded alone")
        m.close()


@pytest.mark.parametrize("layers,width,vocab,groups", [
    ([A(1, 1, 4, 4, window=3)], 8, 11, 1),                                                          # the smallest of everything
    ([LA(1, 2, 2, 2, 3, 4)], 8, 11, 2),
    ([A(8, 8, 8, 8, window=100, ff=8)], 40, 64, 5),                                                 # no key sharing; a window nothing reaches
    ([A(8, 1, 12, 28, window=7, ff=20, limit=0.3)], 56, 77, 7),                                     # one shared key head, value wider than key
    ([LA(5, 6, 10, 3, 7, 33, scaling=YARN, ff=20), A(3, 3, 36, 4, window=2)], 48, 200, 4),          # odd ranks and sizes
    ([A(3, 1, 4, 36, window=90, v_mix=True, ff=72), LA(2, 16, 16, 16, 24, 24, rope_dims=8, scaling={"factor": 9.0, "original": 32, "fast": 4.0, "slow": 1.0})], 48, 200, 2),
    ([A(16, 4, 32, 32, window=48, v_mix=True, ff=96), A(16, 4, 32, 32, window=48, v_mix=True, ff=96)], 128, 300, 1),
    ([A(5, 5, 6, 10, window=5, ff=37, limit=1.1), LA(3, 5, 6, 3, 7, 9, rope_dims=6, ff=13)], 50, 101, 5),                      # nothing a multiple of four
])
def test_other_sizes(tmp_path, layers, width, vocab, groups):
    d, cfg, t = make(tmp_path, layers, width=width, vocab=vocab, seed=14, eps=1e-5, groups=groups)
    toks = tokens(vocab, 75, 14)
    ref = R.forward(cfg, t, toks)
    m = arch.load_model(d, dtype="float32", max_batch=32, n_ctx=80)
    check(run(m, toks), ref, "float32", "portions of 32")
    check(run(m, toks, [2, 31, 1]), ref, "float32", "ragged portions")
    check(run(m, toks[:40], [1]), ref[:40], "float32", "token by token")
    m.close()
    m = arch.load_model(d, dtype="bfloat16", max_batch=80, n_ctx=80)
    check(run(m, toks), ref, "bfloat16", "whole prompt")
    m.close()


# ------------------------------------------------------------------------------------------------- entry points
def test_greedy_generation_through_the_entry_points(tmp_path):
    d, cfg, t = make(tmp_path, MIXED, width=72, vocab=130, seed=15, groups=3)
    prompt = tokens(130, 21, 15)
    m = arch.load_model(d, dtype="float32", max_batch=8, n_ctx=64)
    ids, lg = m.generate(prompt, 12, batch_size=8)                  # prefill in portions + one forward per token
    m.reset()
    m.prefill(prompt, 8)
    ids2 = [int(v) for v in m.decode_greedy(prompt[-1], 12)]        # the device-side greedy loop
    assert ids == ids2
    assert m.position == len(prompt) - 1 + 12
    seq = list(prompt)
    for step, tok in enumerate(ids):
        ref = R.forward(cfg, t, seq)[-1]
        assert rel_err(lg[step][None], ref[None]).max() < 4e-5
        assert ref[tok] >= ref.max() - 1e-4 * np.abs(ref).max()
        seq.append(tok)
    m.forward_lazy([seq[-1]])
    vals, idx = m.sample_topk(5)
    full = R.forward(cfg, t, seq)[-1]
    assert list(idx) == [int(v) for v in np.argsort(-full, kind="stable")[:5]]
    m.close()


def test_bad_geometries_are_refused(tmp_path):
    # blended value rows of different widths; a width that does not split into the norm groups
    d, cfg, t = make(tmp_path, [A(2, 1, 8, 8, window=4, v_mix=True), A(2, 2, 8, 8, window=4, v_mix=True)], seed=16)
    with pytest.raises(capi.PsCudaError):
        arch.load_model(d, dtype="float32", max_batch=8, n_ctx=16)
    d, cfg, t = make(tmp_path, [A(2, 1, 8, 8, window=4)], width=50, seed=16, groups=4, name="g")
    with pytest.raises(capi.PsCudaError):
        arch.load_model(d, dtype="float32", max_batch=8, n_ctx=16)


def test_trace_runner_and_generation_command_lines(tmp_path):
    d, cfg, t = make(tmp_path, MIXED, width=72, vocab=130, seed=17, groups=3)
    a, b = tokens(130, 40, 30), tokens(130, 17, 31)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:32], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[32:], "want": [7, 3]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "b", "tokens": b, "want": [16]}], "end": ["b"]}]
    out = tmp_path / "out"
    ra, rb = R.forward(cfg, t, a), R.forward(cfg, t, b)
    for dtype in ("float32", "bfloat16"):
        p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out), "--max-tokens", "40", "--max-batch", "16"],
                           input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
        check(np.fromfile(out / "0.f32", "<f4").reshape(2, 130), ra[[0, 29]], dtype, "step 0")
        assert not (out / "1.f32").exists()
        check(np.fromfile(out / "2.f32", "<f4").reshape(2, 130), ra[[39, 35]], dtype, "step 2 (order of `want`)")
        check(np.fromfile(out / "3.f32", "<f4").reshape(1, 130), rb[[16]], dtype, "step 3")
        for f in out.iterdir():
            f.unlink()
    prompt = tokens(130, 19, 18)
    exe = os.path.join(ROOT, "bin", "ps_generate")
    p = subprocess.run([exe, "--model", d, "--dtype", "float32", "--ids", " ".join(map(str, prompt)), "--n", "10", "--prefill-batch", "8"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    ids = json.loads(p.stdout.strip().splitlines()[-1])["ids"]
    m = arch.load_model(d, dtype="float32", max_batch=32, n_ctx=32)
    want, _ = m.generate(prompt, 10, batch_size=8)
    assert ids == want
    m.close()
