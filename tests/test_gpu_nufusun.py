"""GPU tests of the Nufusun design on the layer-list path: the CUDA backend (forward / sessions / decode_greedy behind
arch.load_model) against the plain numpy oracle in tests/_nufusun_ref.py, on small random models made here.

float32 mode is compared tightly with the oracle; bfloat16 mode loosely with the oracle and tightly with itself (the
same positions reached through different schedules)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from powerserve_b200 import arch, arch_synth, capi
from tests import _nufusun_ref as R

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
L = arch_synth.nufusun_layer


def make(tmp_path, layers, width=64, vocab=96, seed=0, rel_rows=8, eps=1e-5, embed_scale=0.5, edit=None, name="m"):
    cfg = arch_synth.nufusun_config(width, vocab, layers, eps=eps, embed_scale=embed_scale)
    t = arch_synth.nufusun_weights(cfg, seed=seed, rel_rows=rel_rows)
    if edit:
        edit(t)
        t = {k: R.bf16_round(v) if v.dtype != np.int32 else v for k, v in t.items()}
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
    if dtype == "bfloat16":
        # bfloat16 noise in the residual stream can turn a near-tie of two router scores the other way for a single token (the
        # float32 runs are the sharp check): the typical position must be close, and all but a few within the tolerance
        assert np.median(e) < 1e-2 and (e > TOL[dtype]).sum() <= max(1, len(e) // 40), \
            f"{what}: median relative error {np.median(e):.3g}, {(e > TOL[dtype]).sum()} of {len(e)} positions over {TOL[dtype]} ({dtype})"
        return
    assert e.max() < TOL[dtype], f"{what}: worst relative error {e.max():.3g} at position {int(e.argmax())} ({dtype})"


# ------------------------------------------------------------------------------------------------- mechanisms alone
def test_attention_layer_alone(tmp_path):
    d, cfg, t = make(tmp_path, [L(4, 2, 16, 8, bias_max=20.0)], seed=1)
    toks = tokens(96, 45, 1)
    taps = []
    ref = R.forward(cfg, t, toks, taps=taps)
    m = arch.load_model(d, dtype="float32", max_batch=64, n_ctx=64)
    m.be.set_option("arch_taps", 1)
    check(run(m, toks), ref, "float32", "attention-only layer")
    check(m.layer_tap(0, len(toks)), taps[0], "float32", "residual after the layer")
    m.close()


def test_routed_ff_alone(tmp_path):
    # the mixer's output projection and bias are zero: the layer adds ff(h) only
    def edit(t):
        t["l0.mix.o"] = np.zeros_like(t["l0.mix.o"])
        t["l0.mix.o.b"] = np.zeros_like(t["l0.mix.o.b"])
    for experts, top in ((4, 1), (4, 2), (3, 3)):
        d, cfg, t = make(tmp_path, [L(2, 1, 8, 8, experts=experts, top=top, ff=24, limit=0.8)], seed=2, edit=edit, name=f"ff{experts}{top}")
        toks = tokens(96, 70, 2)
        taps = []
        ref = R.forward(cfg, t, toks, taps=taps)
        h = R.unit_offset_norm(R.embed(t["embed"].astype(np.float64), toks, 0.5), t["l0.norm1"].astype(np.float64), 1e-5)
        fw = {k[7:]: v.astype(np.float64) for k, v in t.items() if k.startswith("l0.mlp.")}
        np.testing.assert_allclose(taps[0], R.embed(t["embed"].astype(np.float64), toks, 0.5) + R.routed_ff(h, fw, cfg["layers"][0]["mlp"]), atol=1e-12)
        m = arch.load_model(d, dtype="float32", max_batch=32, n_ctx=80)     # 70 tokens: three portions, the last one ragged
        m.be.set_option("arch_taps", 1)
        lg = run(m, toks)
        check(lg, ref, "float32", f"routed ff, {experts} experts top {top}")
        m.reset()
        m.forward(toks[:32], lm_head=False)
        check(m.layer_tap(0, 32), taps[0][:32], "float32", "x + ff(h)")
        m.close()


def test_sink_dominates_when_all_scores_are_low(tmp_path):
    # every distance bias is -9: the keys share e^-9-ish of the mass, the value-less sink takes the rest, the mixer adds ~ its bias
    def edit(t):
        t["l0.mix.rel"] = np.full_like(t["l0.mix.rel"], -9.0)
        t["l0.mix.talk"] = np.eye(4, dtype=np.float32)
        t["l0.mix.q"] = t["l0.mix.q"] * 0.05
    d, cfg, t = make(tmp_path, [L(4, 4, 8, 8, bias_max=20.0)], seed=3, edit=edit)
    toks = tokens(96, 12, 3)
    taps = []
    ref = R.forward(cfg, t, toks, taps=taps)
    x0 = R.embed(t["embed"].astype(np.float64), toks, 0.5)
    assert np.abs(taps[0] - x0 - t["l0.mix.o.b"]).max() < 0.05       # the oracle itself: almost nothing but the output bias
    m = arch.load_model(d, dtype="float32", max_batch=16, n_ctx=16)
    check(run(m, toks), ref, "float32", "sink-dominated attention")
    check(run(m, toks, [1]), ref, "float32", "sink-dominated attention, token by token")
    m.close()


@pytest.mark.parametrize("rows,dmax,target", [(8, 64.0, 3), (8, 64.0, 4), (8, 64.0, 6), (8, 64.0, 7), (10, 33.0, 5), (10, 33.0, 9), (9, 50.0, 4), (6, 7.0, 5)])
def test_distance_bias_edges(tmp_path, rows, dmax, target):
    """q = k = 0, so the scores are the distance biases alone; ONE row of the table is +9 for head 0: that head attends to
    exactly the keys whose distance falls into that bucket, so a table that is off by one position at either edge of the
    bucket (in a prompt portion or for a token decoded alone) moves the output by O(1)."""
    def edit(t):
        for n in ("q", "k"):
            t[f"l0.mix.{n}"] = np.zeros_like(t[f"l0.mix.{n}"])
            t[f"l0.mix.{n}.b"] = np.zeros_like(t[f"l0.mix.{n}.b"])
        rel = np.zeros_like(t["l0.mix.rel"])
        rel[target, 0] = 9.0
        rel[:, 1] = np.linspace(-2, 2, rows)
        t["l0.mix.rel"] = rel
        t["l0.mix.talk"] = np.eye(2, dtype=np.float32)
        t["l0.mix.temp"] = np.ones(2, np.float32)
    d, cfg, t = make(tmp_path, [L(2, 1, 8, 16, bias_max=dmax)], seed=4, rel_rows=rows, edit=edit)
    n = 150
    toks = tokens(96, n, 4)
    ref = R.forward(cfg, t, toks)
    m = arch.load_model(d, dtype="float32", max_batch=64, n_ctx=160)
    check(run(m, toks), ref, "float32", "portions of 64")
    check(run(m, toks, [7, 2, 33, 1]), ref, "float32", "ragged portions")
    m.reset()
    m.forward(toks[:60], lm_head=False)
    m.forward(toks[60:90], lm_head=False)
    dec = np.concatenate([m.forward(toks[i:i + 1]) for i in range(90, n)])
    check(dec, ref[90:], "float32", "decoded alone")
    m.close()


def test_far_key_stands_out(tmp_path):
    """one early token's key is made 30x larger along a direction every later query shares: hundreds of positions later the
    soft-max still has to find it (prompt portions, and tokens decoded alone, across the portion edges)"""
    far_at = 5

    def edit(t):
        t["l0.mix.rel"] = t["l0.mix.rel"] * 0.1
    d, cfg, t = make(tmp_path, [L(2, 2, 16, 8, bias_max=50.0, scale=0.25)], width=32, vocab=40, seed=5, edit=edit)
    toks = tokens(39, 330, 5)
    toks[far_at] = 39                                           # a token that occurs once
    # its embedding: large along the first right-singular direction of W_k, so its key is large along the matching left-singular
    # direction; the query bias has a component along that direction, so every later query sees it
    U, sv, Vt = np.linalg.svd(t["l0.mix.k"].astype(np.float64))
    t["embed"][39] = R.bf16_round((Vt[0] * 40).astype(np.float32))
    t["l0.mix.q.b"] = R.bf16_round((U[:, 0] * 2.0).astype(np.float32))
    arch_synth.write_model_dir(d, cfg, t)
    ref = R.forward(cfg, t, toks)
    alt = list(toks)
    alt[far_at] = 1
    assert rel_err(R.forward(cfg, t, alt)[300:], ref[300:]).max() > 1e-3      # the far key matters to the late positions
    m = arch.load_model(d, dtype="float32", max_batch=128, n_ctx=336)
    check(run(m, toks), ref, "float32", "far key, portions of 128")
    m.reset()
    m.forward(toks[:128], lm_head=False)
    for i in range(128, 290, 54):
        m.forward(toks[i:i + 54], lm_head=False)
    dec = np.concatenate([m.forward(toks[i:i + 1]) for i in range(290, 330)])
    check(dec, ref[290:], "float32", "far key, decoded alone")
    m.close()


# ------------------------------------------------------------------------------------------------- schedules
MIXED = [L(4, 2, 16, 8, bias_max=30.0, experts=4, top=2, ff=32, limit=1.5), L(6, 3, 8, 12, bias_max=11.0), L(2, 2, 24, 20, bias_max=60.0, experts=3, top=1, ff=40, limit=0.6)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_decode_and_portions_agree(tmp_path, dtype):
    d, cfg, t = make(tmp_path, MIXED, width=72, vocab=130, seed=6, rel_rows=10)
    toks = tokens(130, 140, 6)
    ref = R.forward(cfg, t, toks)
    m = arch.load_model(d, dtype=dtype, max_batch=64, n_ctx=144)
    whole = run(m, toks)
    check(whole, ref, dtype, "whole prompt")
    one = run(m, toks, [1])
    check(one, ref, dtype, "token by token")
    for cuts in ([2], [3, 2, 64, 1, 5], [37, 2, 2, 28, 1, 1, 9], [63, 64, 13]):
        got = run(m, toks, cuts)
        check(got, ref, dtype, f"portions {cuts}")
        assert rel_err(got, whole).max() < (1e-5 if dtype == "float32" else 2e-2), cuts   # the schedule changes rounding only
    assert rel_err(one, whole).max() < (1e-5 if dtype == "float32" else 2e-2)
    m.close()


def test_single_token_kernels_match_the_tiled_ones(tmp_path):
    d, cfg, t = make(tmp_path, MIXED, width=72, vocab=130, seed=7, rel_rows=10)
    toks = tokens(130, 60, 7)
    for dtype in ("float32", "bfloat16"):
        m = arch.load_model(d, dtype=dtype, max_batch=32, n_ctx=64)
        a = run(m, toks, [1])
        m.be.set_option("arch_simple", 1)
        b = run(m, toks, [1])
        # same operands, same roundings: only the summation order differs (in bfloat16 mode a last-bit difference of an fp32
        # activation now and then lands on the other side of a bfloat16 rounding)
        assert rel_err(a, b).max() < (1e-5 if dtype == "float32" else 1e-3), dtype
        m.close()


def test_replayed_step_matches_the_plain_launches(tmp_path):
    """token-by-token decoding through the captured-and-replayed step (the default) against the same kernels launched one by one"""
    d, cfg, t = make(tmp_path, MIXED, width=72, vocab=130, seed=15, rel_rows=10)
    toks = tokens(130, 90, 15)
    for dtype in ("float32", "bfloat16"):
        m = arch.load_model(d, dtype=dtype, max_batch=40, n_ctx=96)
        g0 = m.be.counter("graph_replays")
        a = run(m, toks, [1])
        assert m.be.counter("graph_replays") - g0 == len(toks)
        m.reset()
        m.forward(toks[:40], lm_head=False)
        ids_a = list(m.decode_greedy(toks[40], 20))
        m.be.set_option("graph", 0)
        g1 = m.be.counter("graph_replays")
        b = run(m, toks, [1])
        assert m.be.counter("graph_replays") == g1
        m.reset()
        m.forward(toks[:40], lm_head=False)
        ids_b = list(m.decode_greedy(toks[40], 20))
        np.testing.assert_array_equal(a, b)             # the same kernels on the same data
        assert ids_a == ids_b
        m.be.set_option("arch_fork", 0)                 # gate | up of the experts behind the attention instead of beside it
        np.testing.assert_array_equal(run(m, toks, [1]), a)
        m.be.set_option("graph", 1)
        np.testing.assert_array_equal(run(m, toks, [1]), a)
        m.be.set_option("arch_pdl", 0)                  # every launch waits for the whole kernel before it
        np.testing.assert_array_equal(run(m, toks, [1]), a)
        m.close()


def test_tensor_core_gemm_matches_the_tile_kernels(tmp_path):
    """bfloat16 batches: the tcgen05 GEMM (dense, fused gate|up, down with scatter) against the fp32-FMA tile kernels on the same
    rounded operands - several row tiles, several column tiles, K not a multiple of the k block, experts with ragged row lists"""
    layers = [L(6, 3, 24, 20, bias_max=30.0, experts=5, top=2, ff=200, limit=1.2), L(4, 2, 40, 24, bias_max=11.0, experts=3, top=3, ff=72)]
    d, cfg, t = make(tmp_path, layers, width=136, vocab=300, seed=14, rel_rows=10)
    toks = tokens(300, 300, 14)
    m = arch.load_model(d, dtype="bfloat16", max_batch=160, n_ctx=304)
    n0 = m.be.counter("kernel_launches")
    a = run(m, toks)
    n1 = m.be.counter("kernel_launches")
    m.be.set_option("arch_tc", 0)
    b = run(m, toks)
    n2 = m.be.counter("kernel_launches")
    assert n1 - n0 > n2 - n1                                    # the tensor-core path adds its operand-tiling launches: it did run
    e = rel_err(a, b)
    # same operands, another summation order: an fp32 activation that differs in its last bit now and then lands on the other side of
    # a bfloat16 rounding (one operand off by 2^-8 of itself), which shows as 1e-3 at that position; a wrong tile would show as O(1)
    assert np.median(e) < 1e-5 and np.quantile(e, 0.9) < 2e-3 and e.max() < 8e-3, (np.median(e), e.max())
    check(a, R.forward(cfg, t, toks), "bfloat16", "tensor-core path against the oracle")
    m.close()


def test_sessions_interleaved_and_slots_reused(tmp_path):
    d, cfg, t = make(tmp_path, MIXED, width=72, vocab=130, seed=8, rel_rows=10)
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
    # the same cache set used again from position 0, and after a rollback
    m.session_select(sid[0])
    m.reset()
    check(run(m, reqs[2], [16]), refs[2], "float32", "cache set reused after reset")
    m.be.kv_rollback(13)
    assert m.position == 20
    tail = np.concatenate([m.forward(reqs[2][20:27]), m.forward(reqs[2][27:])])
    check(tail, refs[2][20:], "float32", "continued after a rollback")
    m.close()


def test_long_decoding(tmp_path):
    d, cfg, t = make(tmp_path, [L(4, 1, 8, 8, bias_max=100.0, experts=4, top=2, ff=16), L(2, 2, 8, 4, bias_max=25.0)], width=32, vocab=50, seed=9, rel_rows=12)
    toks = tokens(50, 400, 9)
    ref = R.forward(cfg, t, toks)
    for dtype in ("float32", "bfloat16"):
        m = arch.load_model(d, dtype=dtype, max_batch=8, n_ctx=400)
        m.reset()
        m.forward(toks[:6], lm_head=False)
        dec = np.concatenate([m.forward(toks[i:i + 1]) for i in range(6, 400)])
        check(dec, ref[6:], dtype, "394 tokens decoded alone")
        m.close()


@pytest.mark.parametrize("layers,width,vocab,rows", [
    ([L(1, 1, 4, 4, bias_max=5.0)], 8, 11, 4),                                            # the smallest of everything
    ([L(8, 8, 8, 8, bias_max=40.0, experts=2, top=2, ff=8)], 40, 64, 32),                 # no key sharing; every expert used
    ([L(8, 1, 12, 28, bias_max=17.0, experts=7, top=3, ff=20, limit=0.3)], 56, 77, 6),    # one shared key head, value wider than key
    ([L(3, 3, 36, 4, bias_max=9.0), L(3, 1, 4, 36, bias_max=90.0, experts=5, top=1, ff=72)], 48, 200, 14),
    ([L(16, 4, 32, 32, bias_max=64.0, experts=9, top=4, ff=96)], 128, 300, 16),
])
def test_other_sizes(tmp_path, layers, width, vocab, rows):
    d, cfg, t = make(tmp_path, layers, width=width, vocab=vocab, seed=10, rel_rows=rows, eps=1e-6, embed_scale=1.5)
    toks = tokens(vocab, 75, 10)
    ref = R.forward(cfg, t, toks)
    m = arch.load_model(d, dtype="float32", max_batch=32, n_ctx=80)
    check(run(m, toks), ref, "float32", "portions of 32")
    check(run(m, toks, [2, 31, 1]), ref, "float32", "ragged portions")
    m.close()
    m = arch.load_model(d, dtype="bfloat16", max_batch=80, n_ctx=80)
    check(run(m, toks), ref, "bfloat16", "whole prompt")
    m.close()


# ------------------------------------------------------------------------------------------------- entry points
def test_greedy_generation_through_the_entry_points(tmp_path):
    d, cfg, t = make(tmp_path, MIXED, width=72, vocab=130, seed=11, rel_rows=10)
    prompt = tokens(130, 21, 11)
    m = arch.load_model(d, dtype="float32", max_batch=8, n_ctx=64)
    ids, lg = m.generate(prompt, 12, batch_size=8)                  # prefill in portions + one forward per token
    m.reset()
    m.prefill(prompt, 8)
    ids2 = [int(v) for v in m.decode_greedy(prompt[-1], 12)]        # the device-side greedy loop
    assert ids == ids2
    assert m.position == len(prompt) - 1 + 12
    # the oracle agrees with every pick wherever its own margin is not a rounding matter
    seq = list(prompt)
    for step, tok in enumerate(ids):
        ref = R.forward(cfg, t, seq)[-1]
        assert rel_err(lg[step][None], ref[None]).max() < 4e-5
        assert ref[tok] >= ref.max() - 1e-4 * np.abs(ref).max()
        seq.append(tok)
    # device-side top-k of the last logits row
    m.forward_lazy([seq[-1]])
    vals, idx = m.sample_topk(5)
    full = R.forward(cfg, t, seq)[-1]
    assert list(idx) == [int(v) for v in np.argsort(-full, kind="stable")[:5]]
    m.close()


def test_llama_only_entry_points_refuse_a_layer_list_context(tmp_path):
    d, cfg, t = make(tmp_path, [L(2, 1, 8, 8, bias_max=9.0)], seed=12)
    m = arch.load_model(d, dtype="float32", max_batch=8, n_ctx=16)
    with pytest.raises(capi.PsCudaError):
        m.forward_tree([1, 2], [0, 1])
    with pytest.raises(capi.PsCudaError):
        m.forward_sessions([0], [1])
    with pytest.raises(capi.PsCudaError):
        m.forward(tokens(96, 9))                                    # wider than the batch cap
    with pytest.raises(capi.PsCudaError):
        m.forward([96])                                             # outside the vocabulary
    m.forward(tokens(96, 8))
    m.forward(tokens(96, 8))
    with pytest.raises(capi.PsCudaError):
        m.forward([1])                                              # the cache is full
    m.close()


def test_trace_runner_replays_steps(tmp_path):
    d, cfg, t = make(tmp_path, MIXED, width=72, vocab=130, seed=13, rel_rows=10)
    a, b = tokens(130, 40, 30), tokens(130, 17, 31)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:32], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[32:], "want": [7, 3]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "b", "tokens": b, "want": [16]}], "end": ["b"]}]
    out = tmp_path / "out"
    for dtype in ("float32", "bfloat16"):
        p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out), "--max-tokens", "40", "--max-batch", "16"],
                           input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
        ra, rb = R.forward(cfg, t, a), R.forward(cfg, t, b)
        check(np.fromfile(out / "0.f32", "<f4").reshape(2, 130), ra[[0, 29]], dtype, "step 0")
        assert not (out / "1.f32").exists()
        check(np.fromfile(out / "2.f32", "<f4").reshape(2, 130), ra[[39, 35]], dtype, "step 2 (order of `want`)")
        check(np.fromfile(out / "3.f32", "<f4").reshape(1, 130), rb[[16]], dtype, "step 3")
        for f in out.iterdir():
            f.unlink()


def test_generation_command_line(tmp_path):
    """bin/ps_generate on a layer-list directory: greedy ids equal the model's own generate(); top-k sampling stays inside the k best"""
    d, cfg, t = make(tmp_path, MIXED, width=72, vocab=130, seed=16, rel_rows=10)
    prompt = tokens(130, 19, 16)
    exe = os.path.join(ROOT, "bin", "ps_generate")
    p = subprocess.run([exe, "--model", d, "--dtype", "float32", "--ids", " ".join(map(str, prompt)), "--n", "10", "--prefill-batch", "8"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    ids = json.loads(p.stdout.strip().splitlines()[-1])["ids"]
    m = arch.load_model(d, dtype="float32", max_batch=32, n_ctx=32)
    want, _ = m.generate(prompt, 10, batch_size=8)
    assert ids == want
    p = subprocess.run([exe, "--model", d, "--dtype", "float32", "--ids", ",".join(map(str, prompt)), "--n", "6", "--top-k", "3", "--seed", "5"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    sampled = json.loads(p.stdout.strip().splitlines()[-1])["ids"]
    seq = list(prompt)
    for tok in sampled:
        m.reset()
        lg = m.forward(seq)[-1]
        assert tok in np.argsort(-lg, kind="stable")[:3]
        seq.append(tok)
    m.close()
    assert subprocess.run([exe, "--model", d, "--ids", "", "--n", "3"], capture_output=True, text=True, timeout=600).returncode == 2
