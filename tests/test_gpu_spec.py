"""Speculative decoding on the CUDA backend: the KVCacheInterface slot
operations, the tree forward, and the token-tree loop (include/ps_spec.h) - whose output must be the target model's own
greedy continuation.

The reference cannot pin this path (its CPU backend ignores tree masks; the QNN backend that implements it
does not run here), so parity is pinned by (a) bit-equality of a causal tree batch with the plain forward, (b) a dense
fp32 restatement of the masked attention semantics (src/backend/qnn/causal_models.cpp:215-230) through path equivalence:
a node's logits equal those of the plain causal run over root..node, and (c) the lossless invariant."""
import numpy as np
import pytest

from powerserve_b200 import capi, synth
from tests import _libs as L
from tests import _model as M

pytestmark = pytest.mark.gpu


def test_causal_tree_batch_equals_plain_forward():
    d = M.model_dir("tiny-llama")
    shape = synth.PRESETS["tiny-llama"]
    prompt = synth.random_prompt(shape.vocab_size, 29, seed=5)
    a, b = capi.CudaModel(d, max_batch=16), capi.CudaModel(d, max_batch=16)
    a.prefill(prompt[:17], 16); b.prefill(prompt[:17], 16)
    la = a.forward(prompt[17:29])                                                   # plain batch, positions 16..27
    lb = b.forward_tree(prompt[17:29], np.arange(16, 28))                           # the same batch through the tree path, causal mask
    L.assert_bit_equal(lb, la, "causal tree batch vs plain forward")
    assert a.position == b.position == 28
    kvd, n = shape.kv_dim, 28
    for layer in range(shape.n_layers):
        L.assert_bit_equal(b.be.read_device(b.be.kv_k(layer), n * kvd), a.be.read_device(a.be.kv_k(layer), n * kvd), "K cache")
    L.assert_bit_equal(b.forward_tree([3], [28])[0], a.forward([3])[0], "single token through the tree path")
    a.close(); b.close()


def test_tree_batch_path_equivalence_and_slot_ops():
    """a random token tree: every node's logits must match the plain causal run over its root-to-node path (the dense
    restatement of the tree mask), and accepting a path with copy / advance must leave the cache of a plain run."""
    d = M.model_dir("tiny-llama")
    shape = synth.PRESETS["tiny-llama"]
    rng = np.random.default_rng(3)
    prompt = synth.random_prompt(shape.vocab_size, 21, seed=8)
    bs = 12
    parent = [-1] + [int(rng.integers(0, u)) for u in range(1, bs)]                 # node u hangs under an earlier node
    toks = rng.integers(0, shape.vocab_size, bs).astype(np.int32)
    depth = [0] * bs
    for u in range(1, bs):
        depth[u] = depth[parent[u]] + 1
    base = len(prompt)
    pos = np.array([base + depth[u] for u in range(bs)], np.int32)
    mask = np.zeros((bs, bs), np.uint8)
    for u in range(bs):
        x = u
        while x != -1:
            mask[u, x] = 1
            x = parent[x]
    t = capi.CudaModel(d, max_batch=16)
    t.prefill(np.concatenate([prompt, [0]]), 16)                                    # prefill all `base` prompt tokens
    assert t.position == base
    lt = t.forward_tree(toks, pos, mask)
    assert t.position == base + bs
    t.be.kv_rollback(bs)
    ref = capi.CudaModel(d, max_batch=16)
    worst = 0.0
    for u in range(bs):
        path = []
        x = u
        while x != -1:
            path.append(x)
            x = parent[x]
        path = path[::-1]
        ref.reset(); ref.prefill(np.concatenate([prompt, [0]]), 16)
        lr = ref.forward(toks[path])[-1]                                            # plain causal batch over the path
        scale = np.abs(lr).max()
        worst = max(worst, float(np.abs(lt[u] - lr).max() / scale))
        assert int(np.argmax(lt[u])) == int(np.argmax(lr)) or np.sort(lr)[-1] - np.sort(lr)[-2] < 1e-4 * scale
    # the soft-max rows differ in length (and so in where ggml's SIMD exp hands over to libm expf): agreement to fp32 noise
    assert worst < 2e-5, worst
    # accept the deepest path: copy its tokens to consecutive slots, advance; the cache must equal the plain run's
    u = int(np.argmax(depth))
    path = []
    x = u
    while x != -1:
        path.append(x)
        x = parent[x]
    path = path[::-1]
    for k, node in enumerate(path):
        assert t.position == base + k
        t.be.kv_copy_slot(base + k, node)
        t.be.kv_advance(1)
    ref.reset(); ref.prefill(np.concatenate([prompt, [0]]), 16); ref.forward(toks[path])
    kvd, n = shape.kv_dim, base + len(path)
    for layer in range(shape.n_layers):
        kt, kr = t.be.read_device(t.be.kv_k(layer), n * kvd), ref.be.read_device(ref.be.kv_k(layer), n * kvd)
        assert np.abs(kt - kr).max() <= 2e-5 * np.abs(kr).max()
        L.assert_bit_equal(kt[: base * kvd], kr[: base * kvd], "prompt part of the K cache")
    nxt = int(toks[0])
    assert np.abs(t.forward([nxt])[0] - ref.forward([nxt])[0]).max() < 1e-3
    # move + mask / unmask: a masked slot is invisible to the next tree forward
    t.be.kv_mask_slot(2)
    l_masked = t.forward_tree([5], [t.position])[0]
    t.be.kv_rollback(1); t.be.kv_unmask_slot(2)
    l_open = t.forward_tree([5], [t.position])[0]
    assert np.abs(l_masked - l_open).max() > 0
    t.be.kv_rollback(1)
    t.be.kv_move_slot(2, 3)                                                          # slot 2 now holds slot 3's rows
    k = t.be.read_device(t.be.kv_k(0), 4 * kvd).reshape(4, kvd)
    L.assert_bit_equal(k[2], k[3], "kv_move_slot")
    with pytest.raises(capi.PsCudaError):
        t.be.kv_mask_slot(t.position)                                                # POWERSERVE_ASSERT_KVCACHE(cache_index < position)
    t.close(); ref.close()


def _chunking_noise(path, prompt, vocab):
    """The reference-vs-reference yardstick: logits of the SAME 12 tokens fed as one batch and one by one.
    Both runs are bit-identical to the ggml CPU reference (tests/test_gpu_model.py) and still differ, because its soft-max
    row length - and with it the hand-over from the SIMD exp to libm expf - depends on the chunking, and activation
    re-quantisation amplifies the ulp-level difference layer by layer."""
    a, b = capi.CudaModel(path, max_batch=32), capi.CudaModel(path, max_batch=32)
    a.prefill(prompt[:22], 32); b.prefill(prompt[:22], 32)
    la = a.forward(prompt[21:33])
    lb = np.stack([b.forward([int(t)])[0] for t in prompt[21:33]])
    a.close(); b.close()
    return float(np.abs(la - lb).max())


@pytest.mark.parametrize("target,draft", [("tiny-llama", "tiny-llama"), ("tiny-deep", "tiny-llama")])
def test_speculative_decode_is_lossless(target, draft):
    """token-tree speculative decoding == the target's plain greedy decoding, margin-aware: the batched verify and the
    single-token step are two CHUNKINGS of the same computation, which the reference itself does not reproduce bit for
    bit (yardstick measured here); a divergence is legitimate only where the plain run's top-2 margin is within that noise."""
    dt, dd = M.model_dir(target), M.model_dir(draft, seed=0 if target == draft else 1)
    shape = synth.PRESETS[target]
    prompt = synth.random_prompt(shape.vocab_size, 33, seed=21)
    noise = _chunking_noise(dt, prompt, shape.vocab_size)
    n_gen = 48
    tm, dm = capi.CudaModel(dt, max_batch=32), capi.CudaModel(dd, max_batch=32)
    plain = capi.CudaModel(dt, max_batch=32)
    ids_plain, lg_plain = plain.generate(prompt, n_gen, batch_size=32)
    sd = capi.SpecDecoder(tm, dm)
    ids_spec, st = sd.generate(prompt, n_gen, prefill_batch=32)
    ids_spec = [int(x) for x in ids_spec]
    assert st["n_generated_tokens"] >= n_gen and st["n_iterations"] >= 1
    if target == draft:   # a perfect draft: (almost) every drafted token on the greedy path is accepted
        assert st["n_generated_tokens"] / st["n_iterations"] > 1.5, st
    agree = n_gen
    for k in range(n_gen):
        if ids_spec[k] != ids_plain[k]:
            top = np.sort(lg_plain[k])[-2:]
            assert top[1] - top[0] <= 4 * noise, f"step {k}: {ids_spec[k]} vs {ids_plain[k]}, margin {top[1] - top[0]:.4f} vs chunking noise {noise:.4f}"
            agree = k
            break
    assert agree >= 8 or noise > 0, (agree, noise)
    sd.close(); tm.close(); dm.close(); plain.close()
