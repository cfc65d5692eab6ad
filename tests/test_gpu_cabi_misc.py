"""GPU tests of the C-ABI entries the first suite did not touch: ps_cuda_copy_2d (the `copy` / `cont` twin), the KV
position bookkeeping (truncate / advance / rollback, kv_cache.hpp:97-163 semantics), the exposed cache pointers
(ps_cuda_kv_k / ps_cuda_kv_v against the oracle's cache contents) and ps_cuda_logits_dev."""
import numpy as np
import pytest

from powerserve_b200 import capi, synth
from tests import _libs as L
from tests import _model as M

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    b = capi.CudaBackend(capi.ModelDesc(512, 1536, 1, 8, 2, 64, 1024, 512, 1e-5, 64, 0, 5e5, 1.0, 1.0, 0, 32, 0, 1))
    yield b
    b.close()


@pytest.mark.parametrize("ne0,ne1", [(64, 8), (37, 5), (1, 129), (128, 1)])
def test_copy_2d_strided(be, ne0, ne1):
    rng = np.random.default_rng(ne0 * 131 + ne1)
    # (a) the V-cache store of NormAttention::build: contiguous {ne0, ne1} source -> transposed destination with row pitch n_ctx
    n_ctx = 160
    src = rng.standard_normal(ne0 * ne1).astype(np.float32)
    dst0 = rng.standard_normal(n_ctx * ne0).astype(np.float32)
    sd, dd = be.upload(src), be.upload(dst0)
    be.copy_2d(dd, 4 * n_ctx, 4, sd, 4, 4 * ne0, ne0, ne1)          # dst[i0][i1] (pitch n_ctx) = src[i1][i0]
    want = dst0.reshape(ne0, n_ctx).copy()
    want[:, :ne1] = src.reshape(ne1, ne0).T
    L.assert_bit_equal(dd.numpy(), want.reshape(-1), "transposed strided store")
    # (b) `cont` of a permuted view: {ne0, ne1} read with swapped strides into a contiguous buffer
    cd = be.empty(ne0 * ne1)
    be.copy_2d(cd, 4, 4 * ne1, sd, 4 * ne0, 4, ne1, ne0)           # dst[j][i] contiguous in i = src[i][j]
    L.assert_bit_equal(cd.numpy(), src.reshape(ne1, ne0).T.reshape(-1), "cont of a permuted view")
    for b in (sd, dd, cd):
        b.free()


def test_copy_4d_views_of_the_unfused_graph(be):
    """The three dup shapes of NormAttention::build (norm_attention.cpp:82-151): rope_k {hs, n_kv_heads, bs} into the 1-D cache
    view at an offset, the transposed v into the {bs, kv_dim} view of the transposed cache, and `cont` of the permuted
    {hs, n_heads, bs} view of the P.V product into {dim, bs}."""
    rng = np.random.default_rng(11)
    hs, nkv, nh, bs, n_ctx, pos = 64, 2, 8, 5, 96, 17
    kvd, dim = hs * nkv, hs * nh
    k = rng.standard_normal(kvd * bs).astype(np.float32)
    cache0 = rng.standard_normal(n_ctx * kvd).astype(np.float32)
    kd, cd = be.upload(k), be.upload(cache0)
    be.copy_4d(cd, [bs * kvd, 1, 1, 1], [4, 4 * bs * kvd, 4 * bs * kvd, 4 * bs * kvd], kd, [hs, nkv, bs, 1], [4, 4 * hs, 4 * kvd, 4 * kvd * bs], dst_off=4 * kvd * pos)
    want = cache0.copy()
    want[kvd * pos: kvd * (pos + bs)] = k
    L.assert_bit_equal(cd.numpy(), want, "k rows into the cache view")
    # v {kv_dim, bs} seen transposed as {bs, kv_dim} (strides swapped) -> cache^T view {bs, kv_dim} with row pitch n_ctx
    v = rng.standard_normal(kvd * bs).astype(np.float32)
    vt0 = rng.standard_normal(kvd * n_ctx).astype(np.float32)
    vd, vtd = be.upload(v), be.upload(vt0)
    be.copy_4d(vtd, [bs, kvd, 1, 1], [4, 4 * n_ctx, 4 * n_ctx * kvd, 4 * n_ctx * kvd], vd, [bs, kvd, 1, 1], [4 * kvd, 4, 4 * kvd * bs, 4 * kvd * bs], dst_off=4 * pos)
    want = vt0.reshape(kvd, n_ctx).copy()
    want[:, pos:pos + bs] = v.reshape(bs, kvd).T
    L.assert_bit_equal(vtd.numpy(), want.reshape(-1), "transposed v into the cache view")
    # kqv {hs, bs, n_heads} permuted {0, 2, 1, 3} -> view {hs, n_heads, bs} -> cont {dim, bs}
    kqv = rng.standard_normal(hs * bs * nh).astype(np.float32)
    qd, od = be.upload(kqv), be.empty(dim * bs)
    be.copy_4d(od, [dim, bs, 1, 1], [4, 4 * dim, 4 * dim * bs, 4 * dim * bs], qd, [hs, nh, bs, 1], [4, 4 * hs * bs, 4 * hs, 4 * hs * bs * nh])
    L.assert_bit_equal(od.numpy(), kqv.reshape(nh, bs, hs).transpose(1, 0, 2).reshape(-1), "cont of the permuted P.V product")
    for b in (kd, cd, vd, vtd, qd, od):
        b.free()


@pytest.mark.parametrize("hs,nkv,r2,bs,n_kv", [(64, 2, 4, 1, 1), (64, 2, 4, 3, 37), (128, 2, 2, 2, 70), (32, 1, 1, 1, 257), (96, 2, 3, 4, 33)])
def test_matmul_f32_strided_attention_products(be, hs, nkv, r2, bs, n_kv):
    """matmul with FP32 src0 over the strided views of the unfused graph: scores = k_view {hs, n_kv, n_kv_heads} . q {hs, bs, n_heads}
    (a permuted view of the rope output) and P.V = v_view {n_kv, hs, n_kv_heads} . kq {n_kv, bs, n_heads}; every output element
    must be ggml_vec_dot_f32 of its row and column (oracle: ps_or_vec_dot_f32, ggml.c:2092-2131)."""
    o = L.oracle()
    rng = np.random.default_rng(hs * 7 + n_kv)
    nh, kvd, n_ctx = nkv * r2, hs * nkv, 260
    kc = rng.standard_normal(n_ctx * kvd).astype(np.float32)            # [pos][kv_dim]
    q = rng.standard_normal(bs * nh * hs).astype(np.float32)            # rope output {hs, n_heads, bs}
    kcd, qd, sd = be.upload(kc), be.upload(q), be.empty(n_kv * bs * nh)
    be.matmul_f32(sd, kcd, hs, n_kv, nkv, 4 * kvd, 4 * hs, qd, bs, nh, 4 * hs * nh, 4 * hs)   # q viewed {hs, bs, n_heads}: strides (4, hs*nh*4, hs*4)
    got = sd.numpy().reshape(nh, bs, n_kv)
    K3, Q3 = kc.reshape(n_ctx, nkv, hs), q.reshape(bs, nh, hs)
    for h in range(nh):
        for i in range(bs):
            for j in range(n_kv):
                a, b = np.ascontiguousarray(K3[j, h // r2]), np.ascontiguousarray(Q3[i, h])
                assert L.bits(np.float32(o.ps_or_vec_dot_f32(hs, L.fptr(a), L.fptr(b)))) == L.bits(got[h, i, j]), (h, i, j)
    vt = rng.standard_normal(kvd * n_ctx).astype(np.float32)            # [kv_dim][n_ctx]
    p = rng.standard_normal(nh * bs * n_kv).astype(np.float32)          # {n_kv, bs, n_heads}
    vtd, pd, od = be.upload(vt), be.upload(p), be.empty(hs * bs * nh)
    be.matmul_f32(od, vtd, n_kv, hs, nkv, 4 * n_ctx, 4 * n_ctx * hs, pd, bs, nh, 4 * n_kv, 4 * n_kv * bs)
    got = od.numpy().reshape(nh, bs, hs)
    V3, P3 = vt.reshape(nkv, hs, n_ctx), p.reshape(nh, bs, n_kv)
    for h in range(nh):
        for i in range(bs):
            for d in range(hs):
                a, b = np.ascontiguousarray(V3[h // r2, d, :n_kv]), np.ascontiguousarray(P3[h, i])
                assert L.bits(np.float32(o.ps_or_vec_dot_f32(n_kv, L.fptr(a), L.fptr(b)))) == L.bits(got[h, i, d]), (h, i, d)
    for b in (kcd, qd, sd, vtd, pd, od):
        b.free()


@pytest.mark.parametrize("ne0,rows", [(1, 3), (8, 2), (37, 5), (300, 4), (4097, 1)])
def test_softmax_plain(be, ne0, rows):
    """GGMLBackend::softmax = soft_max with scale 1 and no mask (ggml.c:15060-15089); the oracle's softmax_ext with a zero mask
    computes the same rows (x * 1 + 0)."""
    o = L.oracle()
    x = (np.random.default_rng(ne0).standard_normal(ne0 * rows) * 6).astype(np.float32)
    ref = np.zeros_like(x)
    o.ps_or_softmax_ext(L.fptr(ref), L.fptr(x), L.fptr(np.zeros(ne0 * rows, np.float32)), ne0, rows, 1, 1.0)
    xd, dd = be.upload(x), be.empty(x.size)
    be.softmax(dd, xd, ne0, rows)
    L.assert_bit_equal(dd.numpy(), ref, "softmax")
    xd.free(); dd.free()


def test_kv_bookkeeping_and_cache_contents():
    d = M.model_dir("tiny-llama")
    shape = synth.PRESETS["tiny-llama"]
    prompt = synth.random_prompt(shape.vocab_size, 21, seed=3)
    cm = capi.CudaModel(d, max_batch=8)
    om = M.OracleModel(d)
    cm.prefill(prompt, 8); om.reset()
    i = 0
    while i < len(prompt) - 1:                                           # same chunking on the oracle
        bs = min(8, len(prompt) - 1 - i)
        om.forward(prompt[i:i + bs], lm_head=False)
        i += bs
    n = len(prompt) - 1
    assert cm.position == n == om.position
    kvd, n_ctx = shape.kv_dim, shape.n_ctx
    for layer in range(shape.n_layers):                                  # cache contents, layouts of ggml_kv_cache.cpp:35-58
        k = cm.be.read_device(cm.be.kv_k(layer), n * kvd)
        v = cm.be.read_device(cm.be.kv_v(layer), kvd * n_ctx).reshape(kvd, n_ctx)[:, :n]
        ko = np.ctypeslib.as_array(om.lib.ps_or_model_k_cache(om.h, layer), shape=(n_ctx * kvd,))[: n * kvd]
        vo = np.ctypeslib.as_array(om.lib.ps_or_model_v_cache(om.h, layer), shape=(kvd * n_ctx,)).reshape(kvd, n_ctx)[:, :n]
        L.assert_bit_equal(k, ko, f"K cache layer {layer}")
        L.assert_bit_equal(np.ascontiguousarray(v), np.ascontiguousarray(vo), f"V cache layer {layer}")
    assert cm.be.kv_k(shape.n_layers) is None and cm.be.kv_v(-1) is None
    # truncate_tokens (kv_cache.hpp:265-271): only ever shrinks
    cm.be.kv_truncate(n + 5); assert cm.position == n
    cm.be.kv_truncate(n - 4); assert cm.position == n - 4
    cm.be.kv_advance(4); assert cm.position == n                       # advance_tokens: the 4 slots still hold their rows
    lg_c = cm.forward([int(prompt[-1])])[0]
    lg_o = om.forward([int(prompt[-1])])[0]
    L.assert_bit_equal(lg_c, lg_o, "decode after truncate + advance")
    # ps_cuda_logits_dev: the device copy of what forward() returned
    L.assert_bit_equal(cm.be.read_device(cm.be.logits_dev(), shape.vocab_size), lg_c, "logits_dev")
    with pytest.raises(capi.PsCudaError):
        cm.be.kv_advance(n_ctx)                                          # KV full
    with pytest.raises(capi.PsCudaError):
        cm.be.kv_rollback(cm.position + 1)
    cm.close(); om.close()


@pytest.mark.parametrize("preset,k", [("tiny-llama", 1), ("tiny-llama", 40), ("tiny-bigvocab", 64), ("tiny-qwen2", 7)])
def test_device_topk_equals_host_partial_sort(preset, k):
    """ps_cuda_sample_topk = ProbArray + TopKSampler::apply (prob_array.hpp:43-49, sampler.cpp:39-56) on the device: the k largest
    logits of the last forward pass, descending, ties by ascending id - compared with a host sort of the same logits (which
    are themselves bit-exact vs the oracle in the model tests), with lazy logits (nothing but 2k words crosses PCIe)."""
    d = M.model_dir(preset)
    shape = synth.PRESETS[preset]
    cm = capi.CudaModel(d, max_batch=8)
    prompt = synth.random_prompt(shape.vocab_size, 11, seed=21)
    cm.prefill(prompt, 8)
    tok = int(prompt[-1])
    for step in range(4):
        d2h0 = cm.be.counter("d2h_bytes")
        cm.forward_lazy([tok])
        vals, ids = cm.sample_topk(k)
        assert cm.be.counter("d2h_bytes") - d2h0 == 8 * k            # the logits stayed on the device
        lg = cm.be.read_device(cm.be.logits_dev(), shape.vocab_size)
        order = np.lexsort((np.arange(shape.vocab_size), -lg.astype(np.float64)))[:k]   # logit descending, then id ascending
        assert list(ids) == [int(i) for i in order]
        L.assert_bit_equal(vals, lg[order], "top-k logits")
        tok = int(ids[0])
    # duplicate logits: ties resolve by ascending id (checked on a crafted row through the same kernels is not possible from
    # the C ABI; equal logits inside real rows are covered by the lexsort comparison above)
    cm.close()
