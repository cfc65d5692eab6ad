"""bench.py --arch nufusun: prefill and decode throughput of the Nufusun design at layer sizes that resemble real models
(random weights), beside the closest existing model of the framework - a llama stack (Q4_K) with the same width, head
geometry, layer count, vocabulary and as many ACTIVE feed-forward rows per token (ffn = top_k x expert ff).

Timing: the backend's CUDA events around every forward / decode call (counter last_device_ns), warm-up first; the weights
of every size exceed the 126 MB L2, so consecutive steps do not find them cached.  One JSON line per run.
"""
from __future__ import annotations

import json
import os
import shutil
import tempfile
import time

import numpy as np

from . import arch, arch_synth, capi, gguf, synth

# name: (width, heads, kv_heads, head size, experts, top, expert ff, layers, vocab)
SIZES = {
    "s": (1024, 16, 4, 64, 8, 2, 1024, 4, 32000),
    "m": (2048, 16, 4, 128, 8, 2, 2816, 4, 32000),
    "l": (4096, 32, 8, 128, 8, 2, 7168, 2, 32000),
}


def _peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def _timed_prefill(model, prompt, chunk):
    model.reset()
    ns = 0
    for lo in range(0, len(prompt), chunk):
        model.forward(prompt[lo:lo + chunk], lm_head=False)
        ns += model.be.counter("last_device_ns")
    return ns / 1e9


def _timed_decode(model, tok, steps, warmup):
    model.decode_greedy(tok, warmup)
    model.decode_greedy(tok, steps)
    return model.be.counter("last_device_ns") / 1e9 / steps


def run_size(name, prompt_len, steps, warmup, seed, chunk):
    W, H, G, hs, E, top, ff, nl, V = SIZES[name]
    hbm, tflops, src = _peaks()
    n_ctx = -(-(prompt_len + steps + warmup + 8) // 256) * 256
    prompt = [int(v) for v in np.random.default_rng(1234).integers(0, V, prompt_len)]
    out = {"size": name, "width": W, "heads": [H, G], "head_size": hs, "experts": [E, top, ff], "layers": nl, "vocab": V, "context": prompt_len}

    # ---- Nufusun
    cfg = arch_synth.nufusun_config(W, V, [arch_synth.nufusun_layer(H, G, hs, hs, bias_max=float(prompt_len), experts=E, top=top, ff=ff, limit=7.0) for _ in range(nl)])
    d = tempfile.mkdtemp(prefix="ps_nufusun_")
    try:
        arch_synth.write_model_dir(d, cfg, arch_synth.nufusun_weights(cfg, seed=seed, rel_rows=32, fast=True))
        m = arch.load_model(d, dtype="bfloat16", max_batch=chunk, n_ctx=n_ctx)
    finally:
        shutil.rmtree(d, ignore_errors=True)
    for _ in range(2):
        t_pre = _timed_prefill(m, prompt, chunk)
    l0 = m.be.counter("kernel_launches")
    t_dec = _timed_decode(m, prompt[-1], steps, warmup)
    launches = m.be.counter("kernel_launches") - l0
    t0 = time.perf_counter()
    tok = prompt[-1]
    for _ in range(16):
        tok = int(np.argmax(m.forward([tok])[0]))
    e2e = 16 / (time.perf_counter() - t0)
    m.close()
    qkv = (H + 2 * G) * hs * W
    act_params = nl * (qkv + H * hs * W + E * W + top * 3 * ff * W) + V * W
    kv_bytes = nl * 2 * G * hs * 4 * prompt_len
    attn_flops = nl * 2 * 2 * H * hs * prompt_len / 2                     # per token, averaged over a causal prompt
    out["nufusun"] = {
        "prefill_tok_s": prompt_len / t_pre, "prefill_chunk": chunk,
        "prefill_tflops": (2 * act_params + attn_flops) * prompt_len / t_pre / 1e12,
        "prefill_frac_of_bf16_peak": (2 * act_params + attn_flops) * prompt_len / t_pre / 1e12 / tflops,
        "decode_tok_s": 1 / t_dec, "decode_ms": t_dec * 1e3, "decode_launches_per_step": launches / (steps + warmup),
        "decode_bytes_per_token": 2 * act_params + kv_bytes, "decode_frac_of_hbm_peak": (2 * act_params + kv_bytes) / t_dec / 1e9 / hbm,
        "e2e_decode_tok_s": e2e}

    # ---- the closest existing model: llama, Q4_K, ffn = top x ff
    shape = synth.ModelShape(f"llama-like-{name}", "llama", W, top * ff, nl, H, G, hs, V, False, 0, 5e5, 1e-5, gguf.GGML_Q4_K, n_ctx=n_ctx)
    tensors = synth.generate_tensors(shape, seed)
    tmap = {n: gguf.GGUFTensor(n, t, tuple(s), np.ascontiguousarray(dd).view(np.uint8).reshape(-1)) for n, t, s, dd in tensors}
    lm = capi.CudaModel(desc=capi.desc_from_model_json(synth.model_json(shape), max_batch=128, n_ctx=n_ctx), tensors=tmap)
    for _ in range(2):
        t_pre_l = _timed_prefill(lm, prompt, 128)
    t_dec_l = _timed_decode(lm, prompt[-1], steps, warmup)
    lm.close()
    l_params = nl * (qkv + H * hs * W + 3 * top * ff * W) + V * W
    l_bytes = l_params * 0.5625 + kv_bytes
    out["llama_q4k"] = {
        "prefill_tok_s": prompt_len / t_pre_l, "prefill_chunk": 128,
        "prefill_tflops": (2 * l_params + attn_flops) * prompt_len / t_pre_l / 1e12,
        "prefill_frac_of_bf16_peak": (2 * l_params + attn_flops) * prompt_len / t_pre_l / 1e12 / tflops,
        "decode_tok_s": 1 / t_dec_l, "decode_ms": t_dec_l * 1e3,
        "decode_bytes_per_token": l_bytes, "decode_frac_of_hbm_peak": l_bytes / t_dec_l / 1e9 / hbm}
    out["peaks"] = {"hbm_gbs": hbm, "bf16_tflops": tflops, "source": src}
    return out


def main(args) -> int:
    if capi.load_library().ps_cuda_device_count() == 0:
        print(json.dumps({"arch": "nufusun", "unavailable": "no CUDA device: there is no CPU fallback"}))
        return 1
    sizes = [s for s in args.arch_sizes.split(",") if s]
    res = [run_size(s, args.arch_prompt, max(args.steps, 8), max(args.warmup, 3), args.seed, args.arch_chunk) for s in sizes]
    print(json.dumps({"arch": "nufusun", "dtype": "bf16", "data": "synthetic", "timing": "CUDA events around every call, warm-up first; weights exceed L2",
                      "sizes": res}))
    return 0
