"""Layer-list models (config.json + model.safetensors) on the CUDA backend, and the model registry.

`load_model(path)` is how every front end (bin/trace_run, the generation command line, bench.py, tests) gets a model: a
PowerServe model directory (model.json + ggml/weights.gguf) becomes a `capi.CudaModel`, a directory with a config.json
becomes the class its "architecture" names in `ARCHITECTURES`.  Both are the same kind of object - a bound ps_cuda
context with forward / prefill / generate / decode_greedy / sample_topk / sessions.

A design registers a function that turns its config.json into the backend's layer descriptions (include/ps_cuda.h,
"layer-list models") and one that names its tensors; the constants a design fixes live in that function, everything a
config file may vary is read from the file.
"""
from __future__ import annotations

import ctypes as C
import json
import os
from typing import Callable, Dict, List, Optional, Tuple

from . import capi, safetensors
from .capi import ArchDesc, ArchLayerWeights, ArchWeights, LayerDesc, Tensor


class LayerListModel(capi.CudaModel):
    """A layer-list model bound through ps_cuda_create_arch / ps_cuda_bind_arch.  Everything after construction is
    capi.CudaModel's: the context behaves like a llama context behind the shared entry points."""

    def __init__(self, path: str, *, dtype: str = "bfloat16", max_batch: int = 128, n_ctx: int = 4096, device: int = 0):
        cfg = json.load(open(os.path.join(path, "config.json")))
        name = cfg.get("architecture")
        if name not in ARCHITECTURES:
            raise capi.PsCudaError(f"{path}: unknown architecture {name!r} (known: {sorted(ARCHITECTURES)})")
        describe, tensor_names = ARCHITECTURES[name]
        self.cfg = cfg
        self._file = safetensors.SafeTensorsFile(os.path.join(path, "model.safetensors"))
        self.tensors = self._file.tensors
        compute = {"bfloat16": capi.COMPUTE_BF16, "float32": capi.COMPUTE_F32}[dtype]
        layers, top = describe(cfg, self.tensors)
        self._layer_descs = (LayerDesc * len(layers))(*layers)
        self.desc = ArchDesc(top["dim"], top["vocab_size"], len(layers), int(n_ctx), int(max_batch), top["norm_eps"], top["embed_scale"],
                             top["norm_unit_offset"], compute, self._layer_descs, int(top.get("norm_groups", 1)))
        self.vocab = self.desc.vocab_size
        self.be = capi.CudaBackend(self.desc, device)

        def T(n: Optional[str]) -> Tensor:
            if n is None:
                return Tensor(None, 0, 0)
            if n not in self.tensors:
                raise capi.PsCudaError(f"{path}: tensor {n} is missing")
            t = self.tensors[n]
            return Tensor(t.host_ptr, t.ps_type, 0)

        names = tensor_names(cfg)
        self._keep: List[object] = []
        self._lw = (ArchLayerWeights * len(layers))()
        for i, ln in enumerate(names["layers"]):
            lw = ArchLayerWeights()
            for f in ("norm", "q", "q_bias", "k", "k_bias", "v", "v_bias", "o", "o_bias", "rel", "head_mix", "head_temp", "router") + capi.ARCH_LAYER_VECTORS_2:
                setattr(lw, f, T(ln.get(f)))
            for f in ("gate", "up", "down"):
                lst = ln.get(f)
                if lst:
                    arr = (Tensor * len(lst))(*[T(n) for n in lst])
                    self._keep.append(arr)
                    setattr(lw, f, arr)
            self._lw[i] = lw
        self._w = ArchWeights(T(names["embed"]), T(names["final_norm"]), T(names["head"]), self._lw)
        self.be._ck(self.be.L.ps_cuda_bind_arch(self.be.h, C.byref(self._w)))

    def layer_tap(self, layer: int, bs: int):
        """residual stream after `layer` of the last forward pass (option arch_taps)"""
        import numpy as np
        out = np.empty((bs, self.desc.dim), np.float32)
        self.be._ck(self.be.L.ps_cuda_arch_tap(self.be.h, layer, out.ctypes.data, bs))
        return out


# ------------------------------------------------------------------------------------------------------------ Nufusun
# Decoder-only; every layer is a parallel block (one unit-offset RMS norm feeds the mixer AND the feed-forward).  Mixer:
# grouped-query attention without rotation, projection biases, per-head temperature, a bucketed distance bias, head mixing
# before the soft-max, a value-less sink in the denominator.  Feed-forward: sigmoid-routed experts whose score scales the
# expert's input, scores not renormalised; expert activation g * sigmoid(1.702 g) * (u + 1) on clamped g, u.
def _nufusun_describe(cfg: dict, tensors) -> Tuple[List[LayerDesc], dict]:
    layers = []
    for i, l in enumerate(cfg["layers"]):
        if l["type"] != "attention":
            raise capi.PsCudaError(f"Nufusun layer {i}: unknown mixer type {l['type']!r}")
        m = l["mixer"]
        d = LayerDesc()
        d.mixer_kind = capi.MIXER_ATTENTION
        d.n_heads, d.n_kv_heads, d.qk_dim, d.v_dim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        d.score_scale = m["scale"]
        d.proj_bias, d.head_temp, d.head_mix, d.sink = 1, 1, 1, 1
        d.rel_buckets = int(tensors[f"l{i}.mix.rel"].shape[0])      # the table's own row count
        d.rel_max_dist = m["bias_max"]
        mlp = l.get("mlp")
        if mlp is None:
            d.mlp_kind = capi.MLP_NONE
        elif mlp.get("kind") == "moe":
            d.mlp_kind = capi.MLP_ROUTED
            d.n_experts, d.top_k = mlp["router"]["experts"], mlp["router"]["top"]
            d.expert_ff, d.act_limit = mlp["expert"]["ff"], mlp["expert"]["limit"]
            d.router_act, d.route_on_input, d.route_renorm = 1, 1, 0
            d.act_alpha, d.up_shift = 1.702, 1.0
        else:
            raise capi.PsCudaError(f"Nufusun layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        layers.append(d)
    top = {"dim": cfg["width"], "vocab_size": cfg["vocab"], "norm_eps": cfg["norm"]["eps"], "embed_scale": cfg["embedding"]["scale"],
           "norm_unit_offset": 1}
    return layers, top


def _nufusun_tensor_names(cfg: dict) -> dict:
    out = {"embed": "embed", "final_norm": "final.norm", "head": "head", "layers": []}
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        n = {"norm": p + "norm1", "q": p + "mix.q", "q_bias": p + "mix.q.b", "k": p + "mix.k", "k_bias": p + "mix.k.b", "v": p + "mix.v",
             "v_bias": p + "mix.v.b", "o": p + "mix.o", "o_bias": p + "mix.o.b", "rel": p + "mix.rel", "head_mix": p + "mix.talk",
             "head_temp": p + "mix.temp"}
        if l.get("mlp") is not None:
            E = l["mlp"]["router"]["experts"]
            n["router"] = p + "mlp.router"
            for f in ("gate", "up", "down"):
                n[f] = [f"{p}mlp.e{e}.{f}" for e in range(E)]
        out["layers"].append(n)
    return out


# ------------------------------------------------------------------------------------------------------------ Vanapel
# Decoder-only; every layer is a sequential block whose sublayers are normed on the way in AND on the way out,
#   x <- x + N1b(mixer(N1(x))),  x <- x + N2b(ff(N2(x))),
# with RMS norms taken over `norm.groups` equal parts of the vector.  Two mixers, chosen per layer by "type":
#   "attention"         grouped-query, no rotation and no biases; q and k of every head scaled to unit RMS; the score loses
#                       r1_h ln(1 + r2_h (i - j)) with distance; a sliding window of mask.size keys; a learned per-head sink
#                       logit in the soft-max denominator; layers marked v_mix blend their values with those of the FIRST marked
#                       layer (weight '.vmix'; the first one's own is unused).
#   "latent_attention"  queries through a normed latent, keys / values up-projected from a shared normed latent plus one
#                       rotated key part common to all heads (rotate-half pairs, YaRN-scaled frequencies); causal; learned sink.
# Feed-forward: one gated unit, y = g sigmoid(1.702 g) (u + 1) on g = min(gate, limit), u = clamp(up, +-limit).
def _vanapel_describe(cfg: dict, tensors) -> Tuple[List[LayerDesc], dict]:
    layers = []
    v_source_seen = False
    for i, l in enumerate(cfg["layers"]):
        m = l["mixer"]
        d = LayerDesc()
        d.block_kind, d.post_norm = capi.BLOCK_SEQUENTIAL, 1
        d.n_heads, d.qk_dim, d.v_dim = m["heads"], m["dim"], m["vdim"]
        d.score_scale = m["scale"]
        d.sink = capi.SINK_LEARNED
        if l["type"] == "attention":
            d.mixer_kind = capi.MIXER_ATTENTION
            d.n_kv_heads = m["kv_heads"]
            d.qk_norm, d.log_bias = 1, 1
            d.window = int((m.get("mask") or {}).get("size", 0))
            if m.get("v_mix"):
                d.v_mix = capi.VMIX_BLEND if v_source_seen else capi.VMIX_SOURCE
                v_source_seen = True
        elif l["type"] == "latent_attention":
            d.mixer_kind = capi.MIXER_LATENT
            d.n_kv_heads = 1
            d.q_rank, d.kv_rank, d.rot_dim = m["q_rank"], m["kv_rank"], m["rot_dim"]
            rot = m.get("rot") or {}
            d.rope_dims, d.rope_base = int(rot.get("dims", d.rot_dim)), float(rot.get("base", 10000.0))
            sc = rot.get("scaling")
            if sc:
                d.rope_factor, d.rope_original, d.rope_fast, d.rope_slow = float(sc["factor"]), int(sc["original"]), float(sc["fast"]), float(sc["slow"])
            d.window = int((m.get("mask") or {}).get("size", 0))
        else:
            raise capi.PsCudaError(f"Vanapel layer {i}: unknown mixer type {l['type']!r}")
        mlp = l.get("mlp")
        if mlp is None:
            d.mlp_kind = capi.MLP_NONE
        elif mlp.get("kind") == "dense":
            d.mlp_kind = capi.MLP_DENSE
            d.expert_ff, d.act_limit = mlp["ff"], mlp["limit"]
            d.act_alpha, d.up_shift = 1.702, 1.0
        else:
            raise capi.PsCudaError(f"Vanapel layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        layers.append(d)
    top = {"dim": cfg["width"], "vocab_size": cfg["vocab"], "norm_eps": cfg["norm"]["eps"], "embed_scale": 1.0, "norm_unit_offset": 0,
           "norm_groups": int(cfg["norm"].get("groups", 1))}
    return layers, top


def _vanapel_tensor_names(cfg: dict) -> dict:
    out = {"embed": "embed", "final_norm": "final.norm", "head": "head", "layers": []}
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        n = {"norm": p + "norm1", "norm_mix_out": p + "norm1b", "o": p + "mix.o", "sink": p + "mix.sink"}
        if l["type"] == "attention":
            n.update({"q": p + "mix.q", "k": p + "mix.k", "v": p + "mix.v", "r1": p + "mix.r1", "r2": p + "mix.r2"})
            if l["mixer"].get("v_mix"):
                n["vmix"] = p + "mix.vmix"
        else:
            n.update({"dq": p + "mix.dq", "dq_norm": p + "mix.dq.norm", "uq": p + "mix.uq", "dkv": p + "mix.dkv", "dkv_norm": p + "mix.dkv.norm",
                      "uk": p + "mix.uk", "uv": p + "mix.uv"})
        if l.get("mlp") is not None:
            n.update({"norm_ff": p + "norm2", "norm_ff_out": p + "norm2b"})
            for f in ("gate", "up", "down"):
                n[f] = [f"{p}mlp.{f}"]
        out["layers"].append(n)
    return out


ARCHITECTURES: Dict[str, Tuple[Callable, Callable]] = {
    "Nufusun": (_nufusun_describe, _nufusun_tensor_names),
    "Vanapel": (_vanapel_describe, _vanapel_tensor_names),
}


def load_model(path: str, *, dtype: str = "bfloat16", max_batch: int = 128, n_ctx: Optional[int] = None, device: int = 0):
    """The model class is chosen by what the directory holds."""
    if os.path.exists(os.path.join(path, "model.json")):
        if dtype != "bfloat16" and dtype != "native":
            raise capi.PsCudaError("GGUF models run in their stored quantised formats; --dtype does not apply")
        return capi.CudaModel(path, max_batch=max_batch, device=device)
    if os.path.exists(os.path.join(path, "config.json")):
        return LayerListModel(path, dtype=dtype, max_batch=max_batch, n_ctx=n_ctx or 4096, device=device)
    raise capi.PsCudaError(f"{path}: neither model.json (PowerServe / GGUF) nor config.json (layer list) found")
