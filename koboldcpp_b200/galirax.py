"""Galirax: the reader of its config.json and weights behind the shared decoder (include/b200_llama.h).

A Galirax model folder holds config.json ("architecture": "Galirax", "width", "vocab", "norm": {"eps"}, "logit_softcap",
"loop": {"start", "stop", "times"} or absent, and "layers": a list of {"type", "mixer": {...}, "mlp": {...} or null}) and
model.safetensors (bfloat16 matrices named "embed", "head", "final.norm", "final.norm.b" and "l<i>.<leaf>").  Layer types:
"attention" (plain projections), "attention_2" (biases and an RMS norm over the whole q / k projection) and "lightning"
(linear attention with a decay per head).  The graph and the kernels live in the library (csrc/host_galirax.cu); this module
translates the configuration into b200_layer_params, the loop into the order of layer runs, and uploads the tensors under
their own names.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np

from .genesun import SequenceModel, read_safetensors, to_f32, upload
from .lib import BF16, F32, B200Error
from .llama import LayerParams

ARCH_GALIRAX = 2
MIXER_ATTENTION, MIXER_LIGHTNING = 3, 4
MLP_NONE, MLP_MOE_GATED = 0, 2
ROPE_SCALING_NONE, ROPE_SCALING_BANDS = 0, 2


def decays(mx: dict) -> list[float]:
    """The decay of every head; one number stands for all heads."""
    d = mx["decay"]
    return [float(d)] * int(mx["heads"]) if isinstance(d, (int, float)) else [float(x) for x in d]


def layer_params(layer: dict) -> LayerParams:
    mx = layer["mixer"]
    lp = LayerParams(kv_from=-1)
    kind = layer["type"]
    if kind in ("attention", "attention_2"):
        rot = mx.get("rot") or {}
        sc = rot.get("scaling") or {}
        mask = mx.get("mask") or {}
        lp.mixer = MIXER_ATTENTION
        lp.heads, lp.kv_heads, lp.dim, lp.vdim = int(mx["heads"]), int(mx.get("kv_heads", mx["heads"])), int(mx["dim"]), int(mx["vdim"])
        lp.scale = float(mx["scale"])
        lp.qkv_bias = lp.qk_norm = 1 if kind == "attention_2" else 0
        lp.window, lp.keep_first = int(mask.get("size", 0)), int(mask.get("keep_first", 0))
        lp.rope_dims = int(rot.get("dims", 0))
        lp.rope_base = float(rot.get("base", 10000.0))
        if sc:
            lp.rope_scaling = ROPE_SCALING_BANDS
            lp.yarn_factor, lp.band_low, lp.band_high, lp.yarn_original = float(sc["factor"]), float(sc["low"]), float(sc["high"]), int(sc["original"])
    elif kind == "lightning":
        lp.mixer = MIXER_LIGHTNING
        lp.heads, lp.dim, lp.vdim = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"])
        if len(decays(mx)) != lp.heads:
            raise B200Error("Galirax: a lightning layer needs one decay per head")
    else:
        raise B200Error(f"Galirax: unknown layer type {kind!r}")
    mlp = layer.get("mlp")
    if mlp is None:
        lp.mlp, lp.ff = MLP_NONE, 0
    elif mlp.get("kind", "moe") == "moe":
        r = mlp["router"]
        gr = r.get("groups") or {}
        lp.mlp, lp.ff = MLP_MOE_GATED, int(mlp["expert"]["ff"])
        lp.n_expert, lp.n_expert_used = int(r["experts"]), int(r["top"])
        lp.n_group = int(gr.get("count", 1))
        lp.n_group_used = int(gr.get("keep", lp.n_group))
        lp.router_scale = float(r.get("scale", 1.0))
    else:
        raise B200Error(f"Galirax: unknown feed-forward kind {mlp.get('kind')!r}")
    return lp


def run_order(n_layer: int, loop: dict | None) -> list[int]:
    """Layers start .. stop-1 run `times` times in a row, the others once."""
    if not loop:
        return list(range(n_layer))
    a, b, k = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    if not (0 <= a <= b <= n_layer and k >= 1):
        raise B200Error(f"Galirax: loop {loop} does not fit {n_layer} layers")
    return list(range(a)) + list(range(a, b)) * k + list(range(b, n_layer))


def build(config: dict, tensors, dtype: str = "bfloat16", n_ctx: int = 4096, n_seq_max: int = 16, max_batch: int = 512, device: int = 0) -> SequenceModel:
    """config: the parsed config.json; tensors: name -> (dtype, shape, raw bytes)."""
    if dtype not in ("bfloat16", "float32"):
        raise B200Error(f"dtype {dtype!r}: bfloat16 or float32")
    layers = [layer_params(x) for x in config["layers"]]
    model = SequenceModel(ARCH_GALIRAX, int(config["width"]), int(config["vocab"]), layers, float(config["norm"]["eps"]), n_ctx, n_seq_max, max_batch, device,
                          logit_softcap=float(config.get("logit_softcap") or 0.0), order=run_order(len(layers), config.get("loop")))
    matrix_type = BF16 if dtype == "bfloat16" else F32
    for name, (dt, shape, raw) in tensors.items():
        if name.endswith(".mlp.router"):  # the router runs in f32 in both modes
            model.set_tensor(name, F32, shape, to_f32(dt, raw))
        else:
            upload(model, name, dt, shape, raw, matrix_type)
    for il, layer in enumerate(config["layers"]):
        if layer["type"] == "lightning":  # the decays are configuration, the kernel reads them as a tensor
            d = np.asarray(decays(layer["mixer"]), dtype=np.float32)
            model.set_tensor(f"l{il}.mix.decay", F32, d.shape, d)
    model.finalize()
    return model


def load(path, **kw) -> SequenceModel:
    path = Path(path)
    config = json.loads((path / "config.json").read_text())
    return build(config, read_safetensors(path / "model.safetensors"), **kw)
