"""Zevopel: the reader of its config.json and weights behind the shared decoder (include/b200_llama.h).

A Zevopel model folder holds config.json ("architecture": "Zevopel", "width", "vocab", "norm": {"eps"}, "embedding": {"scale"},
"residual_mult", and "layers": a list of {"type", "mixer": {...}, "mlp": {...} or null}) and model.safetensors (bfloat16 matrices
named "embed", "head", "final.norm" and "l<i>.<leaf>").  One layer type, "attention": grouped-query attention with a norm per head
on q and k, rotation of the two halves of the rotated part against each other, a sink per head, chunked visibility and a sigmoid
gate per head; the feed-forward is "dense" (gated, tanh gelu) or "moe" (softmax router, clamped experts).  The graph and the
kernels live in the library (csrc/host_zevopel.cu); this module translates the configuration into b200_layer_params and uploads the
tensors under their own names.
"""
from __future__ import annotations

import json
from pathlib import Path

from .genesun import SequenceModel, read_safetensors, to_f32, upload
from .lib import BF16, F32, B200Error
from .llama import LayerParams

ARCH_ZEVOPEL = 3
MIXER_ATTENTION = 3
MLP_NONE, MLP_MOE_GATED, MLP_DENSE_GATED = 0, 2, 3
ROPE_SCALING_NONE, ROPE_SCALING_BANDS = 0, 2
GLU_GELU_TANH, GLU_SWISH_CLAMPED = 1, 2
ROUTER_SOFTMAX = 1
SWISH_ALPHA = 1.702  # the experts' activation is g * sigmoid(1.702 g): the design fixes the constant


def layer_params(layer: dict) -> LayerParams:
    if layer["type"] != "attention":
        raise B200Error(f"Zevopel: unknown layer type {layer['type']!r}")
    mx = layer["mixer"]
    rot = mx.get("rot") or {}
    sc = rot.get("scaling") or {}
    mask = mx.get("mask") or {}
    lp = LayerParams(kv_from=-1)
    lp.mixer = MIXER_ATTENTION
    lp.heads, lp.kv_heads, lp.dim, lp.vdim = int(mx["heads"]), int(mx.get("kv_heads", mx["heads"])), int(mx["dim"]), int(mx["vdim"])
    lp.scale = float(mx["scale"])
    lp.qk_norm = lp.qk_norm_per_head = 1
    lp.rope_halves = lp.head_gate = 1
    lp.chunk = int(mask.get("size", 0))
    lp.rope_dims = int(rot.get("dims", 0))
    lp.rope_base = float(rot.get("base", 10000.0))
    if sc:
        lp.rope_scaling = ROPE_SCALING_BANDS
        lp.yarn_factor, lp.band_low, lp.band_high, lp.yarn_original = float(sc["factor"]), float(sc["low"]), float(sc["high"]), int(sc["original"])
    mlp = layer.get("mlp")
    if mlp is None:
        lp.mlp, lp.ff = MLP_NONE, 0
    elif mlp["kind"] == "dense":
        lp.mlp, lp.ff, lp.glu_kind = MLP_DENSE_GATED, int(mlp["ff"]), GLU_GELU_TANH
    elif mlp["kind"] == "moe":
        r = mlp["router"]
        lp.mlp, lp.ff = MLP_MOE_GATED, int(mlp["expert"]["ff"])
        lp.glu_kind, lp.glu_limit, lp.glu_alpha = GLU_SWISH_CLAMPED, float(mlp["expert"]["limit"]), SWISH_ALPHA
        lp.n_expert, lp.n_expert_used = int(r["experts"]), int(r["top"])
        lp.n_group = lp.n_group_used = 1
        lp.router_scale, lp.router_score, lp.router_keep_scores = 1.0, ROUTER_SOFTMAX, 1
    else:
        raise B200Error(f"Zevopel: unknown feed-forward kind {mlp['kind']!r}")
    return lp


def build(config: dict, tensors, dtype: str = "bfloat16", n_ctx: int = 4096, n_seq_max: int = 16, max_batch: int = 512, device: int = 0) -> SequenceModel:
    """config: the parsed config.json; tensors: name -> (dtype, shape, raw bytes)."""
    if dtype not in ("bfloat16", "float32"):
        raise B200Error(f"dtype {dtype!r}: bfloat16 or float32")
    layers = [layer_params(x) for x in config["layers"]]
    model = SequenceModel(ARCH_ZEVOPEL, int(config["width"]), int(config["vocab"]), layers, float(config["norm"]["eps"]), n_ctx, n_seq_max, max_batch, device,
                          embed_scale=float((config.get("embedding") or {}).get("scale", 1.0)), residual_mult=float(config.get("residual_mult", 1.0)))
    matrix_type = BF16 if dtype == "bfloat16" else F32
    for name, (dt, shape, raw) in tensors.items():
        if name.endswith(".mlp.router"):  # the router runs in f32 in both modes
            model.set_tensor(name, F32, shape, to_f32(dt, raw))
        else:
            upload(model, name, dt, shape, raw, matrix_type)
    model.finalize()
    return model


def load(path, **kw) -> SequenceModel:
    path = Path(path)
    config = json.loads((path / "config.json").read_text())
    return build(config, read_safetensors(path / "model.safetensors"), **kw)
