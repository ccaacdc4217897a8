"""Medodra: the reader of its config.json and weights behind the shared decoder (include/b200_llama.h).

A Medodra model folder holds config.json ("architecture": "Medodra", "width", "vocab", "norm": {"eps"}, "embedding": {"scale"},
"residual_mult", "loop": {"start", "stop", "times"} and "layers": a list of {"type", "mixer": {...}, "mlp": {...} or null}) and
model.safetensors (bfloat16 matrices named "embed", "head", "final.norm", "loop.in" and "l<i>.<leaf>").  Two layer types: "delta"
(gated delta rule behind a short convolution) and "parallel" (attention with sigmoid weights and a distance bias beside a minGRU).
The feed-forward is a mixture of experts whose sigmoid scores scale the chosen experts' inputs, plus a gated shared expert.  The
graph and the kernels live in the library (csrc/host_medodra.cu); this module translates the configuration into b200_layer_params
and uploads the tensors under their own names.
"""
from __future__ import annotations

import json
from pathlib import Path

from .galirax import run_order
from .genesun import SequenceModel, read_safetensors, to_f32, upload
from .lib import BF16, F32, B200Error
from .llama import LayerParams

ARCH_MEDODRA = 4
MIXER_DELTA, MIXER_SIGMOID_ATTENTION_GRU = 5, 6
MLP_NONE, MLP_MOE_GATED = 0, 2
GLU_SILU = 0
ROUTER_SIGMOID = 0
# small tensors that the library reads in f32 whatever the matrix type: convolution taps, the distance table, the router
F32_LEAVES = (".conv", ".rel", ".mlp.router")


def layer_params(layer: dict, loop_input: bool = False) -> LayerParams:
    mx = layer["mixer"]
    lp = LayerParams(kv_from=-1)
    kind = layer["type"]
    if kind == "delta":
        lp.mixer = MIXER_DELTA
        a = mx
    elif kind == "parallel":
        lp.mixer = MIXER_SIGMOID_ATTENTION_GRU
        a = mx["left"]
        lp.scale = float(a["scale"])
        lp.q_temp_coef, lp.q_temp_every = float(a["q_temp"]["coef"]), int(a["q_temp"]["every"])
        lp.dist_bias_max = int(a["bias_max"])
        lp.side_width = int(mx["right"]["width"])
        if lp.q_temp_every < 1:
            raise B200Error("Medodra: q_temp.every must be at least 1")
    else:
        raise B200Error(f"Medodra: unknown layer type {kind!r}")
    lp.heads, lp.kv_heads, lp.dim, lp.vdim = int(a["heads"]), int(a.get("kv_heads", a["heads"])), int(a["dim"]), int(a["vdim"])
    lp.conv_taps = int(a["conv"])
    lp.loop_input = 1 if loop_input else 0
    mlp = layer.get("mlp")
    if mlp is None:
        lp.mlp, lp.ff = MLP_NONE, 0
    elif mlp.get("kind", "moe") == "moe":
        r = mlp["router"]
        lp.mlp, lp.ff, lp.glu_kind = MLP_MOE_GATED, int(mlp["expert"]["ff"]), GLU_SILU
        lp.n_expert, lp.n_expert_used = int(r["experts"]), int(r["top"])
        lp.n_group = lp.n_group_used = 1
        lp.router_scale, lp.router_score, lp.router_keep_scores, lp.router_scale_input = 1.0, ROUTER_SIGMOID, 1, 1
        lp.shared_ff = int((mlp.get("shared") or {}).get("ff", 0))
    else:
        raise B200Error(f"Medodra: unknown feed-forward kind {mlp.get('kind')!r}")
    return lp


def build(config: dict, tensors, dtype: str = "bfloat16", n_ctx: int = 4096, n_seq_max: int = 16, max_batch: int = 512, device: int = 0) -> SequenceModel:
    """config: the parsed config.json; tensors: name -> (dtype, shape, raw bytes)."""
    if dtype not in ("bfloat16", "float32"):
        raise B200Error(f"dtype {dtype!r}: bfloat16 or float32")
    loop = config.get("loop")
    order = run_order(len(config["layers"]), loop)
    # the first layer of the looped stretch takes the input projection every time it runs (a stretch of no layers has none)
    first = int(loop["start"]) if loop and int(loop["stop"]) > int(loop["start"]) else -1
    layers = [layer_params(x, loop_input=(i == first)) for i, x in enumerate(config["layers"])]
    model = SequenceModel(ARCH_MEDODRA, int(config["width"]), int(config["vocab"]), layers, float(config["norm"]["eps"]), n_ctx, n_seq_max, max_batch, device,
                          order=order, embed_scale=float((config.get("embedding") or {}).get("scale", 1.0)), residual_mult=float(config.get("residual_mult", 1.0)))
    matrix_type = BF16 if dtype == "bfloat16" else F32
    for name, (dt, shape, raw) in tensors.items():
        if name.endswith(F32_LEAVES):
            model.set_tensor(name, F32, shape, to_f32(dt, raw))
        else:
            upload(model, name, dt, shape, raw, matrix_type)
    model.finalize()
    return model


def load(path, **kw) -> SequenceModel:
    path = Path(path)
    config = json.loads((path / "config.json").read_text())
    return build(config, read_safetensors(path / "model.safetensors"), **kw)
