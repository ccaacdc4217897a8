"""Genesun: the reader of its config.json and weights, and the model object behind the shared decoder (include/b200_llama.h).

A Genesun model folder holds config.json ("architecture": "Genesun", "width", "vocab", "norm": {"eps"}, and "layers": a list
of {"type", "mixer": {...}, "mlp": {...} or null}) and model.safetensors (bfloat16 matrices named "embed", "head",
"final.norm" and "l<i>.<leaf>").  The graph and the kernels live in the library (csrc/host_genesun.cu); this module only
translates the configuration into b200_layer_params and uploads the tensors under their own names.
"""
from __future__ import annotations

import ctypes as C
import json
import struct
from pathlib import Path

import numpy as np

from .lib import BF16, F32, B200Error, check
from .llama import LayerParams, LlamaParams, _l

ARCH_GENESUN = 1
MIXER_LATENT_ATTENTION, MIXER_MLSTM = 1, 2
MLP_NONE, MLP_DENSE_POLYNORM = 0, 1


def read_safetensors(path) -> dict[str, tuple[str, tuple[int, ...], np.ndarray]]:
    """name -> (dtype, shape, raw little-endian bytes).  The file is an 8-byte length, that many bytes of JSON, then the data."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        meta = json.loads(f.read(n))
        data = np.frombuffer(f.read(), dtype=np.uint8)
    out = {}
    for name, v in meta.items():
        if name == "__metadata__":
            continue
        a, b = v["data_offsets"]
        out[name] = (v["dtype"], tuple(v["shape"]), data[a:b])
    return out


def to_f32(dtype: str, raw: np.ndarray) -> np.ndarray:
    if dtype == "BF16":
        return (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32)
    if dtype == "F32":
        return raw.view(np.float32)
    if dtype == "F16":
        return raw.view(np.float16).astype(np.float32)
    if dtype == "I32":
        return raw.view(np.int32).astype(np.float32)
    raise B200Error(f"safetensors dtype {dtype} is not supported")


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def layer_params(layer: dict) -> LayerParams:
    mx = layer["mixer"]
    lp = LayerParams(kv_from=-1)
    kind = layer["type"]
    if kind == "latent_attention":
        rot = mx.get("rot") or {}
        sc = rot.get("scaling") or {}
        lp.mixer = MIXER_LATENT_ATTENTION
        lp.heads, lp.dim, lp.vdim = mx["heads"], mx["dim"], mx["vdim"]
        lp.rot_dim, lp.kv_rank, lp.q_rank = mx.get("rot_dim", 0), mx["kv_rank"], mx["q_rank"]
        lp.kv_from = -1 if mx.get("kv_from") is None else int(mx["kv_from"])
        lp.window = int(mx.get("window") or 0)
        lp.scale = float(mx["scale"])
        lp.rope_dims = int(rot.get("dims", lp.rot_dim))
        lp.rope_base = float(rot.get("base", 10000.0))
        lp.yarn_factor = float(sc.get("factor", 0.0))
        lp.yarn_fast, lp.yarn_slow = float(sc.get("fast", 32.0)), float(sc.get("slow", 1.0))
        lp.yarn_original = int(sc.get("original", 0))
    elif kind == "mlstm":
        lp.mixer = MIXER_MLSTM
        lp.heads, lp.dim, lp.vdim = mx["heads"], mx["dim"], mx["vdim"]
        lp.gate_cap = float(mx["gate_cap"])
    else:
        raise B200Error(f"Genesun: unknown layer type {kind!r}")
    mlp = layer.get("mlp")
    if mlp is None:
        lp.mlp, lp.ff = MLP_NONE, 0
    elif mlp.get("kind", "dense") == "dense":
        lp.mlp, lp.ff = MLP_DENSE_POLYNORM, int(mlp["ff"])
    else:
        raise B200Error(f"Genesun: unknown feed-forward kind {mlp.get('kind')!r}")
    return lp


class SequenceModel:
    """A model of an architecture with sequences, resident on one device: tensors in, batch steps out."""

    def __init__(self, arch: int, width: int, vocab: int, layers: list[LayerParams], eps: float, n_ctx: int, n_seq_max: int, max_batch: int, device: int = 0,
                 logit_softcap: float = 0.0, order: list[int] | None = None, embed_scale: float = 1.0, residual_mult: float = 1.0):
        """order: the layer of every run, in execution order (None: every layer once); a layer that runs several times has a cache
        or state per run."""
        L = _l()
        if L.ggml_backend_b200_get_device_count() <= 0:
            raise B200Error("no CUDA device: the B200 backend has no CPU fallback")
        self.width, self.vocab, self.n_layer = width, vocab, len(layers)
        self.n_ctx = (max(n_ctx, 1) + 255) // 256 * 256
        self.n_seq_max, self.max_batch = n_seq_max, max_batch
        p = LlamaParams(n_embd=width, n_layer=len(layers), n_vocab=vocab, n_ctx=self.n_ctx, rms_eps=eps, main_device=device, arch=arch, n_seq_max=n_seq_max,
                        logit_softcap=logit_softcap, embed_scale=embed_scale, residual_mult=residual_mult)
        h = C.c_void_p()
        check(L.b200_llama_new(C.byref(p), C.byref(h)), "b200_llama_new")
        self.h = h
        for il, lp in enumerate(layers):
            check(L.b200_llama_set_layer(self.h, il, C.byref(lp)), f"set_layer {il}")
        if order is not None:
            o = np.ascontiguousarray(order, dtype=np.int32)
            check(L.b200_llama_set_layer_order(self.h, o.ctypes.data, len(o)), "set_layer_order")
        self._logits = None

    def set_tensor(self, name: str, ty: int, shape: tuple[int, ...], data: np.ndarray) -> None:
        """shape as stored: [rows] or [out, in]."""
        data = np.ascontiguousarray(data)
        ne0, ne1 = (shape[0], 1) if len(shape) == 1 else (shape[1], shape[0])
        check(_l().b200_llama_set_tensor(self.h, name.encode(), ty, ne0, ne1, 1, data.ctypes.data), f"set_tensor {name}")

    def finalize(self) -> None:
        check(_l().b200_llama_finalize(self.h, self.max_batch), "b200_llama_finalize")
        self._logits = np.empty((self.max_batch, self.vocab), dtype=np.float32)

    def seq_open(self) -> int:
        s = C.c_int32()
        check(_l().b200_llama_seq_open(self.h, C.byref(s)), "seq_open")
        return s.value

    def seq_close(self, seq: int) -> None:
        check(_l().b200_llama_seq_close(self.h, seq), "seq_close")

    def seq_length(self, seq: int) -> int:
        return _l().b200_llama_seq_length(self.h, seq)

    def decode_batch(self, tokens, seq_ids, want) -> np.ndarray:
        """One step; returns the logits [number of wanted tokens, vocab] (a fresh array)."""
        tok = np.ascontiguousarray(tokens, dtype=np.int32)
        sid = np.ascontiguousarray(seq_ids, dtype=np.int32)
        w = np.ascontiguousarray(want, dtype=np.int8)
        n_out = int(np.count_nonzero(w))
        out = np.empty((n_out, self.vocab), dtype=np.float32)
        check(_l().b200_llama_decode_batch(self.h, tok.ctypes.data, sid.ctypes.data, w.ctypes.data, len(tok), out.ctypes.data if n_out else None), "b200_llama_decode_batch")
        return out

    def replay(self) -> None:
        check(_l().b200_llama_replay(self.h), "replay")

    @property
    def stream(self):
        return _l().b200_llama_stream(self.h)

    def stats(self) -> dict:
        a, b, c, d = C.c_int64(), C.c_int64(), C.c_int64(), C.c_int64()
        check(_l().b200_llama_stats(self.h, C.byref(a), C.byref(b), C.byref(c), C.byref(d)), "stats")
        return {"n_nodes": a.value, "n_kernels": b.value, "weight_bytes": c.value, "kv_bytes": d.value}

    def close(self) -> None:
        if getattr(self, "h", None):
            _l().b200_llama_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def upload(model: SequenceModel, name: str, dtype: str, shape: tuple[int, ...], raw: np.ndarray, matrix_type: int) -> None:
    """Matrices go up in `matrix_type` (BF16 keeps the stored bits, F32 widens them); vectors and the embedding table in f32."""
    as_matrix = len(shape) == 2 and name != "embed"
    if as_matrix and matrix_type == BF16:
        bits = raw.view(np.uint16) if dtype == "BF16" else f32_to_bf16_bits(to_f32(dtype, raw))
        model.set_tensor(name, BF16, shape, bits)
    else:
        model.set_tensor(name, F32, shape, to_f32(dtype, raw))


def build(config: dict, tensors, dtype: str = "bfloat16", n_ctx: int = 4096, n_seq_max: int = 16, max_batch: int = 512, device: int = 0) -> SequenceModel:
    """config: the parsed config.json; tensors: name -> (dtype, shape, raw bytes)."""
    if dtype not in ("bfloat16", "float32"):
        raise B200Error(f"dtype {dtype!r}: bfloat16 or float32")
    layers = [layer_params(x) for x in config["layers"]]
    model = SequenceModel(ARCH_GENESUN, int(config["width"]), int(config["vocab"]), layers, float(config["norm"]["eps"]), n_ctx, n_seq_max, max_batch, device)
    matrix_type = BF16 if dtype == "bfloat16" else F32
    for name, (dt, shape, raw) in tensors.items():
        upload(model, name, dt, shape, raw, matrix_type)
    model.finalize()
    return model


def load(path, **kw) -> SequenceModel:
    path = Path(path)
    config = json.loads((path / "config.json").read_text())
    return build(config, read_safetensors(path / "model.safetensors"), **kw)
