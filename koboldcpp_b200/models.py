"""Model registry: a model folder's config.json names its architecture; the registry maps it to the loader."""
from __future__ import annotations

import json
from pathlib import Path

from . import galirax, genesun, medodra, zevopel
from .lib import B200Error

ARCHITECTURES = {
    "Genesun": genesun.load,
    "Galirax": galirax.load,
    "Zevopel": zevopel.load,
    "Medodra": medodra.load,
}


def load_model(path, **kw):
    """Load the model in `path` with the loader of its architecture (kw: dtype, n_ctx, n_seq_max, max_batch, device)."""
    cfg = json.loads((Path(path) / "config.json").read_text())
    arch = cfg.get("architecture")
    if arch not in ARCHITECTURES:
        raise B200Error(f"{path}: architecture {arch!r} is not one of {sorted(ARCHITECTURES)}")
    return ARCHITECTURES[arch](path, **kw)
