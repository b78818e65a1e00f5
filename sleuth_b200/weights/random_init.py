"""Writing a model folder (``config.json`` + ``model.safetensors``) from a configuration and a seed.

Every matrix and the embedding are drawn from N(0, std) (the reference's ``init_std`` 0.02,
sleuth/forge/model/transformer.py:248-254), biases likewise, norm gains from 1 + N(0, std) so that a
gain that is dropped or applied twice shows in a test. Tensors are drawn in the sorted order of their
names from one seeded counter-based generator (NumPy's Philox), in float64 and then rounded, so the
same seed gives the same folder on every machine and in either stored dtype.
"""

from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

from ..config.registry import Architecture, find_architecture, parse_config
from ..parts.base import BuildContext
from .safetensors import write_safetensors


def expected_tensors(spec, ctx: BuildContext | None = None) -> dict:
    """name -> ParamDecl of a model description, without building anything on a device."""
    from ..engine.model import declare_model
    return declare_model(spec)


def random_tensors(spec, seed: int, dtype: torch.dtype = torch.bfloat16, std: float = 0.02) -> dict[str, torch.Tensor]:
    decls = expected_tensors(spec)
    rng = np.random.Generator(np.random.Philox(seed))
    out = {}
    for name in sorted(decls):
        d = decls[name]
        if d.role == "table":
            out[name] = torch.zeros(d.shape, dtype=torch.int32)
            continue
        v = rng.standard_normal(size=d.shape) * std
        if d.init == "gain":
            v = 1.0 + v
        out[name] = torch.from_numpy(v).to(dtype)
    return out


def write_random_model(folder, config_json: dict, seed: int, dtype: torch.dtype = torch.bfloat16,
                       std: float = 0.02) -> Path:
    """Create ``folder`` with ``config.json`` as given and seeded random weights for it."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    arch, cfg, _ = parse_config(config_json)
    spec = arch.model_spec(cfg)
    tensors = random_tensors(spec, seed, dtype, std)
    cj = dict(config_json)
    cj.setdefault("architectures", [arch.name])
    cj["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}[dtype]
    (folder / "config.json").write_text(json.dumps(cj, indent=2) + "\n")
    write_safetensors(tensors, folder / "model.safetensors", metadata={"format": "pt", "seed": str(seed)})
    return folder
