"""Weights: from safetensors files by tensor name, and a seeded random mode
that writes a model folder.

Reading follows mlx-lm's ``load_model`` (mlx_lm/utils.py:336-343, 444-445):
every ``model*.safetensors`` of the folder is merged into one dictionary, and
the load is strict.  Strictness is spelled out here: names the model expects
and the files lack, names the files hold and the model does not know, and
shapes that differ are collected into ONE ``WeightError``.

dtypes on the device: matrices and embedding tables take the run's dtype
(bfloat16 or float32), gains and biases are float32 whatever they were stored
as, integer tables are int32.  A conversion from bfloat16 to float32 is exact,
so a folder written in bfloat16 gives the same weights to both runs.
"""

from __future__ import annotations

import glob
import json
import os
import re
from typing import Dict, List, Optional, Tuple

import torch

from ..config import get_architecture, load_config
from ..parts.base import INT_TABLE, MATRIX, VECTOR, ParamSpec
from ..parts.model import Model, ModelDescription

PREFIXES = ("transformer.", "model.")


class WeightError(ValueError):
    pass


def _strip(name: str) -> str:
    for p in PREFIXES:
        if name.startswith(p):
            return name[len(p):]
    return name


def read_safetensors(model_path: str) -> Dict[str, torch.Tensor]:
    from safetensors import safe_open

    files = sorted(glob.glob(os.path.join(model_path, "model*.safetensors")))
    if not files:
        raise FileNotFoundError(f"No safetensors found in {model_path}")
    tensors: Dict[str, torch.Tensor] = {}
    for path in files:
        with safe_open(path, framework="pt", device="cpu") as f:
            for name in f.keys():
                tensors[name] = f.get_tensor(name)
    return tensors


def check_tensors(description: ModelDescription, tensors: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Match file tensors to the model's expectations; return ``name -> tensor`` for the
    expected names or raise one error that lists everything that is wrong."""
    specs = {s.name: s for s in description.param_specs()}
    ignored = [re.compile(p + r"\Z") for p in description.ignored_tensors]
    got: Dict[str, torch.Tensor] = {}
    unexpected: List[str] = []
    for raw, t in tensors.items():
        name = _strip(raw)
        if name in specs:
            got[name] = t
        elif not any(r.match(name) for r in ignored):
            unexpected.append(raw)
    missing = [n for n in specs if n not in got]
    wrong = [(n, tuple(got[n].shape), specs[n].shape) for n in specs
             if n in got and tuple(got[n].shape) != tuple(specs[n].shape)]
    if missing or unexpected or wrong:
        lines = [f"weights do not fit model type {description.model_type!r}:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(sorted(missing)))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
        if wrong:
            lines.append(f"  wrong shape ({len(wrong)}): "
                         + "; ".join(f"{n} is {a}, expected {b}" for n, a, b in wrong))
        raise WeightError("\n".join(lines))
    return got


def place(spec: ParamSpec, t: torch.Tensor, dtype: torch.dtype, device) -> torch.Tensor:
    if spec.kind == INT_TABLE:
        target = torch.int32
    elif spec.kind == VECTOR:
        target = torch.float32
    else:
        target = dtype
    return t.to(device=device, dtype=target).contiguous()


def build_model(config: dict, tensors: Dict[str, torch.Tensor], dtype: torch.dtype = torch.bfloat16,
                device="cuda", get_model_classes=None) -> Model:
    """``get_model_classes(config) -> (builder, args class)`` replaces the registry lookup, as the parameter of
    the same name does in mlx-lm's ``load_model`` (mlx_lm/utils.py:296-301)."""
    if get_model_classes is not None:
        build, args_class = get_model_classes(config)
    else:
        arch = get_architecture(config)
        build, args_class = arch.build, arch.args_class
    args = args_class.from_dict(config)
    description = build(args)
    got = check_tensors(description, tensors)
    specs = {s.name: s for s in description.param_specs()}
    placed = {n: place(specs[n], t, dtype, device) for n, t in got.items()}
    return Model(description, placed, dtype, device)


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"dtype {dtype}: the engine runs in bfloat16 or float32")
        return dtype
    table = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
             "f32": torch.float32}
    try:
        return table[str(dtype).lower()]
    except KeyError:
        raise ValueError(f"dtype {dtype!r}: 'bfloat16' or 'float32'") from None


def load_model(model_path: str, dtype="bfloat16", device="cuda", model_config: Optional[dict] = None,
               get_model_classes=None) -> Tuple[Model, dict]:
    """Model folder -> (model on the device, config dict)."""
    config = load_config(model_path)
    if model_config:
        config.update(model_config)
    model = build_model(config, read_safetensors(model_path), parse_dtype(dtype), device, get_model_classes)
    return model, config


# ------------------------------------------------------------------ random weights

def random_tensors(description: ModelDescription, seed: int, dtype: torch.dtype = torch.bfloat16
                   ) -> Dict[str, torch.Tensor]:
    """Every tensor of the model drawn in float32 on the CPU from one generator seeded with
    ``seed``, in the fixed order of ``param_specs()``, then rounded to ``dtype``."""
    g = torch.Generator(device="cpu").manual_seed(int(seed))
    out: Dict[str, torch.Tensor] = {}
    for s in description.param_specs():
        if s.kind == INT_TABLE:
            raise WeightError(f"{s.name}: the random-weights mode has no rule for integer tables")
        if s.init.std == 0.0:
            t = torch.full(s.shape, float(s.init.mean), dtype=torch.float32)
        else:
            t = torch.randn(s.shape, generator=g, dtype=torch.float32) * s.init.std + s.init.mean
        out[s.name] = t.to(dtype)
    return out


def write_random_model(model_path: str, config: dict, seed: int, dtype="bfloat16") -> dict:
    """Write ``config.json`` and ``model.safetensors`` of a randomly initialised model."""
    from safetensors.torch import save_file

    arch = get_architecture(config)
    args = arch.args_class.from_dict(config)
    description = arch.build(args)
    tensors = random_tensors(description, seed, parse_dtype(dtype))
    os.makedirs(model_path, exist_ok=True)
    with open(os.path.join(model_path, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    save_file({k: v.contiguous() for k, v in tensors.items()}, os.path.join(model_path, "model.safetensors"),
              metadata={"format": "pt", "seed": str(seed)})
    return config


def main(argv=None) -> None:
    import argparse

    ap = argparse.ArgumentParser(prog="mlx_lm_b200.random_weights",
                                 description="Write a model folder with seeded random weights.")
    ap.add_argument("--config", required=True, help="a config.json to take the sizes from")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"], help="dtype stored in the file")
    ap.add_argument("--out", required=True, help="folder to write config.json and model.safetensors to")
    a = ap.parse_args(argv)
    with open(a.config) as f:
        config = json.load(f)
    write_random_model(a.out, config, a.seed, a.dtype)
    print(f"wrote {a.out}")


if __name__ == "__main__":
    main()
