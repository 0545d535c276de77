"""Random weights from a configuration and a seed.

Every checkpoint tensor is drawn in float32, in the fixed order in which the
model declares its tensors, from one seeded generator: matrices and tables
from N(0, 0.02), norm weights from 1 + U(-0.1, 0.1).  The same stream either
fills a model folder (``write_model_folder``: config.json + model.safetensors,
the form every other tool reads) or is bound straight to the parts on the
device, which a model too large for a host copy needs.  The reference has no
such mode (its modules keep torch's default initialisation,
tinyvllm/layers.py:87-91, :146-152).
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Iterator

import torch


NORMAL_STD = 0.02
AROUND_ONE_SPREAD = 0.1


def random_tensors(targets, seed: int, device="cpu") -> Iterator[tuple[str, torch.Tensor]]:
    """(checkpoint name, float32 tensor) in declaration order."""
    generator = torch.Generator(device=device)
    generator.manual_seed(seed)
    for _part, spec in targets:
        for source in spec.sources:
            shape = (source.rows,) + tuple(spec.shape[1:])
            if spec.role == "integer":
                raise ValueError(f"{source.name}: integer tables have no random law")
            if spec.init == "around_one":
                t = torch.rand(shape, generator=generator, device=device, dtype=torch.float32)
                t = 1.0 + (2.0 * t - 1.0) * AROUND_ONE_SPREAD
            elif spec.init == "normal":
                t = torch.randn(shape, generator=generator, device=device,
                                dtype=torch.float32) * NORMAL_STD
            else:
                raise ValueError(f"{source.name}: unknown init law {spec.init!r}")
            yield source.name, t


def write_model_folder(folder, config, seed: int, *, dtype: torch.dtype = torch.float32) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` into ``folder``.

    ``config`` is a typed architecture configuration; ``dtype`` is the dtype
    the tensors are stored in (the values are drawn in float32 either way).
    """
    from safetensors.torch import save_file

    from ..engine.model import Model

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config.to_json(), indent=1), encoding="utf-8")
    model = Model(config.to_spec(), device=torch.device("meta"), dtype=torch.float32)
    tensors = {
        name: tensor.to(dtype).contiguous()
        for name, tensor in random_tensors(model.param_targets(), seed)
    }
    save_file(tensors, str(folder / "model.safetensors"))
    return folder
