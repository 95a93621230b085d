"""Where weights come from: a model folder, or a seeded random generator that yields the same tensor names.

Folder: `config.json` is required, every `*.safetensors` file is read in sorted order, and a tensor name found in
two files is an error (std/holon_std/weights/hf/source.py:49-115). Random: the reference has no such mode; its tests
make tiny checkpoints with another library. Here every tensor is drawn from its own generator, seeded by
(seed, stored name), so a tensor does not depend on which others are made, on their order, or on the device's
memory: matrices and tables N(0, 0.02), norm weights 1 + N(0, 0.1).
"""
from __future__ import annotations

import hashlib
import json
import pathlib
from collections.abc import Iterator, Mapping
from typing import Any

import torch


class SafetensorsSource:
    def __init__(self, folder) -> None:
        self.folder = pathlib.Path(folder)
        if not (self.folder / "config.json").is_file():
            raise FileNotFoundError(f"{self.folder}: no config.json")
        self._config = json.loads((self.folder / "config.json").read_text())
        self.files = sorted(self.folder.glob("*.safetensors"))
        if not self.files:
            raise FileNotFoundError(f"{self.folder}: no *.safetensors file")

    def config(self) -> dict[str, Any]:
        return self._config

    def eos_token_ids(self) -> tuple[int, ...]:
        """`eos_token_id` of config.json and of generation_config.json, an int or a list (source.py:62-66)."""
        ids: list[int] = []
        for name in ("config.json", "generation_config.json"):
            path = self.folder / name
            if path.is_file():
                eos = json.loads(path.read_text()).get("eos_token_id")
                ids += [eos] if isinstance(eos, int) else list(eos or ())
        return tuple(dict.fromkeys(ids))

    def tensors(self) -> Iterator[tuple[str, torch.Tensor]]:
        from safetensors import safe_open
        seen: dict[str, pathlib.Path] = {}
        for path in self.files:
            with safe_open(str(path), framework="pt") as f:
                for name in f.keys():
                    if name in seen:
                        raise ValueError(f"tensor {name!r} is stored in both {seen[name].name} and {path.name}")
                    seen[name] = path
                    yield name, f.get_tensor(name)


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & (2 ** 63 - 1)


class RandomSource:
    """Random weights for `config` (a config.json dict), under the stored names of its architecture."""

    STD_MATRIX, STD_GAIN = 0.02, 0.1

    def __init__(self, config: Mapping[str, Any], seed: int, device="cpu", dtype: torch.dtype = torch.bfloat16) -> None:
        self._config, self.seed, self.device, self.dtype = dict(config), int(seed), torch.device(device), dtype

    def config(self) -> dict[str, Any]:
        return self._config

    def eos_token_ids(self) -> tuple[int, ...]:
        eos = self._config.get("eos_token_id")
        return (eos,) if isinstance(eos, int) else tuple(eos or ())

    def table(self) -> list[tuple[str, tuple[int, ...], str]]:
        """(stored name, shape, kind) of every tensor a folder of this architecture holds."""
        from ..config.registry import resolve_architecture
        from ..parts import BuildContext, Model
        from .loader import NameMap
        arch = resolve_architecture(self._config)
        spec = arch.recipe(arch.parse(self._config))
        model = Model(spec, BuildContext("meta", self.dtype, None, max_positions=1))
        names = NameMap(spec.weight_rules)
        return [(names.stored(ours), (rows[1] - rows[0], *p.shape[1:]), p.kind) for ours, p, rows in model.loadables()]

    def tensors(self) -> Iterator[tuple[str, torch.Tensor]]:
        for name, shape, kind in self.table():
            g = torch.Generator(device=self.device).manual_seed(_tensor_seed(self.seed, name))
            x = torch.randn(shape, generator=g, dtype=torch.float32, device=self.device)
            x = x.mul_(self.STD_GAIN).add_(1.0) if kind == "gain" else x.mul_(self.STD_MATRIX)
            yield name, x.to(self.dtype)


def write_model_folder(source, folder) -> pathlib.Path:
    """Writes `config.json` and `model.safetensors` from any source; returns the folder."""
    from safetensors.torch import save_file
    folder = pathlib.Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(source.config(), indent=1))
    save_file({name: t.cpu().contiguous() for name, t in source.tensors()}, str(folder / "model.safetensors"))
    return folder
