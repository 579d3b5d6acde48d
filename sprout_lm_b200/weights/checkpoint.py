"""A model folder's tensors, looked up by name, from one file or an index of shards.

``model.safetensors.index.json`` maps tensor names to shard files
(src/weight-files.ts:13-40); without it the folder holds a single
``model.safetensors``.  ``check`` compares what the model's parts expect with
what the folder holds and reports everything that is wrong in one error.
"""
from __future__ import annotations

import json
import re
from collections import OrderedDict
from pathlib import Path

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile

_SHARD_NAME = re.compile(r"^[a-zA-Z0-9_-][a-zA-Z0-9_.-]*\.safetensors$")
MAX_OPEN_SHARDS = 8


class WeightError(ValueError):
    """Missing, unexpected or wrongly shaped tensors; ``missing``, ``unexpected`` and
    ``wrong_shape`` hold the names."""

    def __init__(self, message, missing=(), unexpected=(), wrong_shape=()):
        super().__init__(message)
        self.missing = tuple(missing)
        self.unexpected = tuple(unexpected)
        self.wrong_shape = tuple(wrong_shape)


class Checkpoint:
    def __init__(self, directory):
        self.directory = Path(directory).resolve()
        self._open: OrderedDict[str, SafetensorsFile] = OrderedDict()
        index_path = self.directory / "model.safetensors.index.json"
        if index_path.exists():
            index = json.loads(index_path.read_text())
            mapping = index.get("weight_map") if isinstance(index, dict) else None
            if not isinstance(mapping, dict) or not mapping:
                raise WeightError("Invalid safetensors weight map.")
            for shard in mapping.values():
                if not isinstance(shard, str) or not _SHARD_NAME.match(shard):
                    raise WeightError("Invalid checkpoint shard filename.")
            self._shard_of = dict(mapping)
        else:
            single = self.directory / "model.safetensors"
            if not single.exists():
                raise WeightError(f"{single} does not exist.")
            self._shard_of = None

    # -- shard handles, at most MAX_OPEN_SHARDS open, least recently used closed first
    def _file(self, shard: str) -> SafetensorsFile:
        handle = self._open.get(shard)
        if handle is not None:
            self._open.move_to_end(shard)
            return handle
        if len(self._open) >= MAX_OPEN_SHARDS:
            _, oldest = self._open.popitem(last=False)
            oldest.close()
        handle = SafetensorsFile(self.directory / shard)
        self._open[shard] = handle
        return handle

    def _shards(self) -> list[str]:
        return ["model.safetensors"] if self._shard_of is None else sorted(set(self._shard_of.values()))

    def inventory(self) -> dict[str, tuple[tuple[int, ...], torch.dtype]]:
        """name -> (shape, stored dtype) of every tensor the folder holds."""
        found = {}
        for shard in self._shards():
            handle = self._file(shard)
            for name in handle.names():
                if self._shard_of is not None and self._shard_of.get(name) != shard:
                    continue
                found[name] = (handle.shape(name), handle.dtype(name))
        if self._shard_of is not None:
            for name, shard in self._shard_of.items():
                if name not in found:
                    found.setdefault(name, None)
        return found

    def check(self, expected: dict[str, tuple[int, ...]], ignorable=()) -> None:
        """Raise one WeightError naming every missing tensor, every tensor no part asked for and
        every tensor whose shape differs from the expected one."""
        found = self.inventory()
        missing = [n for n in expected if found.get(n) is None]
        unexpected = [n for n in found if n not in expected and n not in ignorable]
        wrong = [(n, tuple(expected[n]), found[n][0]) for n in expected
                 if found.get(n) is not None and tuple(found[n][0]) != tuple(expected[n])]
        if not (missing or unexpected or wrong):
            return
        lines = [f"Checkpoint {self.directory} does not fit the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(sorted(missing)))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
        if wrong:
            lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(
                f"{n} expected {list(e)}, got {list(g)}" for n, e, g in sorted(wrong)))
        raise WeightError("\n".join(lines), missing, unexpected, [w[0] for w in wrong])

    def tensor(self, name: str, shape=None) -> torch.Tensor:
        """The named tensor on the CPU in its stored dtype."""
        if self._shard_of is None:
            shard = "model.safetensors"
        else:
            shard = self._shard_of.get(name)
            if shard is None:
                raise WeightError(f"Missing tensor in shard index: {name}.", missing=[name])
        handle = self._file(shard)
        if name not in handle.entries:
            raise WeightError(f"Missing tensor: {name}.", missing=[name])
        if shape is not None and tuple(shape) != handle.shape(name):
            raise WeightError(f"Shape mismatch for {name}: expected {list(shape)}, got {list(handle.shape(name))}.",
                              wrong_shape=[name])
        return handle.tensor(name)

    def close(self):
        for handle in self._open.values():
            handle.close()
        self._open.clear()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


__all__ = ["Checkpoint", "WeightError", "SafetensorsError"]
