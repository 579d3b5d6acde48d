"""Reader and writer for the safetensors container (F32, BF16, F16).

The checks follow the reference's reader (src/safetensors.ts:26-66): an 8-byte
little-endian header length, a JSON header of at most 16 MiB, tensors whose
byte ranges tile the data section exactly (no gap, no overlap, ending at the
end of the file).  Tensors are memory-mapped and handed out in the dtype they
are stored in; nothing is converted here.
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path

import numpy as np
import torch

MAX_HEADER_BYTES = 16 * 1024 * 1024
_ITEM_BYTES = {"F32": 4, "BF16": 2, "F16": 2}
_TORCH_DTYPE = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16}
_NAME_OF = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16"}


class SafetensorsError(ValueError):
    """A malformed or unsupported safetensors file."""


class SafetensorsFile:
    def __init__(self, path):
        self.path = Path(path)
        size = self.path.stat().st_size
        with open(self.path, "rb") as handle:
            prefix = handle.read(8)
            if len(prefix) < 8:
                raise SafetensorsError("Truncated safetensors file.")
            (header_len,) = struct.unpack("<Q", prefix)
            if header_len <= 0 or header_len > MAX_HEADER_BYTES or header_len + 8 > size:
                raise SafetensorsError("Invalid safetensors header length.")
            header_bytes = handle.read(header_len)
            if len(header_bytes) < header_len:
                raise SafetensorsError("Truncated safetensors file.")
            try:
                parsed = json.loads(header_bytes.decode("utf-8"))
            except (UnicodeDecodeError, json.JSONDecodeError) as error:
                raise SafetensorsError(f"Invalid safetensors header: {error}") from None
            if not isinstance(parsed, dict):
                raise SafetensorsError("Invalid safetensors header.")
            self._start = 8 + header_len
            data_bytes = size - self._start
            self.entries: dict[str, dict] = {}
            for name, entry in parsed.items():
                if name == "__metadata__":
                    continue
                ok = (isinstance(entry, dict) and entry.get("dtype") in _ITEM_BYTES
                      and isinstance(entry.get("shape"), list)
                      and all(isinstance(n, int) and not isinstance(n, bool) and n > 0 for n in entry["shape"])
                      and isinstance(entry.get("data_offsets"), list) and len(entry["data_offsets"]) == 2)
                if not ok:
                    raise SafetensorsError(f"Unsupported or malformed tensor: {name}.")
                begin, end = entry["data_offsets"]
                count = int(np.prod(entry["shape"], dtype=np.int64)) if entry["shape"] else 1
                if not (isinstance(begin, int) and isinstance(end, int)) or begin < 0 \
                        or end - begin != count * _ITEM_BYTES[entry["dtype"]] or end > data_bytes:
                    raise SafetensorsError(f"Invalid tensor offsets: {name}.")
                self.entries[name] = entry
            previous_end = 0
            for entry in sorted(self.entries.values(), key=lambda e: e["data_offsets"][0]):
                if entry["data_offsets"][0] != previous_end:
                    raise SafetensorsError("Safetensors data contains gaps or overlapping tensors.")
                previous_end = entry["data_offsets"][1]
            if previous_end != data_bytes:
                raise SafetensorsError("Safetensors data size does not match its header.")
            self._map = mmap.mmap(handle.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self):
        return self.entries.keys()

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(self.entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _TORCH_DTYPE[self.entries[name]["dtype"]]

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor in the stored dtype (a copy of the mapped bytes)."""
        entry = self.entries[name]
        begin, end = entry["data_offsets"]
        raw = np.frombuffer(self._map, dtype=np.uint8, count=end - begin, offset=self._start + begin)
        kind = entry["dtype"]
        if kind == "F32":
            out = torch.from_numpy(raw.view("<f4").copy())
        elif kind == "F16":
            out = torch.from_numpy(raw.view("<f2").copy())
        else:
            out = torch.from_numpy(raw.view("<u2").copy().view(np.int16)).view(torch.bfloat16)
        return out.reshape(entry["shape"])

    def close(self):
        if self._map is not None:
            self._map.close()
            self._map = None


def write_safetensors(path, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    """Write CPU tensors (float32, bfloat16 or float16) in the order given."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name, tensor in tensors.items():
        if tensor.dtype not in _NAME_OF:
            raise SafetensorsError(f"cannot store {tensor.dtype} for {name}")
        tensor = tensor.detach().cpu().contiguous()
        if tensor.dtype == torch.bfloat16:
            blob = tensor.view(torch.int16).numpy().tobytes()
        else:
            blob = tensor.numpy().tobytes()
        header[name] = {"dtype": _NAME_OF[tensor.dtype], "shape": list(tensor.shape),
                        "data_offsets": [offset, offset + len(blob)]}
        offset += len(blob)
        blobs.append(blob)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(text)))
        handle.write(text)
        for blob in blobs:
            handle.write(blob)
