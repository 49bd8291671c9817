"""`ModelLoader::load_llama_weights` (src/loader.rs:10-80): fill a model's named parameters from a
`.safetensors` file.

Same behaviour as the reference: the file is memory-mapped, every parameter of the model is looked up
by its Hugging Face name, F32 and BF16 tensors are accepted (anything else is an error), a parameter
missing from the file is reported and skipped, a size mismatch is an error.  Unlike the reference a
BF16 tensor is not widened on the host: its bits go to the device as they are (the library widens
them when the model stores f32 weights, and keeps them when it stores bf16).

The container format (safetensors 0.3, the version the reference pins in Cargo.toml:16) is an 8-byte
little-endian header length, a JSON header {name: {dtype, shape, data_offsets}}, then the raw
little-endian tensor data.
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path

import numpy as np

_DTYPES = {"F32": (np.float32, 4), "BF16": (np.uint16, 2)}


class SafeTensorsFile:
    """A memory-mapped safetensors file: `names()`, `tensor(name) -> (dtype_str, shape, array view)`."""

    def __init__(self, path):
        self.path = Path(path)
        self._f = open(self.path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        if len(self._mm) < 8:
            raise ValueError(f"{self.path}: too short for a safetensors header")
        (hlen,) = struct.unpack("<Q", self._mm[:8])
        if 8 + hlen > len(self._mm):
            raise ValueError(f"{self.path}: header length {hlen} exceeds the file")
        self._base = 8 + hlen
        self._meta = {k: v for k, v in json.loads(self._mm[8:8 + hlen].decode("utf-8")).items() if k != "__metadata__"}

    def names(self):
        return list(self._meta)

    def tensor(self, name: str):
        info = self._meta[name]
        dt = info["dtype"]
        if dt not in _DTYPES:
            raise ValueError(f"Unsupported dtype: {dt} for {name}")  # loader.rs:67
        npdt, esz = _DTYPES[dt]
        shape = tuple(int(d) for d in info["shape"])
        b, e = info["data_offsets"]
        n = int(np.prod(shape)) if shape else 1
        if e - b != n * esz:
            raise ValueError(f"{name}: {e - b} bytes do not match shape {shape}")
        arr = np.frombuffer(self._mm, dtype=npdt, count=n, offset=self._base + b).reshape(shape)
        return dt, shape, arr

    def close(self):
        self._mm.close()
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        try:
            self.close()
        except BufferError:  # views handed out are still alive; the map goes with them
            pass


def load_llama_weights(path, model, verbose: bool = False) -> list:
    """Fill `model` (a `LlamaModel`) from `path`.  Returns the names that were not found in the file."""
    missing = []
    with SafeTensorsFile(path) as f:
        present = set(f.names())
        for name, shape in model.config.param_shapes().items():
            if name not in present:
                missing.append(name)  # loader.rs:72-77: warn and go on
                if verbose:
                    print(f"Warning: Parameter {name} not found in safetensors file")
                continue
            dt, fshape, arr = f.tensor(name)
            if int(np.prod(fshape)) != int(np.prod(shape)):
                raise ValueError(f"Shape mismatch for {name}: file {fshape}, model {tuple(shape)}")  # loader.rs:45,61
            model.set_param(name, arr.reshape(shape), as_bf16_bits=(dt == "BF16"))
            if verbose:
                print(f"Loaded: {name}")
    return missing


def save_safetensors(path, tensors: dict) -> None:
    """Write {name: f32 array | uint16 array of bf16 bits} in the safetensors container (for tests and for
    exporting synthetic checkpoints)."""
    header, blobs, off = {}, [], 0
    for name, a in tensors.items():
        a = np.ascontiguousarray(a)
        if a.dtype == np.float32:
            dt = "F32"
        elif a.dtype == np.uint16:
            dt = "BF16"
        else:
            raise ValueError(f"{name}: only f32 and bf16-bit (uint16) arrays can be written")
        raw = a.tobytes()
        header[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for raw in blobs:
            f.write(raw)
