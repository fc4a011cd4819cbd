"""Export a trained model to one self-describing weight file for deployment, optionally with int8 weights, and load it back.

Counterpart of the exporters of the reference's LightSeq subset (oslo/lightseq2/training/ops/pytorch/export.py:7-400,
export_quant.py: protobuf / HDF5 files read by the inference engine).  Neither ``h5py`` nor a protobuf compiler is part of
this stack, so the container is a flat binary::

    b"OSLOLSW1" | u64 header bytes | JSON header | zero padding to 64 B | tensor data (each 64-byte aligned)

The header holds the model configuration, free-form metadata and, per tensor, ``dtype``, ``shape``, ``offset``, ``nbytes``
and for quantised tensors the clip value (``x ~ q * clip / 127``).  ``quantize=True`` stores every floating-point matrix
(>= 2 dimensions) as symmetric per-tensor int8 with its clip value; vectors (biases, norms) stay in their dtype.  The file
is read with ``numpy.memmap`` so loading touches only what is asked for.
"""
from __future__ import annotations

import json
import struct
from dataclasses import asdict, is_dataclass
from typing import Dict, Optional, Tuple

import numpy as np
import torch

MAGIC = b"OSLOLSW1"
_ALIGN = 64
_NP = {"float32": np.float32, "float16": np.float16, "bfloat16": np.uint16, "int8": np.int8, "int32": np.int32,
       "int64": np.int64, "uint8": np.uint8, "bool": np.bool_}
_TORCH = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16, "int8": torch.int8,
          "int32": torch.int32, "int64": torch.int64, "uint8": torch.uint8, "bool": torch.bool}


def _config_dict(config) -> dict:
    if config is None:
        return {}
    if is_dataclass(config):
        return asdict(config)
    if hasattr(config, "to_dict"):
        return config.to_dict()
    return dict(vars(config))


def _raw(t: torch.Tensor) -> Tuple[bytes, str]:
    name = str(t.dtype).replace("torch.", "")
    if name not in _NP:
        raise TypeError(f"unsupported dtype {t.dtype}")
    t = t.detach().contiguous().cpu()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().tobytes(), name
    return t.numpy().tobytes(), name


def export_model(model_or_state, path: str, config=None, quantize: bool = False, metadata: Optional[dict] = None) -> dict:
    """Write ``model_or_state`` (a module or a state dict) to ``path``; returns the header that was written."""
    state = model_or_state.state_dict() if hasattr(model_or_state, "state_dict") else dict(model_or_state)
    if config is None and hasattr(model_or_state, "config"):
        config = model_or_state.config
    from .kernels import ls_quantize_int8

    blobs, tensors, offset, seen = [], {}, 0, {}
    for name, t in state.items():
        key = (t.data_ptr(), tuple(t.shape), t.dtype)
        if key in seen and t.numel() > 0:  # tied weights are stored once
            tensors[name] = {"alias": seen[key]}
            continue
        seen[key] = name
        entry = {"shape": list(t.shape)}
        if quantize and t.is_floating_point() and t.dim() >= 2:
            clip = float(t.detach().abs().max().clamp(min=1e-8))
            q = ls_quantize_int8(t.detach(), clip)
            raw, dtype = _raw(q)
            entry.update(dtype=dtype, clip=clip, orig_dtype=str(t.dtype).replace("torch.", ""))
        else:
            raw, dtype = _raw(t)
            entry.update(dtype=dtype)
        pad = (-len(raw)) % _ALIGN
        entry.update(offset=offset, nbytes=len(raw))
        offset += len(raw) + pad
        blobs.append(raw + b"\0" * pad)
        tensors[name] = entry
    header = {"format": 1, "model_class": type(model_or_state).__name__, "config": _config_dict(config),
              "quantized": bool(quantize), "metadata": metadata or {}, "tensors": tensors}
    hb = json.dumps(header, sort_keys=True, default=str).encode()
    with open(path, "wb") as f:
        f.write(MAGIC)
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        f.write(b"\0" * ((-(len(MAGIC) + 8 + len(hb))) % _ALIGN))
        for b in blobs:
            f.write(b)
    return header


def read_header(path: str) -> Tuple[dict, int]:
    """Returns ``(header, offset of the tensor data)``."""
    with open(path, "rb") as f:
        if f.read(len(MAGIC)) != MAGIC:
            raise ValueError(f"{path} is not an exported weight file")
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
    base = len(MAGIC) + 8 + n
    return header, base + (-base) % _ALIGN


def load_exported(path: str, device="cpu", dequantize: bool = True) -> Tuple[Dict[str, torch.Tensor], dict]:
    """Returns ``(state_dict, header)``.  Quantised tensors come back in their original dtype (``dequantize=True``) or as
    int8 tensors with ``header["tensors"][name]["clip"]`` giving the scale."""
    header, base = read_header(path)
    data = np.memmap(path, dtype=np.uint8, mode="r", offset=base) if any("offset" in e for e in header["tensors"].values()) else None
    out: Dict[str, torch.Tensor] = {}
    for name, e in header["tensors"].items():
        if "alias" in e:
            continue
        raw = np.array(data[e["offset"] : e["offset"] + e["nbytes"]])  # copy out of the map
        arr = raw.view(_NP[e["dtype"]])
        t = torch.from_numpy(arr)
        if e["dtype"] == "bfloat16":
            t = t.view(torch.int16).view(torch.bfloat16)
        t = t.reshape(e["shape"]).to(device)
        if "clip" in e and dequantize:
            t = (t.float() * (e["clip"] / 127.0)).to(_TORCH[e["orig_dtype"]])
        out[name] = t
    for name, e in header["tensors"].items():
        if "alias" in e:
            out[name] = out[e["alias"]]
    return out, header


def import_into(model: torch.nn.Module, path: str, strict: bool = True) -> dict:
    """Load an exported file into ``model`` (dequantising int8 tensors); returns the header."""
    state, header = load_exported(path, device="cpu", dequantize=True)
    model.load_state_dict(state, strict=strict)
    return header


__all__ = ["export_model", "load_exported", "import_into", "read_header", "MAGIC"]
