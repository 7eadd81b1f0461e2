"""Weight stores: load tensors by key, pack them on the GPU, cache by value name.

Mirrors `WeightStore` (cacheir/runtime/cpu.py:18-79) and `CudaWeightStore`
(cacheir/runtime/cuda.py:49-94): `get(name)` returns a dense tensor in the
runtime dtype (2-D weights are quantize->dequantize simulated when the
artifact is quantized, cpu.py:34-35); `get_quantized(name)` returns the packed
form. The pack itself runs on the device (`quantization.pack_weight_device`).
"""
from __future__ import annotations

from pathlib import Path
from typing import Any, Callable, Mapping

import numpy as np
import torch

from .quantization import B200PackedWeight, dequantize_device, pack_weight_device


class TensorSource:
    """Where raw tensors come from: an .npz file/directory, a mapping key -> array,
    or a callable key -> tensor (synthetic weights generated on the device)."""

    def __init__(self, source: str | Path | Mapping[str, Any] | Callable[[str, tuple[int, ...]], torch.Tensor]):
        self._npz: dict[str, np.ndarray] | None = None
        self._mapping: Mapping[str, Any] | None = None
        self._callable = None
        self._path: Path | None = None
        if callable(source):
            self._callable = source
        elif isinstance(source, Mapping):
            self._mapping = source
        else:
            self._path = Path(source)

    def load(self, key: str, shape: tuple[int, ...], file: str | None) -> Any:
        if self._callable is not None:
            return self._callable(key, shape)
        if self._mapping is not None:
            return self._mapping[key]
        path = self._path
        assert path is not None
        if path.is_file() and path.suffix == ".npz":
            npz_path = path
        elif path.is_dir():
            npz_path = path / (file or "weights.npz")
        else:
            raise FileNotFoundError(f"could not load weight {key!r} from {path}")
        if npz_path.suffix != ".npz" or not npz_path.exists():
            raise FileNotFoundError(f"cacheir_b200 loads .npz weights; {npz_path} not found")
        if self._npz is None:
            with np.load(npz_path) as data:
                self._npz = {k: data[k] for k in data.files}
        return self._npz[key]


class B200WeightStore:
    def __init__(self, source: TensorSource, specs: Mapping[str, Any], quant: str | None, *, device: torch.device,
                 dtype: torch.dtype):
        self.source = source
        self.specs = specs
        self.quant = quant
        self.device = device
        self.dtype = dtype
        self._cache: dict[str, torch.Tensor] = {}
        self._qcache: dict[str, B200PackedWeight] = {}

    def _raw_fp32(self, value_name: str) -> torch.Tensor:
        spec = self.specs[value_name]
        shape = tuple(getattr(spec, "shape", None) or getattr(getattr(spec, "tensor_type", None), "shape", ()) or ())
        raw = self.source.load(spec.key, shape, getattr(spec, "file", None))
        if isinstance(raw, torch.Tensor):
            return raw.to(device=self.device, dtype=torch.float32)
        return torch.from_numpy(np.ascontiguousarray(np.asarray(raw, dtype=np.float32))).to(self.device)

    def get(self, value_name: str) -> torch.Tensor:
        if value_name not in self._cache:
            tensor = self._raw_fp32(value_name)
            if self.quant and tensor.dim() == 2:
                # quantize -> dequantize simulation of a non-matmul 2-D weight; the pack is not kept
                packed = pack_weight_device(tensor.contiguous(), self.quant)
                if packed is None:
                    raise ValueError(f"Unsupported quantization mode {self.quant!r}")
                tensor = dequantize_device(packed, self.dtype)
            self._cache[value_name] = tensor.to(self.dtype).contiguous()
        return self._cache[value_name]

    def get_quantized(self, value_name: str) -> B200PackedWeight:
        if value_name not in self._qcache:
            tensor = self._raw_fp32(value_name)
            if tensor.dim() != 2:
                raise ValueError(f"Weight {value_name!r} is not a 2D matrix and cannot be packed")
            self._pack(value_name, tensor)
        return self._qcache[value_name]

    def _pack(self, value_name: str, tensor: torch.Tensor) -> B200PackedWeight:
        if value_name not in self._qcache:
            packed = pack_weight_device(tensor.contiguous(), self.quant)
            if packed is None:
                raise ValueError(f"Unsupported quantization mode {self.quant!r}")
            self._qcache[value_name] = packed
        return self._qcache[value_name]

    def put_quantized(self, value_name: str, packed: B200PackedWeight) -> None:
        """Install an already packed weight (e.g. group-wise int4 codes made elsewhere)."""
        self._qcache[value_name] = packed

    def release(self, value_name: str) -> None:
        """Forget the cached copies of a weight (its owner keeps a fused form)."""
        self._cache.pop(value_name, None)
        self._qcache.pop(value_name, None)
