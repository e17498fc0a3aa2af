"""Seeded random-init weights and the `-split-params` writer for them.

nncv's `-split-params` (src/nncv/compiler/Conversion/Transforms/SplitParamsFlatArray.cpp:99-206,
writer src/nncv/compiler/Utils/BinaryParams.cpp:45-78) dumps every constant of the model into one
container file beside the compiled object.  The fixtures of the reference carry elided weights,
so the weights here are seeded random tensors with the distributions the benchmark configs name:
conv Kaiming-normal (fan_in, ReLU gain); BN gamma~U[0.5,1.5], beta~N(0,0.1), running_mean~N(0,0.1),
running_var~U[0.5,1.5]; FC weight and bias ~U(-1/sqrt(fan_in), 1/sqrt(fan_in)).
One Philox stream per tensor, keyed by (seed, crc32(name)), generated in fp32 and cast after.
"""
from __future__ import annotations

import math
import zlib
from typing import Dict

import numpy as np

from .memref import MemRefFlatArray
from .netspec import conv_groups, fc_in, tensor_order


def _rng(seed: int, name: str) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=[seed, zlib.crc32(name.encode())]))


def random_state_dict(depth: int, seed: int = 0) -> Dict[str, np.ndarray]:
    """fp32 tensors keyed by state-dict name."""
    sd: Dict[str, np.ndarray] = {}
    for g in conv_groups(depth):
        fan_in = g.cin * g.k * g.k
        sd[f"{g.name}.weight"] = (_rng(seed, f"{g.name}.weight").standard_normal(
            (g.cout, g.cin, g.k, g.k), dtype=np.float32) * np.float32(math.sqrt(2.0 / fan_in)))
        sd[f"{g.bn}.weight"] = _rng(seed, f"{g.bn}.weight").uniform(0.5, 1.5, g.cout).astype(np.float32)
        sd[f"{g.bn}.bias"] = (_rng(seed, f"{g.bn}.bias").standard_normal(g.cout, dtype=np.float32) * np.float32(0.1))
        sd[f"{g.bn}.running_mean"] = (_rng(seed, f"{g.bn}.running_mean").standard_normal(g.cout, dtype=np.float32) * np.float32(0.1))
        sd[f"{g.bn}.running_var"] = _rng(seed, f"{g.bn}.running_var").uniform(0.5, 1.5, g.cout).astype(np.float32)
    bound = 1.0 / math.sqrt(fc_in(depth))
    sd["fc.weight"] = _rng(seed, "fc.weight").uniform(-bound, bound, (1000, fc_in(depth))).astype(np.float32)
    sd["fc.bias"] = _rng(seed, "fc.bias").uniform(-bound, bound, 1000).astype(np.float32)
    return sd


def to_flat_array(depth: int, state_dict: Dict[str, np.ndarray], dtype=np.float32) -> MemRefFlatArray:
    """Pack a state dict into the container in the reference's tensor order."""
    arr = MemRefFlatArray(np.dtype(dtype).itemsize)
    for name, shape in tensor_order(depth):
        t = state_dict[name]
        if tuple(t.shape) != shape:
            raise ValueError(f"{name}: shape {t.shape} != {shape}")
        arr.add(name, t.astype(dtype))
    return arr


def write_model_bin(path: str, depth: int, seed: int = 0, dtype=np.float32) -> MemRefFlatArray:
    arr = to_flat_array(depth, random_state_dict(depth, seed), dtype)
    arr.write(path)
    return arr


def random_input(n: int, h: int, w: int, seed: int = 0, dist: str = "uniform") -> np.ndarray:
    """NCHW fp32 input: U[0,1) (the fp32 config) or N(0,1) (the fp16 configs)."""
    g = _rng(seed, f"input.{n}x3x{h}x{w}.{dist}")
    if dist == "uniform":
        return g.random((n, 3, h, w), dtype=np.float32)
    return g.standard_normal((n, 3, h, w), dtype=np.float32)
