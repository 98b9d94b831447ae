"""Helpers shared by the GPU parity tests: NumPy (ml_dtypes) <-> torch conversions and
seeded inputs with the benchmark configurations' distributions."""
import ml_dtypes
import numpy as np
import torch

BF16 = ml_dtypes.bfloat16
F8 = ml_dtypes.float8_e4m3fn


def to_torch_bf16(a: np.ndarray, device="cuda") -> torch.Tensor:
    a = np.ascontiguousarray(np.asarray(a).astype(BF16))
    return torch.from_numpy(a.view(np.int16)).to(device).view(torch.bfloat16)


def from_torch_bf16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).cpu().numpy().view(BF16)


def f8_bytes(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint8).cpu().numpy()


def f32(t: torch.Tensor) -> np.ndarray:
    return t.float().cpu().numpy()


def normal_bf16(rng, shape, std=1.0, outlier_p=0.0, outlier_mul=50.0):
    x = rng.standard_normal(shape).astype(np.float32) * np.float32(std)
    if outlier_p:
        x[rng.random(shape) < outlier_p] *= np.float32(outlier_mul)
    return x.astype(BF16)
