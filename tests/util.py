"""Shared helpers for the GPU parity tests."""
import numpy as np
import torch


def dev(a, device="cuda:0"):
    """numpy -> CUDA tensor (fp32 arrays holding fp16 values are sent as fp16 when asked)."""
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


def dev16(a, device="cuda:0"):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.float16).to(device)


def host(t):
    t = t.detach().cpu()
    if t.dtype == torch.float16:
        return t.float().numpy()
    return t.numpy()


def code_mismatch_fraction(a, b):
    a = np.asarray(a)
    b = np.asarray(b)
    return float(np.mean(a != b))


def nrmse(actual, expected):
    """Normalised RMSE, the reference's layer-stack metric (src/cuda/encoder.rs:204-239)."""
    actual = np.asarray(actual, dtype=np.float64)
    expected = np.asarray(expected, dtype=np.float64)
    return float(np.sqrt(np.mean((actual - expected) ** 2)) / (np.sqrt(np.mean(expected ** 2)) + 1e-30))
