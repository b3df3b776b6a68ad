"""Synthetic fp32 data sets, seeded, generated on the requested device.

``sinusoid_field``  sum of 3 unit sinusoids with random frequencies in [1, 50] cycles plus
                    N(0, 1e-3) noise (the smooth 1-D field of the message-size sweep)
``blob_field_3d``   sum of 8 Gaussian blobs (sigma 20-80 voxels, amplitudes U[-1, 1]) plus
                    N(0, 1e-4) noise on a 3-D grid (single-GPU codec throughput)
``gradient_like``   N(0, 0.01) with 1 % of the entries scaled x10 (heavy-tailed gradients)
``from_distribution`` the generator of the reference's dataset script: uniform / normal /
                    exponential / randomwalk with optional box smoothing
                    (HomComp/src/utils/dataset_generator.py:34-49)
"""
from __future__ import annotations

import math

import torch


def _gen(device, seed):
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def sinusoid_field(n: int, seed: int = 0, device="cpu", noise: float = 1e-3) -> torch.Tensor:
    g = _gen("cpu", seed)
    freqs = torch.empty(3).uniform_(1.0, 50.0, generator=g)
    phases = torch.empty(3).uniform_(0.0, 2 * math.pi, generator=g)
    t = torch.arange(n, device=device, dtype=torch.float32) / max(n, 1)
    x = torch.zeros(n, device=device, dtype=torch.float32)
    for f, p in zip(freqs.tolist(), phases.tolist()):
        x += torch.sin(2 * math.pi * f * t + p)
    if noise:
        x += torch.randn(n, device=device, generator=_gen(device, seed + 1)) * noise
    return x


def blob_field_3d(shape=(512, 512, 256), seed: int = 0, device="cpu", noise: float = 1e-4) -> torch.Tensor:
    g = _gen("cpu", seed)
    nz, ny, nx = shape
    z = torch.arange(nz, device=device, dtype=torch.float32).view(nz, 1, 1)
    y = torch.arange(ny, device=device, dtype=torch.float32).view(1, ny, 1)
    x = torch.arange(nx, device=device, dtype=torch.float32).view(1, 1, nx)
    out = torch.zeros(shape, device=device, dtype=torch.float32)
    for _ in range(8):
        c = torch.rand(3, generator=g)
        sigma = float(torch.empty(1).uniform_(20.0, 80.0, generator=g))
        amp = float(torch.empty(1).uniform_(-1.0, 1.0, generator=g))
        cz, cy, cx = float(c[0]) * nz, float(c[1]) * ny, float(c[2]) * nx
        k = -0.5 / (sigma * sigma)
        # separable Gaussian: three 1-D factors, one fused broadcast product
        out += amp * (torch.exp(k * (z - cz) ** 2) * torch.exp(k * (y - cy) ** 2) * torch.exp(k * (x - cx) ** 2))
    if noise:
        out += torch.randn(shape, device=device, generator=_gen(device, seed + 1)) * noise
    return out.reshape(-1)


def gradient_like(n: int, seed: int = 0, device="cpu") -> torch.Tensor:
    g = _gen(device, seed)
    x = torch.randn(n, device=device, generator=g) * 0.01
    mask = torch.rand(n, device=device, generator=g) < 0.01
    return torch.where(mask, x * 10.0, x)


def from_distribution(n: int, dist: str = "uniform", seed: int = 0, device="cpu", mean=0.0, std=1.0, low=0.0,
                      high=1.0, scale=1.0, rw_mean=0.0, rw_std=1.0, smooth: bool = False,
                      kernel_size: int = 5) -> torch.Tensor:
    g = _gen(device, seed)
    x = torch.empty(n, device=device, dtype=torch.float32)
    if dist == "uniform":
        x.uniform_(low, high, generator=g)
    elif dist == "normal":
        x.normal_(mean, std, generator=g)
    elif dist == "exponential":
        x.exponential_(scale, generator=g)
    elif dist == "randomwalk":
        x.normal_(rw_mean, rw_std, generator=g)
        x = torch.cumsum(x, dim=0)
    else:
        raise ValueError("unknown distribution %r" % dist)
    if smooth and kernel_size > 1 and kernel_size % 2 == 1:
        k = torch.full((1, 1, kernel_size), 1.0 / kernel_size, device=device)
        x = torch.nn.functional.conv1d(x.view(1, 1, -1), k, padding=kernel_size // 2).view(-1)
    return x
