"""Helpers shared by the tests: seeded inputs and torch <-> bit-pattern views."""
import numpy as np
import torch


def bits(t: torch.Tensor) -> np.ndarray:
    """Storage view of a CPU tensor: uint16 for f16/bf16, uint8 for f8, float32 otherwise
    (strides preserved)."""
    t = t.detach().cpu()
    if t.dtype == torch.float32:
        return t.numpy()
    if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        return t.view(torch.uint8).numpy()
    return t.view(torch.int16).numpy().view(np.uint16)


def code(dt) -> int:
    return {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2, torch.float8_e4m3fn: 3,
            torch.float8_e5m2: 4}[dt]


def gen(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(seed)


def normal(shape, seed, std=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, generator=gen(seed)) * std).to(dtype)


def uniform(shape, seed, lo=-1.0, hi=1.0, dtype=torch.float16):
    return (torch.rand(*shape, generator=gen(seed)) * (hi - lo) + lo).to(dtype)
