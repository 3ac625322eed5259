"""Helpers for the GPU parity tests: numpy bit patterns <-> device tensors, and
the error measure the tolerances in these tests refer to."""
import numpy as np
import torch

TORCH_16 = {"f16": torch.float16, "bf16": torch.bfloat16}


def to_dev_16(bits: np.ndarray, dtype: str) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda().view(TORCH_16[dtype])


def to_dev_e4m3(u8: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(u8)).cuda().view(torch.float8_e4m3fn)


def to_dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits_of(t: torch.Tensor) -> np.ndarray:
    if t.element_size() == 2:
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    if t.element_size() == 1:
        return t.view(torch.uint8).cpu().numpy()
    raise ValueError(t.dtype)


def poisoned(shape, dtype: str) -> torch.Tensor:
    """Output buffer pre-filled with NaN so an unwritten tile cannot pass."""
    return torch.full(shape, float("nan"), dtype=TORCH_16[dtype], device="cuda")


def max_rel_err(got: np.ndarray, ref: np.ndarray, floor: float) -> float:
    """max |got-ref| / max(|ref|, floor): relative error with an absolute floor
    for outputs that cancel to (almost) zero."""
    got = got.astype(np.float64)
    ref = ref.astype(np.float64)
    assert np.isfinite(got).all(), "non-finite output (unwritten tile or overflow)"
    return float((np.abs(got - ref) / np.maximum(np.abs(ref), floor)).max())
