"""Small helpers for the GPU parity tests: host<->device moves and bit-exact
comparison with useful failure output."""
import numpy as np
import torch


def dev(array, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(array))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def host(tensor) -> np.ndarray:
    return tensor.detach().cpu().numpy()


def bf16_dev(bits: np.ndarray):
    """uint16 bit patterns -> a CUDA tensor of the same bits (stored as int16)."""
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda()


def bf16_host(tensor) -> np.ndarray:
    return tensor.detach().cpu().numpy().view(np.uint16)


def assert_bits_equal(actual: np.ndarray, expected: np.ndarray, what: str) -> None:
    a = np.ascontiguousarray(actual)
    e = np.ascontiguousarray(expected)
    assert a.shape == e.shape, f"{what}: shape {a.shape} != {e.shape}"
    both_nan = None
    if a.dtype.kind == "f":
        # a NaN is a NaN: x86 keeps an operand's payload where the GPU returns
        # the canonical pattern, and no consumer distinguishes them
        both_nan = np.isnan(a) & np.isnan(e)
        a = a.view(np.uint32 if a.dtype.itemsize == 4 else np.uint64)
        e = e.view(np.uint32 if e.dtype.itemsize == 4 else np.uint64)
    differs = a != e
    if both_nan is not None:
        differs &= ~both_nan.ravel().reshape(differs.shape)
    bad = np.nonzero(differs)[0]
    assert bad.size == 0, (f"{what}: {bad.size} of {a.size} differ; first at {bad[0]}: "
                           f"got {actual.ravel()[bad[0]]!r}, expected {expected.ravel()[bad[0]]!r}")


def misaligned(n: int, dtype, offset_elements: int = 1):
    """A device tensor whose first element is offset from the allocation's
    (256-byte aligned) base."""
    base = torch.zeros(n + offset_elements + 64, dtype=dtype, device="cuda")
    return base[offset_elements:offset_elements + n]
