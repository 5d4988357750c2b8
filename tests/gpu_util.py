"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch


def dev_bf16(bits: np.ndarray) -> torch.Tensor:
    """uint16 bf16 bit patterns -> cuda bfloat16 tensor of the same shape."""
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda().view(torch.bfloat16)


def host_bits(t: torch.Tensor) -> np.ndarray:
    """cuda bfloat16 tensor -> uint16 bit patterns."""
    return t.detach().view(torch.int16).cpu().numpy().view(np.uint16)


def rel_err(got: np.ndarray, ref: np.ndarray) -> float:
    """max|got-ref| / max|ref|, the reference gates' metric (tests/gate_gemv.cu:113-115);
    non-finite values are flagged explicitly instead of being swallowed by max()."""
    got = np.asarray(got, np.float64)
    assert np.all(np.isfinite(got)), "non-finite values in the GPU result"
    return float(np.max(np.abs(got - ref)) / max(np.max(np.abs(ref)), 1e-30))


def bf16_ulp(ref: np.ndarray) -> np.ndarray:
    """one bf16 ulp at |ref| (8 significant bits)."""
    a = np.maximum(np.abs(np.asarray(ref, np.float64)), 2.0 ** -126)
    return 2.0 ** (np.floor(np.log2(a)) - 7)


class Guarded:
    """A device buffer with canary bands on both sides, to catch out-of-bounds writes."""

    def __init__(self, shape, dtype, band=256, fill=0):
        n = int(np.prod(shape))
        self.band, self.n, self.dtype = band, n, dtype
        self.raw = torch.empty(n + 2 * band, dtype=dtype, device="cuda")
        self.pattern = 0x5A if dtype in (torch.int8, torch.uint8) else None
        self.raw.view(torch.uint8).fill_(0x5A)
        self.t = self.raw[band:band + n].view(shape)
        if fill is not None:
            self.t.zero_()

    def intact(self) -> bool:
        b = self.raw.view(torch.uint8)
        es = self.raw.element_size()
        lo, hi = b[: self.band * es], b[(self.band + self.n) * es:]
        return bool((lo == 0x5A).all().item() and (hi == 0x5A).all().item())
