"""Inputs for the GPU tests with poisoned guard bands.

A kernel that reads outside an operand and USES what it read must not pass by luck (allocator padding is
often zero): every input goes to the device inside a larger buffer whose bands before and after it hold
NaN (fp32, bf16) or a wild integer. The bands are a multiple of 256 bytes, so the operand keeps the
alignment a fresh allocation has. Outputs have their own canary bands (written bytes are checked); this
is the read-side counterpart, and together they stand in for a memory checker.
"""
import numpy as np
import torch

BAND = 256  # elements on each side


def guarded_input(a: np.ndarray, dev) -> torch.Tensor:
    """numpy -> device inside poisoned bands; uint16 arrays are bf16 bit patterns, uint32 stays uint32."""
    a = np.ascontiguousarray(a)
    n = a.size
    if a.dtype == np.uint16:
        host = np.full(n + 2 * BAND, 0x7FC0, dtype=np.uint16)          # bf16 NaN
        host[BAND:BAND + n] = a.reshape(-1)
        return torch.from_numpy(host.view(np.int16)).to(dev).view(torch.bfloat16)[BAND:BAND + n].view(*a.shape)
    if a.dtype == np.uint32:
        host = np.full(n + 2 * BAND, 0x7F7F7F7F, dtype=np.uint32)
        host[BAND:BAND + n] = a.reshape(-1)
        return torch.from_numpy(host.view(np.int32)).to(dev).view(torch.uint32)[BAND:BAND + n].view(*a.shape)
    if a.dtype == np.int32:
        host = np.full(n + 2 * BAND, 0x7F7F7F7F, dtype=np.int32)
    elif a.dtype == np.float32:
        host = np.full(n + 2 * BAND, np.nan, dtype=np.float32)
    else:
        return torch.from_numpy(a).to(dev)
    host[BAND:BAND + n] = a.reshape(-1)
    return torch.from_numpy(host).to(dev)[BAND:BAND + n].view(*a.shape)
