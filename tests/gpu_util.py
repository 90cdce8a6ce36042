"""Helpers for the GPU parity tests: device buffers via torch, calls through the C ABI."""
import ctypes as C

import numpy as np
import torch

from decidra_b200 import _lib

DT = {0: torch.float32, 1: torch.bfloat16}


def dev(a, dtype: int):
    """numpy f32 -> CUDA tensor of the storage type."""
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda().to(DT[dtype]).contiguous()


def devi(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).cuda()


def devf(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


def host(t) -> np.ndarray:
    return t.float().cpu().numpy()


def empty(shape, dtype: int):
    return torch.empty(shape, dtype=DT[dtype], device="cuda")


def p(t):
    """Identity marker for a device-pointer argument: `call` turns tensors into pointers while the
    argument tuple keeps them alive (a pointer taken from a temporary tensor would dangle)."""
    return t


def call(name, *args):
    conv = [C.c_void_p(a.data_ptr()) if isinstance(a, torch.Tensor) else a for a in args]
    rc = getattr(_lib.load(), name)(*conv)
    torch.cuda.synchronize()
    assert rc == 0, f"{name} returned {rc}"


def tol(dtype: int):
    """(rtol, atol) for one elementwise op: f32 rounding noise, or one bf16 ulp."""
    return (2e-5, 2e-6) if dtype == 0 else (8e-3, 1e-3)


def sm_count() -> int:
    return torch.cuda.get_device_properties(0).multi_processor_count
