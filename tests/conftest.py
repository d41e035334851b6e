import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (runs the sm_100a kernels through the C ABI)")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (test infrastructure), built on demand."""
    from oracle import lokal_oracle
    lokal_oracle.build()
    lokal_oracle.lib()
    return lokal_oracle


@pytest.fixture(scope="session")
def ctx():
    """One lokal_cuda context on cuda:0. Fails loudly when the library or the device is missing."""
    import torch
    assert torch.cuda.is_available(), "gpu-marked test running without a CUDA device"
    import lokal_b200
    torch.cuda.set_device(0)
    c = lokal_b200.Context(0)
    yield c
    c.close()


class Dev:
    """numpy <-> device helpers; torch is only the allocator here."""

    def __init__(self):
        import torch
        self.torch = torch
        self.tdt = {0: torch.float32, 1: torch.float16, 30: torch.bfloat16}

    def put(self, a, dtype=0):
        t = self.torch.from_numpy(np.ascontiguousarray(a))
        if a.dtype == np.float32 and dtype != 0:
            t = t.to(self.tdt[dtype])
        return t.cuda()

    def empty(self, shape, dtype=0, fill=None):
        t = self.torch.empty(shape, dtype=self.tdt[dtype], device="cuda")
        if fill is not None:
            t.fill_(fill)
        return t

    def get(self, t):
        """Device tensor -> numpy f32 (exact widening for 16-bit types)."""
        self.torch.cuda.synchronize()
        return t.detach().to(self.torch.float32).cpu().numpy()

    def bits16(self, t):
        self.torch.cuda.synchronize()
        return t.detach().view(self.torch.uint16).cpu().numpy() if hasattr(self.torch, "uint16") else \
            t.detach().view(self.torch.int16).cpu().numpy().view(np.uint16)


@pytest.fixture(scope="session")
def dev():
    return Dev()
