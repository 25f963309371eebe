import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with `-m gpu` on a B200")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def mojo_registered():
    import torch_mojo_backend_b200 as tmb

    tmb.register_mojo_devices()
    return tmb


class BridgeSpy:
    """Records every call that would reach the native library (host-wiring tests)."""

    def __init__(self):
        self.calls = []

    def fwd(self, q, k, v, out, lse_ptr, dtype, causal, scale, stream, device, status_ptr=0, *, simt=False,
            dropout=None):
        self.calls.append(("fwd", dict(q=q, k=k, v=v, out=out, lse_ptr=lse_ptr, dtype=dtype, causal=causal,
                                       scale=scale, stream=stream, device=device, status_ptr=status_ptr,
                                       dropout=dropout)))
        return 0

    def bwd(self, q, k, v, out, dout, lse_ptr, dq, dk, dv, workspace_ptr, workspace_bytes, dtype, causal, scale,
            stream, device, status_ptr=0, *, simt=False, parts=7, dropout=None):
        self.calls.append(("bwd", dict(q=q, k=k, v=v, out=out, dout=dout, lse_ptr=lse_ptr, dq=dq, dk=dk, dv=dv,
                                       workspace_ptr=workspace_ptr, workspace_bytes=workspace_bytes, dtype=dtype,
                                       causal=causal, scale=scale, stream=stream, device=device,
                                       status_ptr=status_ptr, dropout=dropout)))
        return 0

    def fwd_splitkv(self, q, k, v, out, lse_ptr, workspace_ptr, workspace_bytes, dtype, causal, scale, stream,
                    device, status_ptr=0):
        self.calls.append(("fwd_splitkv", dict(q=q, k=k, v=v, out=out, lse_ptr=lse_ptr, workspace_ptr=workspace_ptr,
                                               workspace_bytes=workspace_bytes, dtype=dtype, causal=causal,
                                               scale=scale, stream=stream, device=device)))
        return 0


@pytest.fixture
def host_backed_mojo(mojo_registered, monkeypatch):
    """The mojo device with allocations redirected to host memory and the native bridge
    replaced by a spy, so the Python host code can be exercised without a GPU (the role of the
    reference's fake_mojo_tensor fixture, tests/conftest.py:121-169)."""
    from torch_mojo_backend_b200 import _lib, flash_ops, tensor

    allocations = []

    def alloc(nbytes, index):
        t = torch.empty((max(int(nbytes), 1),), dtype=torch.uint8)
        allocations.append(int(nbytes))
        return t

    spy = BridgeSpy()
    monkeypatch.setattr(tensor, "_alloc_holder", alloc)
    monkeypatch.setattr(flash_ops, "_stream_for", lambda index: 0)
    monkeypatch.setattr(_lib, "fwd", spy.fwd)
    monkeypatch.setattr(_lib, "bwd", spy.bwd)
    monkeypatch.setattr(_lib, "fwd_splitkv", spy.fwd_splitkv)
    # the per-device status word lives in (redirected) host memory for the duration of the test
    monkeypatch.setattr(flash_ops, "_status_words", {})
    spy.status_ptr = flash_ops._status_ptr(0)
    spy.allocations = allocations
    return spy
