"""The allocation-free backward entry point, `b200fa_bwd_no_alloc` (``-m gpu``).

Some hosts of the library cannot hand it scratch memory: they only forward device pointers
that another runtime owns, or they run the backward where allocating is forbidden (an
allocator that must not be re-entered, a serving loop that is already warm).  For them the
backward's scratch is a fixed array inside the library.  This test calls that entry point
through the C ABI, twice in a row on different inputs (the array keeps the first call's
contents, so the second call proves the kernels clear what they need), and compares with the
ordinary `b200fa_bwd`: dQ/dK/dV bit for bit (the kernels are deterministic; the 16-bit tolerance
is asserted as well).  It also checks that an oversized problem is refused
before anything is launched.  The file sorts last so a run that stops at the first failure has
already run every other test."""

import pytest
import torch

from tests.helpers import TOL_16BIT, assert_within
from torch_mojo_backend_b200 import _lib, raw

pytestmark = pytest.mark.gpu


def _case(seed, B, Hq, Hkv, S, D, dtype, causal):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, Hq, S, D, generator=g) * 0.5).to(dtype).cuda()
    k = (torch.randn(B, Hkv, S, D, generator=g) * 0.5).to(dtype).cuda()
    v = (torch.randn(B, Hkv, S, D, generator=g) * 0.5).to(dtype).cuda()
    dout = torch.randn(B, Hq, S, D, generator=g).to(dtype).cuda()
    out, lse = raw.flash_fwd(q, k, v, causal=causal)
    return q, k, v, dout, out, lse


def _no_alloc_backward(q, k, v, dout, out, lse, causal):
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    dev = q.device.index or 0
    rc = _lib.bwd_no_alloc(raw.t4(q), raw.t4(k), raw.t4(v), raw.t4(out), raw.t4(dout), lse.data_ptr(), raw.t4(dq),
                           raw.t4(dk), raw.t4(dv), raw.dtype_code(q.dtype), causal, q.shape[-1] ** -0.5,
                           torch.cuda.current_stream(dev).cuda_stream, dev, status.data_ptr())
    assert rc == _lib.OK, _lib.strerror(rc)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return dq, dk, dv


def test_no_alloc_backward_matches_workspace_backward_twice_in_a_row():
    assert _lib.no_alloc_scratch_bytes() == 8 << 20
    cases = [
        _case(1, 2, 8, 2, 640, 128, torch.bfloat16, True),   # GQA, partial last tile
        _case(2, 3, 4, 4, 384, 64, torch.float16, False),    # different shape: stale scratch contents differ
    ]
    for q, k, v, dout, out, lse, causal in [c + (i == 0,) for i, c in enumerate(cases)]:
        ref_dq, ref_dk, ref_dv = raw.flash_bwd(dout, q, k, v, out, lse, causal=causal)
        before = _lib.launch_count()
        dq, dk, dv = _no_alloc_backward(q, k, v, dout, out, lse, causal)
        assert _lib.launch_count() - before == 3
        assert torch.equal(dk, ref_dk) and torch.equal(dv, ref_dv) and torch.equal(dq, ref_dq)
        assert_within("dq", dq, ref_dq.float(), TOL_16BIT, q.dtype)


def test_no_alloc_backward_serves_fp32_tensors_too():
    """fp32 tensors go to the exact-fp32 kernels, which read the same two scratch arrays from the
    built-in array (right after the 16-bit calls above have left their contents in it)."""
    q, k, v, dout, out, lse = _case(3, 1, 4, 2, 200, 64, torch.float32, True)
    ref_dq, ref_dk, ref_dv = raw.flash_bwd(dout, q, k, v, out, lse, causal=True)
    before = _lib.launch_count()
    dq, dk, dv = _no_alloc_backward(q, k, v, dout, out, lse, True)
    assert _lib.launch_count() - before == 3
    assert torch.equal(dq, ref_dq) and torch.equal(dk, ref_dk) and torch.equal(dv, ref_dv)


def test_no_alloc_backward_refuses_problems_beyond_its_scratch():
    # 16 x 32 x 4096 rows need 16 MiB of scratch (> 8 MiB); never launched, so dummy pointers suffice
    big = _lib.Tensor4.make(0x7F0000000000, (16, 32, 4096, 128), (32 * 4096 * 128, 4096 * 128, 128, 1))
    before = _lib.launch_count()
    rc = _lib.bwd_no_alloc(big, big, big, big, big, 0x7F0000000000, big, big, big, _lib.BF16, True, 0.1, 0, 0)
    assert rc == _lib.ERR_WORKSPACE
    assert b"built-in scratch" in _lib.load().b200fa_last_error_detail()
    assert _lib.launch_count() == before
