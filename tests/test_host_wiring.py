"""Host-wiring contracts of the mojo-device flash ops, exercised without a GPU.

Modelled on the reference's tests/test_fa4_host_wiring.py: allocations are redirected to host
memory and the native bridge is replaced by a spy (fixture ``host_backed_mojo``), so what is
checked is the Python host code: the eligibility gate, layout routing, what is allocated and
the exact arguments that reach the C ABI."""

import math

import pytest
import torch

from torch_mojo_backend_b200 import _lib, flash_ops
from torch_mojo_backend_b200.tensor import TorchMojoTensor


def mojo(shape, dtype=torch.bfloat16):
    return torch.randn(*shape).to(dtype).to("mojo")


def fused_qkv(batch, seq, heads, dim, dtype=torch.bfloat16):
    fused = mojo((batch, seq, 3 * heads * dim), dtype)
    return fused, tuple(p.view(batch, seq, heads, dim).transpose(1, 2) for p in fused.split(heads * dim, dim=2))


def test_registration_names_the_device_mojo(host_backed_mojo):
    x = mojo((2, 3))
    assert isinstance(x, TorchMojoTensor)
    assert str(x.device) == "mojo:0"
    assert torch.mojo.current_device() == 0
    assert torch.equal(x.cpu(), x._cuda_view())


def test_ineligible_regimes_never_reach_the_bridge(host_backed_mojo):
    spy = host_backed_mojo
    q = mojo((1, 2, 128, 64))
    bad = [
        dict(attn_mask=torch.ones(128, 128, dtype=torch.bool).to("mojo")),
        dict(dropout_p=1.0),
        dict(dropout_p=-0.1),
        dict(scale=-1.0),
        dict(scale=float("inf")),
    ]
    for kwargs in bad:
        with pytest.raises(NotImplementedError):
            torch.nn.functional.scaled_dot_product_attention(q, q, q, is_causal=True, **kwargs)
    with pytest.raises(NotImplementedError):  # head_dim 96
        x = mojo((1, 2, 128, 96))
        torch.nn.functional.scaled_dot_product_attention(x, x, x, is_causal=True)
    with pytest.raises(NotImplementedError):  # GQA shapes without enable_gqa
        torch.nn.functional.scaled_dot_product_attention(mojo((1, 4, 128, 64)), q, q, is_causal=True)
    with pytest.raises(NotImplementedError):  # mixed dtypes
        torch.nn.functional.scaled_dot_product_attention(q, q, mojo((1, 2, 128, 64), torch.float16))
    with pytest.raises(NotImplementedError):  # int tensors
        xi = torch.ones(1, 2, 128, 64, dtype=torch.int32).to("mojo")
        torch.ops.aten._scaled_dot_product_flash_attention.default(xi, xi, xi, 0.0, True, False)
    assert spy.calls == []


def test_gate_is_metadata_only_and_accepts_all_dtypes(host_backed_mojo):
    for dtype in (torch.float32, torch.bfloat16, torch.float16):
        q = mojo((2, 4, 130, 128), dtype)
        k = mojo((2, 2, 130, 128), dtype)
        got = flash_ops.flash_inputs(q, k, k, None, 0.0, False, None, enable_gqa=True)
        assert got is not None and got[0] is q
    assert host_backed_mojo.calls == []


def test_cross_attention_lengths_reach_the_bridge_when_unmasked(host_backed_mojo):
    spy = host_backed_mojo
    q, k, v = mojo((1, 4, 96, 64)), mojo((1, 2, 320, 64)), mojo((1, 2, 320, 64))
    res = torch.ops.aten._scaled_dot_product_flash_attention.default(q, k, v, 0.0, False, False)
    (kind, a), = spy.calls
    assert kind == "fwd" and a["causal"] is False
    assert tuple(a["q"].shape) == (1, 4, 96, 64) and tuple(a["k"].shape) == (1, 2, 320, 64)
    assert tuple(res[0].shape) == (1, 4, 96, 64) and tuple(res[1].shape) == (1, 4, 96)
    assert (res[4], res[5]) == (96, 320)
    grads = torch.ops.aten._scaled_dot_product_flash_attention_backward.default(
        mojo((1, 4, 96, 64)), q, k, v, res[0], res[1], None, None, res[4], res[5], 0.0, False, res[6], res[7])
    kind, b = spy.calls[-1]
    assert kind == "bwd" and tuple(b["dk"].shape) == (1, 2, 320, 64) and tuple(b["dq"].shape) == (1, 4, 96, 64)
    assert [tuple(g.shape) for g in grads] == [(1, 4, 96, 64), (1, 2, 320, 64), (1, 2, 320, 64)]


def test_causal_over_unequal_lengths_keeps_torchs_top_left_rule(host_backed_mojo):
    """is_causal over Sq != Sk reaches the library as causal=True, which _lib maps to
    B200FA_CAUSAL_TOP_LEFT: the convention of torch's own SDPA, not the reference kernels'
    bottom-right one (that one is only reachable through the C ABI)."""
    spy = host_backed_mojo
    q, k = mojo((1, 2, 128, 64)), mojo((1, 2, 320, 64))
    torch.nn.functional.scaled_dot_product_attention(q, k, k, is_causal=True)
    kind, a = spy.calls[-1]
    assert kind == "fwd" and a["causal"] is True and _lib.causal_code(a["causal"]) == _lib.CAUSAL_TOP_LEFT
    assert tuple(a["k"].shape) == (1, 2, 320, 64)


def test_decode_shaped_forward_goes_to_the_split_kv_entry_point(host_backed_mojo):
    spy = host_backed_mojo
    q, k = mojo((2, 8, 1, 128)), mojo((2, 2, 4096, 128))
    before = flash_ops.CALL_COUNTERS["forward_split_kv"]
    res = torch.ops.aten._scaled_dot_product_flash_attention.default(q, k, k, 0.0, False, False)
    kind, a = spy.calls[-1]
    assert kind == "fwd_splitkv" and flash_ops.CALL_COUNTERS["forward_split_kv"] == before + 1
    assert a["workspace_bytes"] == _lib.fwd_splitkv_workspace_bytes(2, 8, 2, 1, 4096, 128) > 0
    assert tuple(res[0].shape) == (2, 8, 1, 128) and tuple(res[1].shape) == (2, 8, 1)
    # too many query rows for one split-KV thread block, or a short key sequence: the prefill kernel
    torch.ops.aten._scaled_dot_product_flash_attention.default(mojo((2, 8, 8, 128)), k, k, 0.0, False, False)
    assert spy.calls[-1][0] == "fwd"
    torch.ops.aten._scaled_dot_product_flash_attention.default(q, mojo((2, 2, 256, 128)), mojo((2, 2, 256, 128)),
                                                               0.0, False, False)
    assert spy.calls[-1][0] == "fwd"


def test_dropout_reserves_philox_state_and_the_backward_repeats_it(host_backed_mojo):
    spy = host_backed_mojo
    torch.mojo.manual_seed_all(1234)
    q = mojo((2, 4, 128, 64)).requires_grad_()
    k = mojo((2, 4, 128, 64)).requires_grad_()
    out = torch.nn.functional.scaled_dot_product_attention(q, k, k, dropout_p=0.25, is_causal=True)
    kind, a = spy.calls[-1]
    assert kind == "fwd" and a["dropout"] == (0.25, 1234, 0)
    # the generator advanced by one counter value per (batch, head)
    assert torch.mojo._reserve_philox_state(0, 0) == (1234, 8)
    out2 = torch.nn.functional.scaled_dot_product_attention(q, k, k, dropout_p=0.25, is_causal=True)
    assert spy.calls[-1][1]["dropout"] == (0.25, 1234, 8)
    out.backward(mojo((2, 4, 128, 64)))
    kind, b = spy.calls[-1]
    assert kind == "bwd" and b["dropout"] == (0.25, 1234, 0)   # the first call's pair, not the generator's current one
    # the aten tuple carries the pair: on the device (uint64[2]) and as a host-side copy
    res = torch.ops.aten._scaled_dot_product_flash_attention.default(q.detach(), k.detach(), k.detach(), 0.5, False, False)
    assert res[6]._philox == (1234, 16) and res[6].cpu().tolist() == [1234, 16]
    assert res[6].detach()._philox == (1234, 16)
    # without dropout nothing is reserved and the library gets no dropout argument
    torch.ops.aten._scaled_dot_product_flash_attention.default(q.detach(), k.detach(), k.detach(), 0.0, False, False)
    assert spy.calls[-1][1]["dropout"] is None and torch.mojo._reserve_philox_state(0, 0) == (1234, 24)


def test_every_call_passes_the_device_status_word_and_check_status_raises(host_backed_mojo):
    spy = host_backed_mojo
    q = mojo((1, 2, 128, 64))
    res = torch.ops.aten._scaled_dot_product_flash_attention.default(q, q, q, 0.0, True, False)
    assert spy.calls[-1][1]["status_ptr"] == spy.status_ptr != 0
    torch.ops.aten._scaled_dot_product_flash_attention_backward.default(
        q, q, q, q, res[0], res[1], None, None, 128, 128, 0.0, True, res[6], res[7])
    assert spy.calls[-1][1]["status_ptr"] == spy.status_ptr
    flash_ops.check_status(0)   # clean
    # what a kernel that gave up on a wait leaves behind
    flash_ops._status_words[0]._cuda_view().fill_(0x57410320)
    with pytest.raises(_lib.B200FAError) as err:
        flash_ops.check_status(0)
    assert err.value.code == _lib.ERR_TIMEOUT and "0x57410320" in str(err.value)
    flash_ops.check_status(0)   # cleared by the failed check


def test_contiguous_bhsd_goes_zero_copy_with_bhsd_output(host_backed_mojo):
    spy = host_backed_mojo
    q, k, v = mojo((2, 4, 256, 64)), mojo((2, 4, 256, 64)), mojo((2, 4, 256, 64))
    n_alloc = len(spy.allocations)
    res = torch.ops.aten._scaled_dot_product_flash_attention.default(q, k, v, 0.0, True, False, scale=0.2)
    (kind, a), = spy.calls
    assert kind == "fwd"
    assert a["q"].ptr == q._ptr and a["k"].ptr == k._ptr and a["v"].ptr == v._ptr
    assert tuple(a["q"].shape) == (2, 4, 256, 64) and tuple(a["q"].stride) == (65536, 16384, 64, 1)
    assert a["dtype"] == _lib.BF16 and a["causal"] is True and a["scale"] == pytest.approx(0.2)
    out, lse = res[0], res[1]
    assert out._is_contiguous and tuple(out.shape) == (2, 4, 256, 64) and out.dtype == torch.bfloat16
    assert a["out"].ptr == out._ptr and a["lse_ptr"] == lse._ptr
    assert lse.dtype == torch.float32 and tuple(lse.shape) == (2, 4, 256)
    # out, lse, rng_state, unused, debug mask: five allocations, no input copies
    assert len(spy.allocations) - n_alloc == 5
    assert spy.allocations[n_alloc] == 2 * 4 * 256 * 64 * 2 and spy.allocations[n_alloc + 1] == 2 * 4 * 256 * 4


def test_aten_wrapper_returns_the_cuda_shaped_nine_tuple(host_backed_mojo):
    q = mojo((1, 2, 128, 64), torch.float16)
    res = torch.ops.aten._scaled_dot_product_flash_attention.default(q, q, q, 0.0, False, False)
    assert len(res) == 9
    out, lse, cum_q, cum_k, max_q, max_k, rng_state, unused, debug = res
    assert max_q == 128 and max_k == 128
    assert rng_state.dtype == torch.uint64 and tuple(rng_state.shape) == (2,)
    assert unused.dtype == torch.uint64 and tuple(unused.shape) == ()
    assert tuple(debug.shape) == (0,) and debug.dtype == torch.float16
    assert host_backed_mojo.calls[0][1]["scale"] == pytest.approx(1 / math.sqrt(64))
    assert host_backed_mojo.calls[0][1]["dtype"] == _lib.F16
    with pytest.raises(NotImplementedError):
        torch.ops.aten._scaled_dot_product_flash_attention.default(q, q, q, 0.0, False, True)


def test_fused_qkv_views_take_the_zero_copy_strided_route(host_backed_mojo):
    spy = host_backed_mojo
    fused, (q, k, v) = fused_qkv(2, 256, 8, 64)
    assert not q._is_contiguous
    n_alloc = len(spy.allocations)
    res = torch.ops.aten._scaled_dot_product_flash_attention.default(q, k, v, 0.0, True, False)
    a = spy.calls[0][1]
    width = 8 * 64
    assert a["q"].ptr == fused._ptr and a["k"].ptr == fused._ptr + width * 2 and a["v"].ptr == fused._ptr + 2 * width * 2
    for name in ("q", "k", "v"):
        assert tuple(a[name].stride) == (256 * 3 * width, 64, 3 * width, 1)
    out = res[0]
    # the output is stored sequence-major, like stock PyTorch flash and the reference
    assert not out._is_contiguous and out.transpose(1, 2)._is_contiguous
    assert tuple(a["out"].stride) == (256 * width, 64, width, 1)
    assert len(spy.allocations) - n_alloc == 5  # still no input copies


def test_misaligned_view_falls_back_to_a_dense_copy(host_backed_mojo):
    spy = host_backed_mojo
    base = mojo((1, 2, 128, 72))
    q = base[..., 4:68]  # head_dim stride 1 but rows are 144 bytes apart and the base is offset by 8 bytes
    assert not flash_ops.kernel_ready_layout(q)
    k = mojo((1, 2, 128, 64))
    torch.ops.aten._scaled_dot_product_flash_attention.default(q, k, k, 0.0, True, False)
    a = spy.calls[0][1]
    assert a["q"].ptr != q._ptr and tuple(a["q"].stride) == (16384, 8192, 64, 1)
    assert a["k"].ptr == k._ptr


def test_layout_predicates_are_strict():
    def fake(shape, strides, ptr=1024, itemsize=2):
        t = object.__new__(TorchMojoTensor.__mro__[1]) if False else type("T", (), {})()
        t._shape, t._strides, t._ptr, t._itemsize = shape, strides, ptr, itemsize
        return t

    ok = fake((2, 4, 128, 64), (32768, 8192, 64, 1))
    assert flash_ops.kernel_ready_layout(ok) and not flash_ops.bthd_stored(ok)
    bthd = fake((2, 4, 128, 64), (32768, 64, 256, 1))
    assert flash_ops.kernel_ready_layout(bthd) and flash_ops.bthd_stored(bthd)
    assert not flash_ops.kernel_ready_layout(fake((2, 4, 128, 64), (32768, 8192, 64, 2)))
    assert not flash_ops.kernel_ready_layout(fake((2, 4, 128, 64), (32768, 8192, 68, 1)))
    assert not flash_ops.kernel_ready_layout(fake((2, 4, 128, 64), (32768, 8192, 64, 1), ptr=1032))
    assert not flash_ops.kernel_ready_layout(fake((2, 4, 128, 64), (32768, 8192, 32, 1)))
    assert not flash_ops.kernel_ready_layout(fake((2, 4, 128, 64), (0, 8192, 64, 1)))
    assert flash_ops.kernel_ready_layout(fake((1, 4, 128, 64), (0, 8192, 64, 1)))


def test_sdpa_with_grad_routes_to_generated_autograd_and_backward_args(host_backed_mojo):
    spy = host_backed_mojo
    fused, (q, k, v) = fused_qkv(2, 256, 4, 128)
    for t in (q, k, v):
        t.requires_grad_()
    out = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
    assert type(out.grad_fn).__name__ == "ScaledDotProductFlashAttentionBackward0"
    assert flash_ops.CALL_COUNTERS["aten::_scaled_dot_product_flash_attention"] >= 1
    before = flash_ops.CALL_COUNTERS["aten::_scaled_dot_product_flash_attention_backward"]
    n_alloc = len(spy.allocations)
    out.backward(mojo((2, 4, 256, 128)))
    assert flash_ops.CALL_COUNTERS["aten::_scaled_dot_product_flash_attention_backward"] == before + 1
    (kind, a) = spy.calls[-1]
    assert kind == "bwd"
    width = 4 * 128
    # q/k/v reach the backward as the same zero-copy views of the fused projection
    assert a["q"].ptr == fused._ptr and a["k"].ptr == fused._ptr + 2 * width
    assert tuple(a["q"].stride) == (256 * 3 * width, 128, 3 * width, 1)
    # out was saved in its sequence-major storage; gradients are allocated in the same layout
    assert tuple(a["out"].stride) == (256 * width, 128, width, 1)
    for name in ("dq", "dk", "dv"):
        assert tuple(a[name].shape) == (2, 4, 256, 128) and tuple(a[name].stride) == (256 * width, 128, width, 1)
    assert a["causal"] is True and a["scale"] == pytest.approx(1 / math.sqrt(128)) and a["dtype"] == _lib.BF16
    need = _lib.bwd_workspace_bytes(2, 4, 4, 256, 128, _lib.BF16)
    assert a["workspace_bytes"] == need
    grads_bytes = 2 * 4 * 256 * 128 * 2
    new = spy.allocations[n_alloc:]
    # the op itself allocates three gradients and one scratch buffer (the engine adds its own copies)
    assert new.count(need) == 1 and new.count(grads_bytes) >= 3
    assert q.grad is not None and tuple(q.grad.shape) == (2, 4, 256, 128)


def test_backward_makes_logsumexp_contiguous_and_checks_arguments(host_backed_mojo):
    spy = host_backed_mojo
    q = mojo((1, 2, 128, 64))
    out = mojo((1, 2, 128, 64))
    lse = torch.zeros(1, 128, 2).to("mojo").transpose(1, 2)  # (1,2,128) but not contiguous
    rng = torch.zeros(2, dtype=torch.uint64).to("mojo")
    off = torch.zeros((), dtype=torch.uint64).to("mojo")
    dq, dk, dv = torch.ops.aten._scaled_dot_product_flash_attention_backward.default(
        out, q, q, q, out, lse, None, None, 128, 128, 0.0, True, rng, off, scale=0.5)
    a = spy.calls[-1][1]
    assert a["lse_ptr"] != lse._ptr  # a contiguous copy was passed
    assert tuple(dq.shape) == (1, 2, 128, 64) and dq._is_contiguous
    with pytest.raises(NotImplementedError):
        torch.ops.aten._scaled_dot_product_flash_attention_backward.default(
            out, q, q, q, out, lse, None, None, 64, 128, 0.0, True, rng, off)


def test_backward_recomputes_the_forward_when_out_or_logsumexp_is_unusable(host_backed_mojo):
    """The reference recomputes the forward when the saved out / logsumexp come back without
    their payload (aten_fast.py:7805-7818) instead of raising inside the autograd engine."""
    spy = host_backed_mojo
    q = mojo((1, 2, 128, 64))
    out = mojo((1, 2, 128, 64))
    rng = torch.zeros(2, dtype=torch.uint64).to("mojo")
    off = torch.zeros((), dtype=torch.uint64).to("mojo")
    before = flash_ops.CALL_COUNTERS["backward_recomputed_forward"]
    n = len(spy.calls)
    for bad_out, bad_lse in ((out, torch.zeros(1, 2, 64).to("mojo")),          # wrong logsumexp shape
                             (out, torch.zeros(1, 2, 128)),                     # a CPU tensor: no payload
                             (torch.zeros(1, 2, 128, 64), torch.zeros(1, 2, 128).to("mojo"))):
        grads = torch.ops.aten._scaled_dot_product_flash_attention_backward.default(
            out, q, q, q, bad_out, bad_lse, None, None, 128, 128, 0.0, True, rng, off)
        assert [tuple(g.shape) for g in grads] == [(1, 2, 128, 64)] * 3
    kinds = [c[0] for c in spy.calls[n:]]
    assert kinds == ["fwd", "bwd"] * 3
    assert flash_ops.CALL_COUNTERS["backward_recomputed_forward"] == before + 3
    # the recomputed out / lse are what the backward kernel reads
    assert spy.calls[-1][1]["out"].ptr == spy.calls[-2][1]["out"].ptr
    assert spy.calls[-1][1]["lse_ptr"] == spy.calls[-2][1]["lse_ptr"]


def test_gqa_gradients_come_back_at_kv_head_count(host_backed_mojo):
    q = mojo((1, 8, 128, 64)).requires_grad_()
    k = mojo((1, 2, 128, 64)).requires_grad_()
    v = mojo((1, 2, 128, 64)).requires_grad_()
    out = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
    out.backward(mojo((1, 8, 128, 64)))
    a = host_backed_mojo.calls[-1][1]
    assert tuple(a["dk"].shape) == (1, 2, 128, 64) and tuple(a["dq"].shape) == (1, 8, 128, 64)
    assert tuple(k.grad.shape) == (1, 2, 128, 64)


def test_autocast_casts_to_the_autocast_dtype(host_backed_mojo):
    q = mojo((1, 2, 128, 64), torch.float32)
    with torch.autocast("mojo", dtype=torch.bfloat16):
        out = torch.nn.functional.scaled_dot_product_attention(q, q, q, is_causal=True)
    assert out.dtype == torch.bfloat16
    assert host_backed_mojo.calls[-1][1]["dtype"] == _lib.BF16


def test_bridge_errors_surface_as_exceptions(host_backed_mojo, monkeypatch):
    monkeypatch.setattr(_lib, "fwd", lambda *a, **k: _lib.ERR_UNSUPPORTED)
    q = mojo((1, 2, 128, 64))
    with pytest.raises(NotImplementedError):
        torch.ops.aten._scaled_dot_product_flash_attention.default(q, q, q, 0.0, True, False)
    monkeypatch.setattr(_lib, "fwd", lambda *a, **k: _lib.ERR_CUDA)
    with pytest.raises(_lib.B200FAError):
        torch.ops.aten._scaled_dot_product_flash_attention.default(q, q, q, 0.0, True, False)


def test_views_share_the_holder_and_pickle_as_cpu(host_backed_mojo):
    import pickle

    x = mojo((2, 8, 6), torch.float32)
    y = x.transpose(0, 1)[1:3]
    assert y._holder is x._holder and y._ptr == x._ptr + 6 * 4
    assert torch.equal(y.cpu(), x.cpu().transpose(0, 1)[1:3])
    z = pickle.loads(pickle.dumps(x))
    assert z.device.type == "cpu" and torch.equal(z, x.cpu())
    empty = torch.empty(0, 4).to("mojo")
    assert empty._holder.numel() >= 1 and empty.cpu().shape == (0, 4)


def test_host_code_has_no_sync_and_no_cpu_math_path():
    """The op layer must not synchronise (launches are asynchronous, reference:
    tests/test_fa4_host_wiring.py:1107-1112) and must not import the test oracle."""
    import inspect

    assert "oracle" not in inspect.getsource(flash_ops)
    for fn in (flash_ops.flash_forward, flash_ops.flash_backward, flash_ops.scaled_dot_product_flash_attention):
        src = inspect.getsource(fn)
        assert "synchronize" not in src and ".cpu()" not in src and ".item()" not in src, fn.__name__
