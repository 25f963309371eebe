"""The operator API on the `mojo` device, end to end on a GPU (``-m gpu``): the reference's
public contract from tests/test_eager_kernels.py:9437-9585 and :10044-10071."""

import pytest
import torch

from oracle import sdpa_oracle as O
from tests.helpers import TOL_16BIT, TOL_LSE, assert_within, load_golden
from torch_mojo_backend_b200 import flash_ops

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mojo(mojo_registered):
    return torch.device("mojo", 0)


@pytest.mark.parametrize("name", ["fused_bf16_d64", "fused_f16_d128", "fused_bf16_d128_b2"])
def test_nanogpt_layout_forward_backward(mojo, name):
    """Fused-QKV gapped views, SDPA with grad, sequence-major output, native flash backward."""
    meta, _, _, _, dout, exp = load_golden(name)
    b, h, s, d = meta["B"], meta["Hq"], meta["S"], meta["D"]
    fused = meta["fused"].to(mojo)
    q, k, v = (p.view(b, s, h, d).transpose(1, 2) for p in fused.split(h * d, dim=2))
    for t in (q, k, v):
        t.requires_grad_()
        assert h == 1 or not t._is_contiguous
    before = dict(flash_ops.CALL_COUNTERS)
    out = torch.nn.functional.scaled_dot_product_attention(q, k, v, dropout_p=0.0, is_causal=True)
    assert type(out.grad_fn).__name__ == "ScaledDotProductFlashAttentionBackward0"
    assert out.dtype == meta["dtype"]
    assert (h == 1 or not out._is_contiguous) and out.transpose(1, 2)._is_contiguous
    out.backward(dout.to(mojo))
    after = flash_ops.CALL_COUNTERS
    assert after["aten::_scaled_dot_product_flash_attention"] == before["aten::_scaled_dot_product_flash_attention"] + 1
    assert (after["aten::_scaled_dot_product_flash_attention_backward"]
            == before["aten::_scaled_dot_product_flash_attention_backward"] + 1)
    assert_within("out", out.cpu(), exp["out"], TOL_16BIT, meta["dtype"])
    for t, key in ((q, "dq"), (k, "dk"), (v, "dv")):
        assert t.grad is not None
        assert_within(key, t.grad.cpu(), exp[key], TOL_16BIT, meta["dtype"])
    # the caller's re-assembly is a free view of the sequence-major output
    y = out.transpose(1, 2).contiguous().view(b, s, h * d)
    assert y._ptr == out._ptr


def test_direct_flash_op_returns_a_real_logsumexp(mojo):
    meta, q, k, v, _, exp = load_golden("gqa_bf16_s256")
    res = torch.ops.aten._scaled_dot_product_flash_attention.default(
        q.to(mojo), k.to(mojo), v.to(mojo), 0.0, True, False, scale=meta["scale"])
    assert len(res) == 9 and res[2] is None and res[3] is None and res[4] == meta["S"]
    assert_within("out", res[0].cpu(), exp["out"], TOL_16BIT, meta["dtype"])
    assert_within("lse", res[1].cpu(), exp["lse"], TOL_LSE)


def test_cross_attention_through_sdpa_with_grad(mojo):
    """A short query over a longer key sequence, no mask, GQA, through the SDPA router and the
    generated autograd node: gradients come back at the key length and head count."""
    g = torch.Generator().manual_seed(13)
    q = (torch.randn(2, 8, 200, 128, generator=g) * 0.5).bfloat16()
    k = (torch.randn(2, 2, 777, 128, generator=g) * 0.5).bfloat16()
    v = (torch.randn(2, 2, 777, 128, generator=g) * 0.5).bfloat16()
    dout = torch.randn(2, 8, 200, 128, generator=g).bfloat16()
    ref_out, rdq, rdk, rdv = O.sdpa_backward(q, k, v, dout, False, 128 ** -0.5)
    qm, km, vm = (t.to(mojo).requires_grad_() for t in (q, k, v))
    out = torch.nn.functional.scaled_dot_product_attention(qm, km, vm, enable_gqa=True)
    out.backward(dout.to(mojo))
    assert_within("out", out.detach().cpu(), ref_out, TOL_16BIT, torch.bfloat16)
    assert tuple(km.grad.shape) == (2, 2, 777, 128)
    for name, got, ref in (("dq", qm.grad, rdq), ("dk", km.grad, rdk), ("dv", vm.grad, rdv)):
        assert_within(name, got.cpu(), ref, TOL_16BIT, torch.bfloat16)
    # is_causal over unequal lengths keeps torch's meaning: the diagonal starts at the top-left corner
    ref_causal, _ = O.sdpa_forward(q, k, v, True, 128 ** -0.5)
    out_causal = torch.nn.functional.scaled_dot_product_attention(qm, km, vm, is_causal=True, enable_gqa=True)
    assert_within("causal out", out_causal.detach().cpu(), ref_causal, TOL_16BIT, torch.bfloat16)


def test_decode_shaped_sdpa_takes_the_split_kv_kernel_and_its_backward_matches(mojo):
    """Two new tokens per sequence against a 3000-token cache, GQA: the forward is served by the
    split-KV call, and the generated autograd node runs the ordinary backward kernels on its
    out / logsumexp."""
    g = torch.Generator().manual_seed(17)
    q = (torch.randn(2, 8, 2, 128, generator=g) * 0.5).bfloat16()
    k = (torch.randn(2, 2, 3000, 128, generator=g) * 0.5).bfloat16()
    v = (torch.randn(2, 2, 3000, 128, generator=g) * 0.5).bfloat16()
    dout = torch.randn(2, 8, 2, 128, generator=g).bfloat16()
    ref_out, rdq, rdk, rdv = O.sdpa_backward(q, k, v, dout, False, 128 ** -0.5)
    qm, km, vm = (t.to(mojo).requires_grad_() for t in (q, k, v))
    before = flash_ops.CALL_COUNTERS["forward_split_kv"]
    out = torch.nn.functional.scaled_dot_product_attention(qm, km, vm, enable_gqa=True)
    assert flash_ops.CALL_COUNTERS["forward_split_kv"] == before + 1
    out.backward(dout.to(mojo))
    assert_within("out", out.detach().cpu(), ref_out, TOL_16BIT, torch.bfloat16)
    for name, got, ref in (("dq", qm.grad, rdq), ("dk", km.grad, rdk), ("dv", vm.grad, rdv)):
        assert_within(name, got.cpu(), ref, TOL_16BIT, torch.bfloat16)


def test_autocast_block_runs_the_bf16_kernel(mojo):
    g = torch.Generator().manual_seed(11)
    q, k, v = (torch.randn(2, 4, 256, 64, generator=g) * 0.5 for _ in range(3))
    ref, _ = O.sdpa_forward(q.bfloat16(), k.bfloat16(), v.bfloat16(), True, 0.125)
    with torch.autocast("mojo", dtype=torch.bfloat16):
        out = torch.nn.functional.scaled_dot_product_attention(q.to(mojo), k.to(mojo), v.to(mojo), is_causal=True)
    assert out.dtype == torch.bfloat16
    assert_within("out", out.cpu(), ref, TOL_16BIT, torch.bfloat16)


def test_in_place_mutation_of_saved_tensors_raises(mojo):
    """Generated autograd owns the saves, so its version-counter check fires
    (reference: tests/test_eager_kernels.py:10044-10071)."""
    q = (torch.randn(1, 2, 128, 64) * 0.5).bfloat16().to(mojo).requires_grad_()
    k = (torch.randn(1, 2, 128, 64) * 0.5).bfloat16().to(mojo)
    v = (torch.randn(1, 2, 128, 64) * 0.5).bfloat16().to(mojo)
    out = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
    k.add_(k)
    with pytest.raises(RuntimeError, match="modified by an inplace operation"):
        out.backward(torch.ones(1, 2, 128, 64).bfloat16().to(mojo))


def test_zero_copy_interop_with_cuda_tensors(mojo_registered):
    x = torch.arange(24, dtype=torch.float32, device="cuda").view(2, 3, 4)
    m = mojo_registered.from_cuda(x)
    assert m._ptr == x.data_ptr() and torch.equal(m.cpu(), x.cpu())
    back = torch.from_dlpack(m)
    assert back.data_ptr() == x.data_ptr()
    assert mojo_registered.to_cuda(m.transpose(0, 1)).data_ptr() == x.data_ptr()


def test_host_attention_pipeline_is_bitwise_the_single_call(mojo_registered):
    """The package's host-tensor entry point: the batch in pieces over three streams gives the
    bits of one F.scaled_dot_product_attention + backward over the whole batch."""
    import torch_mojo_backend_b200 as tmb

    B, Hq, Hkv, S, D = 6, 8, 2, 512, 128
    g = torch.Generator().manual_seed(21)
    host = [tmb.pinned_empty(shape, torch.bfloat16) for shape in
            ((B, Hq, S, D), (B, Hkv, S, D), (B, Hkv, S, D), (B, Hq, S, D))]
    for t in host:
        t.copy_((torch.randn(t.shape, generator=g) * 0.5).to(torch.bfloat16))
    hq, hk, hv, hdo = host
    mq, mk, mv = (t.to("mojo").requires_grad_() for t in (hq, hk, hv))
    out = torch.nn.functional.scaled_dot_product_attention(mq, mk, mv, is_causal=True, enable_gqa=True)
    out.backward(hdo.to("mojo"))
    torch.mojo.synchronize()
    pipe = tmb.HostAttentionPipeline(0, piece_bytes=4 << 20)   # small pieces: several per pass
    assert len(pipe.pieces(hq, hk, True)) > 1
    for _ in range(2):   # twice: result buffers and streams are reused
        res_out, grads = pipe.run(hq, hk, hv, hdo, is_causal=True)
        pipe.synchronize()
        assert torch.equal(res_out, out.detach().cpu())
        assert torch.equal(grads[0], mq.grad.cpu()) and torch.equal(grads[1], mk.grad.cpu())
        assert torch.equal(grads[2], mv.grad.cpu())
    # two passes in flight with different inputs and their own result buffers: the second is enqueued
    # before the first is waited for, and each lands exactly what a pass on its own lands
    hq2 = tmb.pinned_empty(hq.shape, hq.dtype)
    hq2.copy_(hq.flip(2))
    first = pipe.enqueue(hq, hk, hv, hdo, is_causal=True)
    second = pipe.enqueue(hq2, hk, hv, hdo, is_causal=True)
    out1, grads1 = first.wait()
    assert torch.equal(out1, out.detach().cpu()) and torch.equal(grads1[0], mq.grad.cpu())
    out2, grads2 = second.wait()
    alone_out, alone_grads = pipe.run(hq2, hk, hv, hdo, is_causal=True)
    pipe.synchronize()
    assert torch.equal(out2, alone_out) and all(torch.equal(a, b) for a, b in zip(grads2, alone_grads))
    assert not torch.equal(out2, out1)
    # forward only, one batch entry larger than a piece: its kv-head groups are the pieces
    pipe2 = tmb.HostAttentionPipeline(0, piece_bytes=1 << 20)
    assert len(pipe2.pieces(hq, hk, False)) == 2 * B
    res_out, grads = pipe2.run(hq, hk, hv, None, is_causal=True)
    pipe2.synchronize()
    assert grads is None and torch.equal(res_out, out.detach().cpu())
