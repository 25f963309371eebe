"""``AutogradPrivateUse1`` router for ``aten::scaled_dot_product_attention``.

Same design as the reference (torch_mojo_backend/mojo_device/mojo_device_autograd.py:565-643):
eligible calls are re-dispatched to ``aten::_scaled_dot_product_flash_attention`` so PyTorch's
generated autograd node (``ScaledDotProductFlashAttentionBackward0``) owns the saved tensors,
the version checks and the backward call.  Unlike the reference there is no math
decomposition behind it: an ineligible call raises ``NotImplementedError`` from the forward.
"""

from __future__ import annotations

import torch

from . import flash_ops

_registered = False


def scaled_dot_product_attention_autograd(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, *,
                                          scale=None, enable_gqa=False):
    if flash_ops.flash_inputs(query, key, value, attn_mask, dropout_p, is_causal, scale, enable_gqa) is None:
        raise NotImplementedError(
            "scaled_dot_product_attention on the mojo device serves only the flash path: fp32/bf16/fp16 "
            "(B,H,S,D) tensors, head_dim 64 or 128, no attn_mask, 0 <= dropout_p < 1, positive scale, "
            "and enable_gqa=True when the key/value head count differs (no fallback exists)"
        )
    return torch.ops.aten._scaled_dot_product_flash_attention.default(
        query, key, value, dropout_p, is_causal, False, scale=scale
    )[0]


def register_autograd_ops() -> None:
    global _registered
    if _registered:
        return
    torch.library.impl("aten::scaled_dot_product_attention", "AutogradPrivateUse1")(
        scaled_dot_product_attention_autograd
    )
    _registered = True
