"""Attention over HOST tensors with the transfers overlapped with the kernels.

A forward (and backward) pass whose inputs and results live in page-locked host memory spends
most of its time on PCIe: one call over the whole batch uploads everything, computes, then
downloads everything.  ``HostAttentionPipeline`` cuts the batch into pieces of whole
(batch entry, kv-head group) units — attention problems that do not interact — and walks them
through the two flash operators the `mojo` device registers
(``aten::_scaled_dot_product_flash_attention`` and its ``_backward``) with uploads, kernels and
downloads on three CUDA streams, so both PCIe directions and the GPU work at the same time.
Results are bitwise those of a single call over the whole batch: the pieces go through the
same kernels, and nothing is summed across pieces.

The reference has no counterpart (its benchmarks time device-resident tensors,
benchmarks/test_attention.py:36-47); this is the host-buffer entry point of this package.
"""

from __future__ import annotations

import torch


class PendingPass:
    """One enqueued pass of a ``HostAttentionPipeline``: its pinned host result tensors and the
    event behind its last download.  ``wait()`` blocks the host until the results are complete
    and gives the pass's device tensors back to the allocator."""

    def __init__(self, out, grads, done, keep):
        self.out = out
        self.grads = grads
        self._done = done
        self._keep = keep

    def wait(self):
        if self._done is not None:
            self._done.synchronize()
            self._done = None
            self._keep.clear()
        return self.out, self.grads


class HostAttentionPipeline:
    """``run`` computes ``out`` (and ``dq, dk, dv`` when ``dout`` is given) for pinned host
    tensors shaped (B, Hq, S, D) / (B, Hkv, S, D), writing into pinned host result tensors.

    ``enqueue`` is the same pass without a place where the host has to wait: it returns a
    ``PendingPass``.  Passes enqueued one after the other overlap - the uploads of the next one
    run under the downloads of the one before - so a loop that keeps two passes in flight
    (enqueue pass i + 1, then ``wait()`` for pass i and consume its results; two sets of result
    buffers) never leaves a PCIe direction idle while a pass fills or drains."""

    def __init__(self, device_index: int = 0, piece_bytes: int = 40 << 20):
        import torch_mojo_backend_b200 as tmb

        tmb.register_mojo_devices()
        self._tmb = tmb
        self.index = int(device_index)
        self.device = torch.device("mojo", self.index)
        self.piece_bytes = int(piece_bytes)   # upload size of one piece; smaller ones cost more in dispatch than the overlap wins
        self._streams = tuple(torch.cuda.Stream(device=self.index) for _ in range(3))
        self._pending: list[PendingPass] = []

    # ------------------------------------------------------------------ planning
    def pieces(self, q: torch.Tensor, k: torch.Tensor, with_backward: bool):
        """[(batch slice, query-head slice, kv-head slice)]: ranges of batch entries, or - when a
        single batch entry is larger than a piece - its kv heads in two groups (a GQA group is
        never cut)."""
        B, Hq = q.shape[0], q.shape[1]
        Hkv = k.shape[1]
        per_entry = (q[0].numel() * (2 if with_backward else 1) + 2 * k[0].numel()) * q.element_size()
        wanted = max(1, min(2 * B, (per_entry * B) // self.piece_bytes))
        if wanted <= B:
            bounds = [round(n * B / wanted) for n in range(wanted + 1)]
            return [(slice(a, b), slice(None), slice(None)) for a, b in zip(bounds, bounds[1:]) if b > a]
        split = 2 if Hkv % 2 == 0 else 1
        rep = Hq // Hkv
        return [(slice(i, i + 1), slice(g * Hkv // split * rep, (g + 1) * Hkv // split * rep),
                 slice(g * Hkv // split, (g + 1) * Hkv // split))
                for i in range(B) for g in range(split)]

    # ------------------------------------------------------------------ one pass
    def enqueue(self, q, k, v, dout=None, *, is_causal: bool, scale: float | None = None, out=None,
                grads=None) -> PendingPass:
        """Enqueue one pass and return at once.  ``out`` / ``grads``: pinned host result tensors to
        fill (e.g. from ``torch_mojo_backend_b200.pinned_empty``; allocated when omitted); a buffer
        must not be handed to a new pass before the pass that last wrote it has been waited for.
        The inputs are host tensors: nothing on the current stream is waited for, except by the
        first pass after a ``synchronize()``."""
        tmb = self._tmb
        backward = dout is not None
        if out is None:
            out = tmb.pinned_empty(q.shape, q.dtype)
        if backward and grads is None:
            grads = tuple(tmb.pinned_empty(t.shape, t.dtype) for t in (q, k, v))
        flash_fwd = torch.ops.aten._scaled_dot_product_flash_attention
        flash_bwd = torch.ops.aten._scaled_dot_product_flash_attention_backward
        s_in, s_run, s_out = self._streams
        self._pending = [p for p in self._pending if p._done is not None]
        if not self._pending:
            main = torch.cuda.current_stream(self.index)
            for s in self._streams:
                s.wait_stream(main)
        keep: list = []
        for bs, qs, ks in self.pieces(q, k, backward):
            with torch.cuda.stream(s_in):
                dev_in = [q[bs, qs].to(self.device, non_blocking=True), k[bs, ks].to(self.device, non_blocking=True),
                          v[bs, ks].to(self.device, non_blocking=True)]
                if backward:
                    dev_in.append(dout[bs, qs].to(self.device, non_blocking=True))
                uploaded = torch.cuda.Event()
                uploaded.record(s_in)
            with torch.cuda.stream(s_run):
                s_run.wait_event(uploaded)
                fwd = flash_fwd(dev_in[0], dev_in[1], dev_in[2], 0.0, is_causal, False, scale=scale)
                o, lse = fwd[0], fwd[1]
                g = ()
                if backward:
                    g = flash_bwd(dev_in[3], dev_in[0], dev_in[1], dev_in[2], o, lse, None, None, fwd[4], fwd[5], 0.0,
                                  is_causal, fwd[6], fwd[7], scale=scale)
                computed = torch.cuda.Event()
                computed.record(s_run)
            with torch.cuda.stream(s_out):
                s_out.wait_event(computed)
                out[bs, qs].copy_(o, non_blocking=True)
                for dst, grad, hs in zip(grads or (), g, (qs, ks, ks)):
                    dst[bs, hs].copy_(grad, non_blocking=True)
            # the three streams use one another's allocations: nothing goes back to the allocator
            # before the pass has been waited for
            keep.extend(dev_in)
            keep.extend((o, lse) + tuple(g))
        done = torch.cuda.Event()
        done.record(s_out)   # the download stream runs in order: behind this pass's last copy
        pending = PendingPass(out, grads if backward else None, done, keep)
        self._pending.append(pending)
        return pending

    def run(self, q, k, v, dout=None, *, is_causal: bool, scale: float | None = None, out=None, grads=None):
        """Enqueue one pass; returns ``(out, (dq, dk, dv) or None)`` — pinned host tensors that are
        complete once ``synchronize()`` has returned."""
        pending = self.enqueue(q, k, v, dout, is_causal=is_causal, scale=scale, out=out, grads=grads)
        return pending.out, pending.grads

    def synchronize(self) -> None:
        """Wait for every enqueued pass (their device tensors are released), order the current
        stream behind the pipeline's streams and raise if a kernel reported a timed-out wait."""
        main = torch.cuda.current_stream(self.index)
        for s in self._streams:
            main.wait_stream(s)
        for p in self._pending:
            p.wait()
        self._pending.clear()
        main.synchronize()
        # a kernel that gave up on an internal wait has left its results undefined: say so here
        from . import flash_ops

        flash_ops.check_status(self.index)
