"""y = x W^T (+ b), weight [out, in] as the checkpoint stores it
(ullm/layers/linear.py:165).  The product itself is the vendor library's
matrix product, as in the reference; in float32 it runs without any
reduced-precision mode."""

from __future__ import annotations

from ..csrc import kernels


def linear(x, weight, out, bias=None):
    return kernels().linear(x, weight, out, bias)


def batched_matmul(x, w, out):
    """out[b] = x[b] @ w[b] for b in a batch of small independent products (one per head, say): x [B, T, k],
    w [B, k, n], out [B, T, n], each with unit stride in one of its last two dimensions (views of wider rows are
    fine).  The vendor library's strided batched product; in float32 without any reduced-precision mode."""
    import torch

    if not x.is_cuda:
        raise RuntimeError("batched_matmul runs on CUDA tensors only (no CPU path)")
    torch.bmm(x, w, out=out)
    return out
