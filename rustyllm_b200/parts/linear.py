"""out = a @ W^T (+ bias): the one place that picks a matrix-product kernel.

Every weight is ``[out x in]`` with ``in`` contiguous and is used as ``y = W x``
(SimonWaldherr/RustyLLM src/model.rs:185-186), so both operands are K-major.
float32 weights run on the CUDA cores with float32 accumulation (the true 32-bit
path).  bfloat16 weights run on the tensor cores where the tensor-core kernel takes
the shape, else on the CUDA cores with float32 accumulation.
"""
from __future__ import annotations

from typing import Optional, Union

import torch

from .. import kernels as K
from .base import NormedInput, NormRequest

OUT_SAME, OUT_F32, OUT_ADD_F32 = K.OUT_SAME, K.OUT_F32, K.OUT_ADD_F32


FOLD_NORMS_UP_TO = 64      # tokens: above, a norm costs less than what folding it adds to the products


def can_fold_norms(weight: torch.Tensor, compute_dtype: torch.dtype, num_tokens: int) -> bool:
    """Whether a product of ``num_tokens`` rows with this weight runs on the kernel that
    can fold an RMSNorm into its epilogue (bf16 on the tensor cores, K a multiple of 8, a
    step of at most 64 tokens: there a kernel launch costs as much as the norm itself)."""
    return (num_tokens <= FOLD_NORMS_UP_TO and compute_dtype == torch.bfloat16 and weight is not None
            and weight.dtype == torch.bfloat16 and weight.is_contiguous() and weight.shape[1] % 8 == 0
            and weight.data_ptr() % 16 == 0)


def linear(a: Union[torch.Tensor, NormedInput], weight: torch.Tensor, out: torch.Tensor, out_mode: int,
           bias: Optional[torch.Tensor] = None, then_norm: Optional[NormRequest] = None) -> Optional[NormedInput]:
    """``a``: [M, K]; ``weight``: [N, K]; ``out``: [M, N].

    out_mode OUT_SAME stores in a's dtype, OUT_F32 stores float32, OUT_ADD_F32 adds
    into a float32 buffer (the residual sum, kept in 32-bit).

    ``a`` may be a ``NormedInput`` (a norm that this product finishes; a part accepts one
    only where ``can_fold_norms`` holds for the weight that meets it).  ``then_norm`` (with
    OUT_ADD_F32): also prepare that norm of the updated ``out`` for the next product;
    returns the ``NormedInput``, or ``None`` if this product runs on a kernel that cannot
    (the caller then runs the norm itself).
    """
    if isinstance(a, NormedInput) or (then_norm is not None and out_mode == OUT_ADD_F32):
        x = a.weighted if isinstance(a, NormedInput) else a
        if (x.shape[0] <= FOLD_NORMS_UP_TO and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
                and K.gemm_tc_supported(x, weight, out)):
            kw = {}
            if isinstance(a, NormedInput):
                kw.update(row_sumsq=a.sumsq, row_eps=a.eps)
            made = None
            if then_norm is not None and out_mode == OUT_ADD_F32:
                M, N = out.shape
                made = NormedInput(torch.empty((M, N), dtype=torch.bfloat16, device=out.device),
                                   torch.empty((M, K.norm_pieces(N)), dtype=torch.float32, device=out.device),
                                   then_norm.eps)
                kw.update(norm_weight=then_norm.weight, norm_out=made.weighted, norm_sumsq=made.sumsq)
            K.gemm_tc(x, weight, out, out_mode, bias, **kw)
            return made
        if isinstance(a, NormedInput):
            raise K.KernelError("a product that was to finish a norm cannot run on the tensor-core kernel "
                                f"(input {tuple(x.shape)} {x.dtype}, weight {tuple(weight.shape)} {weight.dtype})")
        # then_norm on a kernel that cannot prepare it: plain product, the caller runs the norm
    if weight.dtype != a.dtype:
        # A weight the checkpoint stores in 32-bit stays 32-bit even in a bf16 run:
        # widen the activations for this product and narrow the result if asked.
        a32 = torch.empty(a.shape, dtype=torch.float32, device=a.device)
        K.convert(a.contiguous(), a32)
        if out_mode == OUT_SAME:
            tmp = torch.empty(out.shape, dtype=torch.float32, device=a.device)
            K.gemm_simt(a32, weight, tmp, OUT_F32, bias)
            K.convert(tmp, out)
        else:
            K.gemm_simt(a32, weight, out, out_mode, bias)
        return
    if a.dtype == torch.bfloat16 and K.gemm_tc_supported(a, weight, out):
        K.gemm_tc(a, weight, out, out_mode, bias)
    else:
        K.gemm_simt(a, weight, out, out_mode, bias)
