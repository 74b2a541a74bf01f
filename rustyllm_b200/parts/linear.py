"""out = a @ W^T (+ bias): the one place that picks a matrix-product kernel.

Every weight is ``[out x in]`` with ``in`` contiguous and is used as ``y = W x``
(SimonWaldherr/RustyLLM src/model.rs:185-186), so both operands are K-major.
float32 weights run on the CUDA cores with float32 accumulation (the true 32-bit
path).  bfloat16 weights run on the tensor cores where the tensor-core kernel takes
the shape, else on the CUDA cores with float32 accumulation.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K

OUT_SAME, OUT_F32, OUT_ADD_F32 = K.OUT_SAME, K.OUT_F32, K.OUT_ADD_F32


def linear(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, out_mode: int,
           bias: Optional[torch.Tensor] = None) -> None:
    """``a``: [M, K]; ``weight``: [N, K]; ``out``: [M, N].

    out_mode OUT_SAME stores in a's dtype, OUT_F32 stores float32, OUT_ADD_F32 adds
    into a float32 buffer (the residual sum, kept in 32-bit).
    """
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
