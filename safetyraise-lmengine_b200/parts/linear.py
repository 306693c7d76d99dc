"""y = x . W^T for a weight kept as [out, in] rows (no bias: src/model/native.rs:119-153).

The kernel is chosen by the weight's dtype: a float32 weight runs the float32
FMA kernel (activations are widened for it if they are bfloat16); a bfloat16
weight runs the tensor-core kernel when it takes the sizes, else the FMA kernel.
"""
from __future__ import annotations

import torch

from ..kernels import ops


class Linear:
    def __init__(self, weight: torch.Tensor, name: str = ""):
        self.weight, self.name = weight, name
        self.out_features, self.in_features = weight.shape

    def __call__(self, ctx, x: torch.Tensor, out_name: str, out_dtype=None) -> torch.Tensor:
        out_dtype = out_dtype or x.dtype
        out = ctx.workspace.get(out_name, x.shape[0], self.out_features, out_dtype)
        self.into(ctx, x, out)
        return out

    def into(self, ctx, x: torch.Tensor, out: torch.Tensor) -> None:
        w = self.weight
        if w.dtype == torch.float32 and x.dtype != torch.float32:
            x32 = ctx.workspace.get("linear.x32", x.shape[0], x.shape[1], torch.float32)
            ops.cast(x, x32)
            if out.dtype == torch.float32:
                ops.gemm_tn_simt(x32, w, out)
            else:
                y32 = ctx.workspace.get("linear.y32", out.shape[0], out.shape[1], torch.float32)
                ops.gemm_tn_simt(x32, w, y32)
                ops.cast(y32, out)
            return
        ops.gemm(x, w, out)
