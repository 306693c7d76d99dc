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

    # ``early`` (everywhere below): whether the product's kernel may start under the tail of the kernel
    # ahead of it.  A part passes False for a product that directly follows a kernel of its own with
    # which that overlap measured slower (the attention kernel of a decode step).
    def __call__(self, ctx, x: torch.Tensor, out_name: str, out_dtype=None, early: bool = True) -> torch.Tensor:
        out_dtype = out_dtype or x.dtype
        out = ctx.workspace.get(out_name, x.shape[0], self.out_features, out_dtype)
        self.into(ctx, x, out, early=early)
        return out

    def into(self, ctx, x: torch.Tensor, out: torch.Tensor, early: bool = True) -> None:
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
        ops.gemm(x, w, out, early=early)

    # ---- fused with the norms around it (decode steps of a few tokens) -------------------------
    def can_fuse(self, ctx, T: int) -> bool:
        return ops.can_fuse_norms(T, ctx.dtype, self.weight)

    def from_normed(self, ctx, nx, out: torch.Tensor, swiglu8: bool = False) -> None:
        """out = norm(x) . W^T for a lazily normalised input (see parts.base.NormedInput)."""
        if nx.ss_parts is None:
            ops.gemm(nx.xw, self.weight, out, swiglu8=swiglu8)
        elif ops.fuses_in_skinny(nx.xw.shape[0], self.weight):
            ops.gemm_tn_skinny_fused(nx.xw, self.weight, out, swiglu8=swiglu8, scale_parts=nx.ss_parts,
                                     norm_width=nx.width, eps=nx.eps)
        else:
            ops.gemm_tn_tcgen05_fused(nx.xw, self.weight, out, swiglu8=swiglu8, scale_parts=nx.ss_parts,
                                      norm_width=nx.width, eps=nx.eps)

    def into_residual(self, ctx, x: torch.Tensor, residual: torch.Tensor, next_norm, slot: str, early: bool = True):
        """residual += x . W^T in the product's epilogue.  With ``next_norm`` (an RMSNorm part) the same
        epilogue prepares the input of the part behind that norm and returns it as a NormedInput.  Both
        kernels that carry these fusions lay the partial sums of squares out as [parts, tokens]: 16
        weight rows a part and 8 tokens wide (weight-streaming), or 128 rows a part (tensor cores); the
        product that consumes them runs the same kernel, since both see the same number of tokens."""
        from .base import NormedInput
        T, N = x.shape[0], self.out_features
        skinny = ops.fuses_in_skinny(T, self.weight)
        if next_norm is None:
            if skinny:
                ops.gemm_tn_skinny_fused(x, self.weight, residual=residual, early=early)
            else:
                ops.gemm_tn_tcgen05_fused(x, self.weight, residual=residual)
            return None
        xw = ctx.workspace.get("fused.xw." + slot, T, N, ctx.dtype)
        if skinny:
            ss = ctx.workspace.get("fused.ss." + slot, (N + 15) // 16, 8, torch.float32, reserve=0)
            ops.gemm_tn_skinny_fused(x, self.weight, residual=residual, next_w=next_norm.weight, xw_out=xw,
                                     ss_out=ss, early=early)
        else:
            ss = ctx.workspace.get("fused.ss128." + slot, (N + 127) // 128, ops.FUSED_TOKENS, torch.float32, reserve=0)
            ops.gemm_tn_tcgen05_fused(x, self.weight, residual=residual, next_w=next_norm.weight, xw_out=xw,
                                      ss_out=ss)
        return NormedInput(xw, ss, next_norm.spec.size, next_norm.spec.eps)
