"""A bias-free linear projection y = x W^T with W stored [out features, in features], as
cuongvng/bare-cuda-4gib keeps every matrix (engine/include/llm/kernels.h:48-57).

It is a building brick of mixers, feed-forwards and the head rather than a family of its own.
Which kernel runs is decided here from the element types: float32 anywhere, or a size the fast
kernel refuses, goes to the plain kernel; bfloat16 activations against bfloat16 weights go to the
tensor-core kernel (see `kernels.gemm`).
"""

from __future__ import annotations

from typing import Optional

import torch

from ..kernels import lib as K


class Linear:
    def __init__(self, weight: torch.Tensor, name: str):
        self.weight = weight.contiguous()
        self.name = name
        self.out_features, self.in_features = weight.shape
        self.fast = None  # set by prepare() when the tensor-core kernel takes this matrix
        self.few = False  # whether the few-token fused kernel takes this matrix

    def prepare(self, act_dtype: torch.dtype) -> None:
        if act_dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16 and self.weight.is_cuda:
            from ..kernels import gemm
            self.fast = gemm.plan_for(self.weight)
            from ..kernels import gemv
            self.few = gemv.supports(self.weight)

    def forward(self, ctx, a, rows: int, out_dtype: torch.dtype, buffer: str,
                allow_partials: bool = False, swiglu: bool = False, epilogue=None) -> Optional[K.Partials]:
        """a[:rows] @ W^T into the workspace buffer `buffer`.  With `swiglu`, W is [gate; up] and
        the result is silu(gate) * up of half the width (fused where the kernel can).  `a` is a
        matrix or a `LazyNorm`.  `epilogue` (`AddTo`, `RotateAndCache`) names what the caller will
        do with the result next: a kernel that can do it itself does, and None comes back; from
        every other kernel the plain result comes back and the epilogue stays the caller's."""
        width = self.out_features // 2 if swiglu else self.out_features
        if self.few and ctx.use_fast_gemm:
            from ..kernels import gemv
            if gemv.takes(rows, self.in_features):
                return gemv.run(ctx, self.weight, a, rows, out_dtype, buffer, swiglu, epilogue)
        if self.fast is not None and ctx.use_fast_gemm:
            from ..kernels import gemm
            return gemm.run(ctx, self.fast, a, rows, out_dtype, buffer, allow_partials, swiglu, epilogue)
        a = K.materialize(a)
        if swiglu:
            full = ctx.ws.get(buffer + ".gate_up", (rows, self.out_features), out_dtype)
            K.matmul_plain(a, self.weight, full, rows, ctx.stream)
            out = ctx.ws.get(buffer, (rows, width), out_dtype)
            K.swiglu(K.Partials(full), out, rows, ctx.stream)
            return K.Partials(out)
        out = ctx.ws.get(buffer, (rows, width), out_dtype)
        K.matmul_plain(a, self.weight, out, rows, ctx.stream)
        return K.Partials(out)
