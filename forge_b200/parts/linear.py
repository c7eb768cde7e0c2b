"""y = x . W^T (+ b): the matrix product every projection is made of, with its epilogue fused.

Not a registered part but the piece parts are built from.  In 32-bit runs it is the fp32 FMA kernel; in
bfloat16 runs it is the tcgen05/TMA tensor-core kernel with fp32 accumulation, and shapes that kernel
refuses (a reduction dimension that is not a multiple of 8) go to the FMA kernel on bfloat16 operands.
Results are fp32, or the activation type where the epilogue says so.
"""
import torch

from .. import kernels


class Linear:
    def __init__(self, weight, bias, rt):
        """weight [N,K] in rt.dtype on the device; bias fp32 [N] or None."""
        self.weight, self.bias, self.rt = weight, bias, rt
        self.out_features, self.in_features = weight.shape
        self.tensor_core = (not rt.full_precision) and kernels.gemm_sm100_supports(self.out_features, self.in_features)

    def replay_tensors(self):
        return [self.weight, self.bias]

    def replay_key(self):
        return ("linear", tuple(self.weight.shape), self.weight.dtype, self.bias is None, self.tensor_core)

    def forward(self, x, accumulate_into=None, epilogue="none"):
        """x [M,K] in rt.dtype.
        epilogue "none":   fp32 [M,N] (added into ``accumulate_into`` if given, which is then returned)
        epilogue "swiglu": rt.dtype [M,N/2], out[:,j] = silu(y[:,2j]) * y[:,2j+1]
        epilogue "cast":   rt.dtype [M,N]
        """
        if self.tensor_core:
            return kernels.gemm_sm100(x, self.weight, bias=self.bias, accumulate_into=accumulate_into, epilogue=epilogue)
        if epilogue == "none":
            return kernels.gemm_simt(x, self.weight, bias=self.bias, out=accumulate_into,
                                     accumulate=accumulate_into is not None)
        y = kernels.gemm_simt(x, self.weight, bias=self.bias)
        if epilogue == "swiglu":
            return kernels.silu_mul_interleaved(y, self.rt.dtype)
        if epilogue == "cast":
            return y.to(self.rt.dtype)
        raise ValueError(f"unknown epilogue {epilogue!r}")
