"""tuisko-kernels-sm100: B200-native quantized projection operators of TuiskoLLM.

The product is the CUDA library ``libtuisko_sm100.so`` behind the C ABI of
``include/tuisko_sm100.h``.  This package is the thin Python mirror of the reference's
operator interface over that ABI (device memory comes from torch tensors).
"""
from .ops import (Context, FullAttentionQkvOp, GdnInputProjectionOp, GpuError, LmHeadOp,  # noqa: F401
                  Nvfp4DownOp, Nvfp4SwiGluOp, ResidualNormOp, Fp8ProjectionOp, Fp8SwiGluOp, Fp8DownOp,
                  GdnOutputProjectionOp, GdnPrepareOp, GdnRecurrenceOp, Sampler, SamplingOptions, Materializer)

__all__ = ["Context", "GpuError", "ResidualNormOp", "FullAttentionQkvOp", "GdnInputProjectionOp",
           "LmHeadOp", "Fp8ProjectionOp", "Nvfp4SwiGluOp", "Nvfp4DownOp", "Fp8SwiGluOp", "Fp8DownOp",
           "GdnOutputProjectionOp", "GdnPrepareOp", "GdnRecurrenceOp", "Sampler", "SamplingOptions", "Materializer"]
