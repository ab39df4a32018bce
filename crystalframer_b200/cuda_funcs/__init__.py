"""Drop-in autograd Functions with the names and signatures of the reference's
``models/cuda_funcs`` package (models/cuda_funcs/__init__.py:12-47), backed by libcfb200.so."""
from .kernel_manager import KernelManager, compile_kernels, current_config
from .framed_proj import RealEncodingWithFramedProjFuncCUDA
from .enc_proj import RealPeriodicEncodingWithProjFuncCUDA
from .max_frame import (ComputeFrame1MaximumMethodCUDA, ComputeFrame1MaximumStaticMethodCUDA, ComputeFrame2MaximumMethodCUDA,
                        ComputeFrame3MaximumMethodCUDA, max_frame3_with_selection,
                        ComputeFrame2MaximumStaticMethodCUDA, ComputeLatticeFrameCUDA, ComputePCAFrame, max_frame_with_selection,
                        max_frames_fused, max_static_frame_with_selection, max_static_frames_fused, weighted_pca_frames)
from .fused_dpa import FusedDotProductAttentionCUDA, FusedDotProductAttentionSigmaMatCUDA, attention_probabilities
from .irregular_mean import IrregularMeanCUDA
from .reci_enc import ReciPeriodicEncodingFuncCUDA
from .real_enc import RealPeriodicEncodingFuncCUDA
from .common import csr_offsets, register_csr

# the reference exports this flag (models/cuda_funcs/__init__.py:2-9); here it says whether the
# CUDA library can be used at all
CUPY_AVAILABLE = True

__all__ = [
    "KernelManager", "compile_kernels", "current_config", "FusedDotProductAttentionCUDA",
    "FusedDotProductAttentionSigmaMatCUDA",
    "ComputeFrame1MaximumMethodCUDA", "ComputeFrame2MaximumMethodCUDA", "ComputeFrame3MaximumMethodCUDA",
    "max_frame3_with_selection", "RealEncodingWithFramedProjFuncCUDA",
    "ComputeFrame1MaximumStaticMethodCUDA", "ComputeFrame2MaximumStaticMethodCUDA", "ComputeLatticeFrameCUDA", "ComputePCAFrame",
    "max_static_frame_with_selection", "max_static_frames_fused",
    "RealPeriodicEncodingWithProjFuncCUDA", "ReciPeriodicEncodingFuncCUDA", "RealPeriodicEncodingFuncCUDA",
    "IrregularMeanCUDA", "max_frame_with_selection", "max_frames_fused", "weighted_pca_frames", "attention_probabilities",
    "csr_offsets", "register_csr", "CUPY_AVAILABLE",
]
