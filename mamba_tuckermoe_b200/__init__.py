"""B200 (sm_100a) forward of the Tucker-MoE expert layer: a drop-in for the reference
``pure_torch_mlx.model.TuckerMoE`` backed by hand-written CUDA kernels behind a C ABI."""
from .tucker_moe import (PATH_AUTO, PATH_DECODE, PATH_SIMT, PATH_TENSOR, RMSNorm, TuckerMoE, TuckerMoEConfig,
                         clear_caches, fused_ffn, fused_out_proj, prepare_factors, read_device_status, rms_norm, tucker_moe_forward, tucker_moe_forward_taps)

__all__ = ["TuckerMoE", "TuckerMoEConfig", "RMSNorm", "tucker_moe_forward", "tucker_moe_forward_taps",
           "read_device_status", "clear_caches", "prepare_factors", "rms_norm", "fused_ffn", "fused_out_proj", "PATH_AUTO", "PATH_SIMT", "PATH_TENSOR", "PATH_DECODE"]
