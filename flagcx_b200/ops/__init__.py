"""Autograd wrappers over the fused sm_100a kernels of ``_flagcx_torch``.

Every function here requires the native extension on a CUDA device and fails
loudly when it is missing: there is no eager fallback."""
from .fused import (add_layernorm, bias_gelu, cross_entropy, enable_direct_grad, fused_adamw_step, gemm, gemm_error, linear, linear_bias_gelu)  # noqa: F401
