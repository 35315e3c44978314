"""hawk_b200: B200 (sm_100a) kernels for Hawk's data-parallel hot path behind the reference's
operator interface.  See hawk_b200.ops for the operators and include/hawk_b200.h for the C ABI."""
from .ops import (Conv1D, check_device_status, decode_conv_step, decode_rglru_step, fused_cross_entropy,  # noqa: F401
                  fused_linear_scan, fused_scan_gelu, sequential_scan_backward, sequential_scan_forward,
                  temporal_conv1d)

__version__ = "0.1.0"
