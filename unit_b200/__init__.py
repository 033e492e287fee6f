"""unit_b200: B200 (sm_100a) kernels behind the operator interface of were/UNIT's
tensorized paths (u8 x s8 -> s32 and fp16 -> fp32 conv2d / GEMM)."""
from .ops import (INTRINSICS, ConvPlan, PackedWeights, conv2d_NCHW16c_OHWI16o, conv2d_NCHW16c_OHWI16o_compute,
                  conv2d_NCHWc_int8, conv2d_NCHWc_int8_plan, conv3d_NCDHWc_int8, pack_conv3d_weights_int8, dense_dotprod, device_status, gemm_f16f32, launch_count,
                  pack_conv_weights_f16, pack_conv_weights_int8, pack_data_nchwc, pack_dense_weights_int8,
                  pack_gemm_weights_f16, pack_weights_oihw_f16, pack_weights_oihw_int8, unpack_data_nchwc)

__all__ = [
    'INTRINSICS', 'ConvPlan', 'PackedWeights', 'conv2d_NCHW16c_OHWI16o', 'conv2d_NCHW16c_OHWI16o_compute',
    'conv2d_NCHWc_int8', 'conv2d_NCHWc_int8_plan', 'conv3d_NCDHWc_int8', 'pack_conv3d_weights_int8',
    'dense_dotprod', 'device_status', 'gemm_f16f32', 'launch_count', 'pack_conv_weights_f16',
    'pack_conv_weights_int8', 'pack_data_nchwc', 'pack_dense_weights_int8', 'pack_gemm_weights_f16',
    'pack_weights_oihw_f16', 'pack_weights_oihw_int8', 'unpack_data_nchwc',
]
