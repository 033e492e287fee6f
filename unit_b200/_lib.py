"""ctypes binding of the C ABI declared in ``include/unit_b200.h``.

There is no fallback: if the shared library is missing, the import of any
operator fails with the reason.
"""
from __future__ import annotations

import ctypes
import os

from . import build as _build

_LIB = None

STATUS = {
    0: 'ok', -1: 'null pointer', -2: 'unsupported shape', -3: 'pointer or pitch not 16-byte aligned',
    -4: 'unsupported channel block or tile', -5: 'device is not sm_100a', -6: 'CUDA launch failed',
    -7: 'a kernel abandoned a bounded wait', -8: 'beyond a fixed capacity',
}

# name -> (restype, argtypes); kept beside the header so a test can check that
# every declared symbol is exported.
_vp, _ci, _i64, _sz = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_size_t


class ConvDesc(ctypes.Structure):
    """Mirror of ``unit_conv_desc``."""
    _fields_ = [(n, ctypes.c_int32) for n in
                ('n', 'c_in', 'h', 'w', 'c_block', 'c_out', 'kh', 'kw', 'stride_h', 'stride_w', 'pad_h', 'pad_w')]


class Conv3dDesc(ctypes.Structure):
    """Mirror of ``unit_conv3d_desc``."""
    _fields_ = [(n, ctypes.c_int32) for n in
                ('n', 'c_in', 'd', 'h', 'w', 'c_out', 'kd', 'kh', 'kw', 'stride_d', 'stride_h', 'stride_w',
                 'pad_d', 'pad_h', 'pad_w')]


class TileEntry(ctypes.Structure):
    """Mirror of ``unit_tile_entry``."""
    _fields_ = [(n, ctypes.c_int32) for n in
                ('c_in', 'c_block', 'c_out', 'kh', 'kw', 'stride_h', 'stride_w', 'n', 'h', 'w', 'bn', 'kc', 'mt', 'ksplit')]


class Epilogue(ctypes.Structure):
    """Mirror of ``unit_epilogue``."""
    _fields_ = [('d_bias', ctypes.c_void_p), ('mul', ctypes.c_int32), ('shift', ctypes.c_int32),
                ('out_u8', ctypes.c_int32), ('d_residual', ctypes.c_void_p), ('x_signed', ctypes.c_int32)]


class ConvPlan(ctypes.Structure):
    """Mirror of ``unit_conv_plan`` (opaque bytes owned by the caller)."""
    _fields_ = [('opaque', ctypes.c_uint64 * 128)]


DEBUG_WAIT_LIMIT_NS = 1
DEBUG_STALL_WEIGHT_COPIES = 2

_dp = ctypes.POINTER(ConvDesc)
_ep = ctypes.POINTER(Epilogue)
_pp = ctypes.POINTER(ConvPlan)
_d3 = ctypes.POINTER(Conv3dDesc)
SIGNATURES = {
    'unit_version': (_ci, []),
    'unit_status_string': (ctypes.c_char_p, [_ci]),
    'unit_device_status': (_ci, [_vp]),
    'unit_launch_count': (ctypes.c_uint64, []),
    'unit_trace_attach': (_ci, [_vp, _ci]),
    'unit_tensor_peak': (_ci, [_ci, _ci, _ci, _ci, ctypes.POINTER(ctypes.c_double), _vp]),
    'unit_tile_table_set': (_ci, [ctypes.POINTER(TileEntry), _ci]),
    'unit_variant_count': (_ci, []),
    'unit_variant_name': (ctypes.c_char_p, [_ci]),
    'unit_variant_launches': (ctypes.c_uint64, [_ci]),
    'unit_debug_set': (_ci, [_ci, ctypes.c_longlong]),
    'unit_packed_weights_bytes_conv_i8': (_sz, [_dp]),
    'unit_pack_weights_conv_i8': (_ci, [_dp, _vp, _vp, _vp]),
    'unit_packed_weights_bytes_conv_f16': (_sz, [_dp]),
    'unit_pack_weights_conv_f16': (_ci, [_dp, _vp, _vp, _vp]),
    'unit_packed_weights_bytes_dense_i8': (_sz, [_ci, _ci]),
    'unit_pack_weights_dense_i8': (_ci, [_ci, _ci, _ci, _vp, _vp, _vp]),
    'unit_packed_weights_bytes_gemm_f16': (_sz, [_ci, _ci]),
    'unit_pack_weights_gemm_f16': (_ci, [_ci, _ci, _vp, _vp, _vp]),
    'unit_conv2d_workspace_bytes': (_sz, [_dp]),
    'unit_conv2d_u8s8s32_nchwc': (_ci, [_dp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    'unit_conv2d_u8s8_requant_nchwc': (_ci, [_dp, _vp, _vp, _vp, _ci, _vp, _vp, _sz, _vp]),
    'unit_conv2d_int8_nchwc': (_ci, [_dp, _vp, _vp, _ep, _vp, _vp, _sz, _vp]),
    'unit_conv2d_plan_int8': (_ci, [_dp, _vp, _vp, _ep, _vp, _vp, _sz, _pp]),
    'unit_conv2d_run': (_ci, [_pp, _vp]),
    'unit_packed_weights_bytes_conv3d_i8': (_sz, [_d3]),
    'unit_pack_weights_conv3d_i8': (_ci, [_d3, _vp, _vp, _vp]),
    'unit_conv3d_int8_ncdhwc': (_ci, [_d3, _vp, _vp, _ep, _vp, _vp]),
    'unit_noalloc_scratch_capacity': (_sz, []),
    'unit_conv2d_u8s8_requant_nchwc_noalloc': (_ci, [_dp, _vp, _vp, _vp, _ci, _vp, _vp]),
    'unit_dense_u8s8s32': (_ci, [_ci, _ci, _ci, _vp, _i64, _vp, _vp, _i64, _vp]),
    'unit_conv2d_f16f32_nchw16c': (_ci, [_dp, _vp, _vp, _vp, _vp]),
    'unit_gemm_f16f32': (_ci, [_ci, _ci, _ci, _vp, _i64, _vp, _vp, _i64, _vp]),
    'unit_pack_data_nchw_to_nchwc': (_ci, [_vp, _vp, _ci, _ci, _ci, _ci, _ci, _ci, _vp]),
    'unit_unpack_data_nchwc_to_nchw': (_ci, [_vp, _vp, _ci, _ci, _ci, _ci, _ci, _ci, _vp]),
    'unit_pack_weights_oihw_to_ref_i8': (_ci, [_vp, _vp, _ci, _ci, _ci, _ci, _ci, _vp]),
    'unit_pack_weights_oihw_to_ref_f16': (_ci, [_vp, _vp, _ci, _ci, _ci, _ci, _vp]),
}


def lib_path() -> str:
    """The in-tree library; UNIT_B200_LIB names another build of it (comparison runs of two builds)."""
    return os.environ.get('UNIT_B200_LIB') or _build.LIB_PATH


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is not None:
        return _LIB
    path = lib_path()
    if not os.path.exists(path):
        raise ImportError(
            f'unit_b200: {path} is missing; build it with `python -m unit_b200.build` '
            '(nvcc, sm_100a). There is no CPU or eager fallback.')
    L = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _LIB = L
    return L


class UnitError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f'{where}: status {status} ({STATUS.get(status, "unknown")})')


def check(status: int, where: str) -> None:
    if status == 0:
        return
    if status in (-1, -2, -3, -4, -8):
        raise ValueError(f'{where}: status {status} ({STATUS.get(status, "unknown")})')
    raise UnitError(status, where)
