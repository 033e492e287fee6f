"""The C-ABI library without a GPU: it loads, exports what the header declares,
and rejects bad arguments before touching the device.  CPU only."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope='module')
def L():
    from unit_b200 import _lib, build
    build.build()
    return _lib.lib()


def declared_functions():
    txt = open(os.path.join(ROOT, 'include', 'unit_b200.h')).read()
    txt = re.sub(r'/\*.*?\*/', '', txt, flags=re.S)
    return sorted(set(re.findall(r'\b(unit_[a-z0-9_]+)\s*\(', txt)))


def test_every_declared_symbol_is_exported_and_bound(L):
    from unit_b200 import _lib
    names = declared_functions()
    assert len(names) >= 20
    for n in names:
        assert hasattr(L, n), f'{n} declared in include/unit_b200.h but not exported'
        assert n in _lib.SIGNATURES, f'{n} has no ctypes signature'
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_status_strings(L):
    assert L.unit_version() >= 100
    seen = set()
    for s in range(0, -9, -1):
        msg = L.unit_status_string(s)
        assert msg and msg != b'unknown status'
        seen.add(msg)
    assert len(seen) == 9
    assert L.unit_status_string(-99) == b'unknown status'


def desc(**kw):
    from unit_b200._lib import ConvDesc
    d = dict(n=1, c_in=64, h=56, w=56, c_block=16, c_out=64, kh=3, kw=3, stride_h=1, stride_w=1, pad_h=1, pad_w=1)
    d.update(kw)
    return ConvDesc(**d)


def test_packed_weight_sizes_are_pure_host_functions(L):
    # 3x3 64->64: 36 K columns of 16 B, one 64-wide N tile; stride 1 with several taps and an even chunk
    # count carries a second copy in the window form's column order (the same size)
    assert L.unit_packed_weights_bytes_conv_i8(ctypes.byref(desc())) == 2 * 36 * 64 * 16
    # stride 2 with several taps per kernel row carries a second copy in the pair form's order: 3 kernel rows x
    # 2 pair offsets x 4 chunks x 2 half-columns = 48 columns (the 12 half-columns that are no tap hold zeros),
    # whatever the input size (the pack call does not know it; odd widths simply do not use the copy)
    assert L.unit_packed_weights_bytes_conv_i8(ctypes.byref(desc(stride_h=2, stride_w=2))) == 36 * 64 * 16 + 48 * 64 * 16
    assert L.unit_packed_weights_bytes_conv_i8(ctypes.byref(desc(stride_h=2, stride_w=2, w=55))) == 36 * 64 * 16 + 48 * 64 * 16
    assert L.unit_packed_weights_bytes_conv_i8(ctypes.byref(desc(stride_h=2, stride_w=2, kh=1, kw=1))) == 4 * 64 * 16
    # 1x1 512->2048: 32 columns, 8 N tiles of 256
    assert L.unit_packed_weights_bytes_conv_i8(ctypes.byref(desc(c_in=512, c_out=2048, kh=1, kw=1))) == 32 * 2048 * 16
    # stem: 7 kh x 2 groups of 4 kw taps = 14 columns in one stage, plus the 16 columns of the folded form
    assert L.unit_packed_weights_bytes_conv_i8(
        ctypes.byref(desc(c_in=4, c_block=4, kh=7, kw=7, h=224, w=224, stride_h=2, stride_w=2, pad_h=3, pad_w=3))) == 14 * 64 * 16 + 16 * 64 * 16
    # odd column count (9 taps x 1 chunk) is padded to an even number of columns
    assert L.unit_packed_weights_bytes_conv_i8(ctypes.byref(desc(c_in=16, c_out=16))) == 10 * 16 * 16
    assert L.unit_packed_weights_bytes_conv_f16(ctypes.byref(desc(c_in=256, c_out=256))) == 288 * 256 * 16
    assert L.unit_packed_weights_bytes_dense_i8(4096, 4096) == 4096 * 4096
    assert L.unit_packed_weights_bytes_gemm_f16(768, 3072) == 768 * 3072 * 2
    # the same stem with stride 1 has no folded form; scratch is needed only for the folded form
    stem = dict(c_in=4, c_block=4, kh=7, kw=7, h=224, w=224, pad_h=3, pad_w=3)
    assert L.unit_packed_weights_bytes_conv_i8(ctypes.byref(desc(**stem))) == 14 * 64 * 16
    assert L.unit_conv2d_workspace_bytes(ctypes.byref(desc(**stem))) == 0
    assert L.unit_conv2d_workspace_bytes(ctypes.byref(desc(stride_h=2, stride_w=2, n=3, **stem))) == 3 * 112 * 112 * 16
    assert L.unit_conv2d_workspace_bytes(ctypes.byref(desc(stride_h=2, stride_w=2, **dict(stem, h=223)))) == 0
    assert L.unit_conv2d_workspace_bytes(ctypes.byref(desc())) == 0
    # unsupported geometries report size 0
    assert L.unit_packed_weights_bytes_conv_i8(ctypes.byref(desc(c_out=20))) == 0
    assert L.unit_packed_weights_bytes_conv_i8(ctypes.byref(desc(c_block=8))) == 0
    assert L.unit_packed_weights_bytes_conv_f16(ctypes.byref(desc(c_block=4, c_in=4))) == 0
    assert L.unit_packed_weights_bytes_dense_i8(100, 64) == 0


def test_argument_checks_return_status_codes(L):
    buf = (ctypes.c_uint8 * 4096)()
    addr = ctypes.addressof(buf)
    addr += (-addr) % 16
    p = ctypes.c_void_p(addr)
    mis = ctypes.c_void_p(addr + 4)
    d = desc()
    assert L.unit_conv2d_u8s8s32_nchwc(None, p, p, None, p, None, 0, None) == -1
    assert L.unit_conv2d_u8s8s32_nchwc(ctypes.byref(d), None, p, None, p, None, 0, None) == -1
    assert L.unit_conv2d_u8s8s32_nchwc(ctypes.byref(d), mis, p, None, p, None, 0, None) == -3
    assert L.unit_conv2d_u8s8s32_nchwc(ctypes.byref(desc(kh=0)), p, p, None, p, None, 0, None) == -2
    assert L.unit_conv2d_u8s8s32_nchwc(ctypes.byref(desc(c_in=60)), p, p, None, p, None, 0, None) == -4
    assert L.unit_conv2d_u8s8s32_nchwc(ctypes.byref(desc(h=1, w=1, pad_h=0, pad_w=0)), p, p, None, p, None, 0, None) == -2
    assert L.unit_conv2d_u8s8_requant_nchwc(ctypes.byref(d), p, p, None, 0, p, None, 0, None) == -2
    assert L.unit_conv2d_u8s8_requant_nchwc(ctypes.byref(d), p, p, None, 32, p, None, 0, None) == -2
    assert L.unit_conv2d_f16f32_nchw16c(ctypes.byref(desc(c_block=4, c_in=4)), p, p, p, None) == -4
    assert L.unit_dense_u8s8s32(0, 64, 64, p, 64, p, p, 64, None) == -2
    assert L.unit_dense_u8s8s32(8, 60, 64, p, 64, p, p, 64, None) == -2
    assert L.unit_dense_u8s8s32(8, 64, 64, p, 72, p, p, 64, None) == -3   # pitch not a multiple of 16
    assert L.unit_dense_u8s8s32(8, 64, 64, p, 64, None, p, 64, None) == -1
    assert L.unit_gemm_f16f32(8, 64, 12, p, 24, p, p, 64, None) == -2
    assert L.unit_pack_weights_dense_i8(64, 64, 48, p, p, None) == -4
    assert L.unit_pack_weights_conv_i8(ctypes.byref(d), None, p, None) == -1
    assert L.unit_pack_data_nchw_to_nchwc(p, p, 1, 3, 4, 4, 8, 1, None) == -4
    assert L.unit_pack_data_nchw_to_nchwc(p, p, 1, 3, 4, 4, 16, 3, None) in (-4, -6)
    assert L.unit_unpack_data_nchwc_to_nchw(None, p, 1, 3, 4, 4, 16, 1, None) == -1


def test_valid_call_without_a_device_reports_arch_not_a_crash(L):
    import torch
    if torch.cuda.is_available():
        pytest.skip('a CUDA device is present')
    buf = (ctypes.c_uint8 * 4096)()
    addr = ctypes.addressof(buf)
    addr += (-addr) % 16
    p = ctypes.c_void_p(addr)
    assert L.unit_conv2d_u8s8s32_nchwc(ctypes.byref(desc()), p, p, None, p, None, 0, None) == -5
    assert L.unit_dense_u8s8s32(8, 64, 64, p, 64, p, p, 64, None) == -5
