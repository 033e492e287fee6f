"""ctypes front end of ``unit_oracle.c`` (TEST INFRASTRUCTURE ONLY).

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of
``bench.py`` load this module; ``unit_b200`` never does.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def host_has_vnni() -> bool:
    try:
        with open('/proc/cpuinfo') as f:
            txt = f.read()
    except OSError:
        return False
    return 'avx512_vnni' in txt and 'avx512f' in txt and 'avx512bw' in txt


def build(force: bool = False) -> None:
    """Compile both variants of the oracle with the system gcc."""
    want = [os.path.join(_HERE, n) for n in ('libunit_oracle_vnni.so', 'libunit_oracle_scalar.so')]
    src = os.path.join(_HERE, 'unit_oracle.c')
    fresh = all(os.path.exists(p) and os.path.getmtime(p) >= os.path.getmtime(src) for p in want)
    if fresh and not force:
        return
    env = dict(os.environ)
    env.pop('CC', None)
    env.pop('CXX', None)
    subprocess.run(['make', '-C', _HERE, '-B', 'all'], check=True, env=env,
                   stdout=subprocess.DEVNULL)


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is not None:
        return _LIB
    name = 'libunit_oracle_vnni.so' if host_has_vnni() else 'libunit_oracle_scalar.so'
    path = os.path.join(_HERE, name)
    if not os.path.exists(path):
        build()
    L = ctypes.CDLL(path)
    vp, ci = ctypes.c_void_p, ctypes.c_int
    L.oracle_has_vnni.restype = ci
    L.oracle_max_threads.restype = ci
    L.oracle_set_threads.argtypes = [ci]
    L.oracle_set_threads.restype = None
    L.oracle_vnni_dot.argtypes = [vp, vp, vp]
    L.oracle_vnni_dot_hw.argtypes = [vp, vp, vp]
    L.oracle_vnni_dot_hw.restype = ci
    conv_args = [vp, vp, vp, vp, vp, ci] + [ci] * 12
    for fn in (L.oracle_conv2d_u8s8, L.vnni_conv2d_u8s8):
        fn.argtypes = conv_args
        fn.restype = ci
    L.oracle_conv2d_i8_ex.argtypes = [vp, ci, vp, vp, ci, vp, vp, vp, ci] + [ci] * 12
    L.oracle_conv2d_i8_ex.restype = ci
    L.oracle_conv3d_u8s8.argtypes = [vp, vp, vp, vp] + [ci] * 15
    L.oracle_conv3d_u8s8.restype = ci
    for fn in (L.oracle_dense_u8s8s32, L.vnni_dense_u8s8s32):
        fn.argtypes = [vp, vp, vp, ci, ci, ci, ci]
        fn.restype = ci
    L.oracle_conv2d_f16f32.argtypes = [vp, vp, vp] + [ci] * 11
    L.oracle_conv2d_f16f32.restype = None
    L.oracle_gemm_f16f32.argtypes = [vp, vp, vp, ci, ci, ci]
    L.oracle_gemm_f16f32.restype = None
    _LIB = L
    return L


def use_all_cores() -> int:
    """Let the OpenMP baseline use every core this process may run on; returns the count."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    lib().oracle_set_threads(n)
    return int(lib().oracle_max_threads())


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dt):
    a = np.ascontiguousarray(a)
    assert a.dtype == dt, (a.dtype, dt)
    return a


def out_hw(h, w, kh, kw, stride, pad):
    return ((h + 2 * pad[0] - kh) // stride[0] + 1, (w + 2 * pad[1] - kw) // stride[1] + 1)


def conv2d_u8s8(x, w, stride=(1, 1), pad=(0, 0), bias=None, requant_shift=None, vnni=False, out=None):
    """x [N][Cc][H][W][cb] u8, w [Oc][Cc][KH][KW][cb/4][16][4] s8.

    Returns s32 [N][Oc][OH][OW][16] (bias added if given), or the requantised
    u8 tensor when ``requant_shift`` is set.  ``vnni=True`` runs the AVX-512
    restatement (the timed baseline) instead of the scalar definition.  ``out``: a preallocated
    result array (the timed baseline reuses one, so that page faults are not timed).
    """
    x = _c(x, np.uint8)
    w = _c(w, np.int8)
    n, cc, h, wd, cb = x.shape
    oc, cc2, kh, kw, c4, l16, r4 = w.shape
    assert cc2 == cc and c4 * 4 == cb and l16 == 16 and r4 == 4
    oh, ow = out_hw(h, wd, kh, kw, stride, pad)
    if bias is not None:
        bias = _c(bias, np.int32)
        assert bias.size == oc * 16
    odt = np.int32 if requant_shift is None else np.uint8
    if out is None:
        out = np.empty((n, oc, oh, ow, 16), odt)
    assert out.shape == (n, oc, oh, ow, 16) and out.dtype == odt and out.flags['C_CONTIGUOUS']
    if requant_shift is None:
        o32, o8, sh = out, None, 0
    else:
        o32, o8, sh = None, out, int(requant_shift)
    fn = lib().vnni_conv2d_u8s8 if vnni else lib().oracle_conv2d_u8s8
    rc = fn(_p(x), _p(w), _p(bias), _p(o32), _p(o8), sh, n, cc, h, wd, cb, oc, kh, kw,
            stride[0], stride[1], pad[0], pad[1])
    if rc < 0:
        raise RuntimeError('oracle: AVX-512 VNNI path not available on this host')
    if rc == 1:
        raise OverflowError('oracle: an accumulator left the s32 range')
    return out


def conv2d_i8_ex(x, w, stride=(1, 1), pad=(0, 0), bias=None, mul=1, requant_shift=None, residual=None):
    """The wider epilogue family: x u8 or s8 (by dtype), ``t = (acc + bias) * mul`` wrapping in s32
    (apps/cpu/relay/conv2d.py:21-23); s32 out, or with ``requant_shift`` the u8 result
    ``clamp(((t + 2^(shift-1)) >> shift) + residual, 0, 255)``."""
    x = np.ascontiguousarray(x)
    assert x.dtype in (np.uint8, np.int8)
    w = _c(w, np.int8)
    n, cc, h, wd, cb = x.shape
    oc, cc2, kh, kw, c4, l16, r4 = w.shape
    assert cc2 == cc and c4 * 4 == cb and l16 == 16 and r4 == 4
    oh, ow = out_hw(h, wd, kh, kw, stride, pad)
    if bias is not None:
        bias = _c(bias, np.int32)
        assert bias.size == oc * 16
    if residual is not None:
        residual = _c(residual, np.uint8)
        assert residual.shape == (n, oc, oh, ow, 16) and requant_shift is not None
    if requant_shift is None:
        out = np.empty((n, oc, oh, ow, 16), np.int32)
        o32, o8, sh = out, None, 0
    else:
        out = np.empty((n, oc, oh, ow, 16), np.uint8)
        o32, o8, sh = None, out, int(requant_shift)
    lib().oracle_conv2d_i8_ex(_p(x), int(x.dtype == np.int8), _p(w), _p(bias), int(mul), _p(residual), _p(o32), _p(o8),
                              sh, n, cc, h, wd, cb, oc, kh, kw, stride[0], stride[1], pad[0], pad[1])
    return out


def conv2d_s8s8_relay_flow(x_s8, w, stride=(1, 1), pad=(0, 0), bias=None, mul=1):
    """The reference's graph for signed activations, step by step (apps/cpu/relay/result.log):
    cast to s32, add 128, cast to u8 (:4-6); u8 x s8 convolution (:14); 128 * sum of each output
    channel's weights (:15-19) subtracted (:21); bias added (:23) and the s32 product with a
    constant (:24, apps/cpu/relay/conv2d.py:21-23).  The reference runs it without padding; with
    padding the shifted tensor is padded with 128 (the image of s8 zero) before a valid convolution."""
    x_s8 = np.ascontiguousarray(x_s8)
    assert x_s8.dtype == np.int8
    w = _c(w, np.int8)
    xu = (x_s8.astype(np.int32) + 128).astype(np.uint8)
    if pad != (0, 0):
        xu = np.pad(xu, ((0, 0), (0, 0), (pad[0], pad[0]), (pad[1], pad[1]), (0, 0)), constant_values=128)
    conv = conv2d_u8s8(xu, w, stride, (0, 0), vnni=host_has_vnni()).astype(np.int64)
    comp = 128 * w.astype(np.int64).sum(axis=(1, 2, 3, 4, 6))        # [Oc][16]: every input channel and tap
    t = conv - comp[None, :, None, None, :]
    if bias is not None:
        t = t + np.asarray(bias, np.int64).reshape(1, -1, 1, 1, 16)
    t = (t * int(mul)) & 0xFFFFFFFF
    return t.astype(np.uint32).view(np.int32)   # wrapping s32, as the reference's int32 arithmetic


def conv3d_u8s8(x, w, stride=(1, 1, 1), pad=(0, 0, 0), bias=None):
    """x [N][Cc][D][H][W][16] u8, w [Oc][Cc][KD][KH][KW][4][16][4] s8 -> s32 [N][Oc][OD][OH][OW][16]
    (apps/cpu/kernel/conv3d.py:58-64), bias added if given."""
    x = _c(x, np.uint8)
    w = _c(w, np.int8)
    n, cc, d, h, wd, cb = x.shape
    oc, cc2, kd, kh, kw, c4, l16, r4 = w.shape
    assert cb == 16 and cc2 == cc and c4 == 4 and l16 == 16 and r4 == 4
    od = (d + 2 * pad[0] - kd) // stride[0] + 1
    oh = (h + 2 * pad[1] - kh) // stride[1] + 1
    ow = (wd + 2 * pad[2] - kw) // stride[2] + 1
    if bias is not None:
        bias = _c(bias, np.int32)
        assert bias.size == oc * 16
    out = np.empty((n, oc, od, oh, ow, 16), np.int32)
    rc = lib().oracle_conv3d_u8s8(_p(x), _p(w), _p(bias), _p(out), n, cc, d, h, wd, oc, kd, kh, kw,
                                  stride[0], stride[1], stride[2], pad[0], pad[1], pad[2])
    if rc == 1:
        raise OverflowError('oracle: an accumulator left the s32 range')
    return out


def dense_u8s8s32(a, bp, vnni=False):
    a = _c(a, np.uint8)
    bp = _c(bp, np.int8)
    m, k = a.shape
    nt, k4, t, r4 = bp.shape
    assert k4 * 4 == k and r4 == 4
    c = np.empty((m, nt * t), np.int32)
    fn = lib().vnni_dense_u8s8s32 if vnni else lib().oracle_dense_u8s8s32
    rc = fn(_p(a), _p(bp), _p(c), m, nt * t, k, t)
    if rc < 0:
        raise RuntimeError('oracle: AVX-512 VNNI dense path not available (rc=%d)' % rc)
    if rc == 1:
        raise OverflowError('oracle: an accumulator left the s32 range')
    return c


def conv2d_f16f32(x, w, stride=(1, 1), pad=(0, 0)):
    x = _c(x, np.float16)
    w = _c(w, np.float16)
    n, cc, h, wd, cb = x.shape
    oc, cc2, kh, kw, ib, ob = w.shape
    assert cb == 16 and cc2 == cc and ib == 16 and ob == 16
    oh, ow = out_hw(h, wd, kh, kw, stride, pad)
    out = np.empty((n, oc, oh, ow, 16), np.float32)
    lib().oracle_conv2d_f16f32(_p(x), _p(w), _p(out), n, cc, h, wd, oc, kh, kw,
                               stride[0], stride[1], pad[0], pad[1])
    return out


def gemm_f16f32(a, b):
    a = _c(a, np.float16)
    b = _c(b, np.float16)
    m, k = a.shape
    k2, n = b.shape
    assert k2 == k
    c = np.empty((m, n), np.float32)
    lib().oracle_gemm_f16f32(_p(a), _p(b), _p(c), m, n, k)
    return c


def vnni_dot(a, b, c, hw=False):
    a = _c(a, np.uint8); b = _c(b, np.int8); c = _c(c, np.int32).copy()
    if hw:
        if lib().oracle_vnni_dot_hw(_p(a), _p(b), _p(c)) != 0:
            raise RuntimeError('no AVX-512 VNNI on this host')
    else:
        lib().oracle_vnni_dot(_p(a), _p(b), _p(c))
    return c
