"""numpy restatement of the reference's layouts and contractions.

TEST INFRASTRUCTURE ONLY: the checker for the CUDA kernels and the source of
the golden fixtures.  Nothing in ``unit_b200`` imports this module.

Two independent things live here so that layout bugs and arithmetic bugs are
caught separately:

* pack / unpack between logical tensors (NCHW, OIHW, row-major matrices) and
  the reference's blocked layouts;
* the contractions on *logical* tensors with int64 / fp32 accumulation.

Reference layouts followed (paths inside were/UNIT):

* data ``[N][C/cb][H][W][cb]`` (``NCHW16c``; ``NCHW4c`` for the 3-channel
  stem): apps/cpu/kernel/conv2d.py:18-30, python/tensorizer/ops/gpu.py:26-28
* int8 weights ``[O/16][C/cb][KH][KW][cb/4][16][4]`` indexed
  ``w[oc/16][ic/cb][kh][kw][(ic%cb)/4][oc%16][ic%4]``:
  apps/cpu/kernel/conv2d.py:26,30 and apps/cpu/kernel/conv3d.py:60-64
* int8 dense weights ``[N/T][K/4][T][4]``: apps/cpu/kernel/int8-gemm.py:11-14
* fp16 weights ``[O/16][C/16][KH][KW][16 i][16 o]``:
  python/tensorizer/ops/gpu.py:29-31
"""
from __future__ import annotations

import numpy as np


# --------------------------------------------------------------------------
# layouts
# --------------------------------------------------------------------------
def _pad_axis(a: np.ndarray, axis: int, mult: int) -> np.ndarray:
    n = a.shape[axis]
    r = (-n) % mult
    if r == 0:
        return a
    pad = [(0, 0)] * a.ndim
    pad[axis] = (0, r)
    return np.pad(a, pad)


def pack_nchw_to_nchwc(x: np.ndarray, cb: int = 16) -> np.ndarray:
    """NCHW -> [N][C/cb][H][W][cb]; channels zero-padded up to a multiple of cb
    (apps/cpu/kernel/conv2d.py:18-19 pads ic to a multiple of 4)."""
    x = _pad_axis(x, 1, cb)
    n, c, h, w = x.shape
    return np.ascontiguousarray(x.reshape(n, c // cb, cb, h, w).transpose(0, 1, 3, 4, 2))


def unpack_nchwc_to_nchw(x: np.ndarray, channels: int | None = None) -> np.ndarray:
    n, cc, h, w, cb = x.shape
    y = x.transpose(0, 1, 4, 2, 3).reshape(n, cc * cb, h, w)
    if channels is not None:
        y = y[:, :channels]
    return np.ascontiguousarray(y)


def pack_oihw_to_int8_weights(w: np.ndarray, cb: int = 16) -> np.ndarray:
    """OIHW s8 -> [O/16][I/cb][KH][KW][cb/4][16][4]."""
    w = _pad_axis(_pad_axis(w, 0, 16), 1, cb)
    o, i, kh, kw = w.shape
    w7 = w.reshape(o // 16, 16, i // cb, cb // 4, 4, kh, kw)
    #            0      1    2       3       4  5   6
    return np.ascontiguousarray(w7.transpose(0, 2, 5, 6, 3, 1, 4))


def unpack_int8_weights_to_oihw(wp: np.ndarray) -> np.ndarray:
    oc, icc, kh, kw, c4, l16, r4 = wp.shape
    w = wp.transpose(0, 5, 1, 4, 6, 2, 3)  # oc,16,icc,c4,4,kh,kw
    return np.ascontiguousarray(w.reshape(oc * 16, icc * c4 * 4, kh, kw))


def pack_dense_weights(b: np.ndarray, tile: int = 128) -> np.ndarray:
    """B logical [N][K] s8 -> [N/T][K/4][T][4]."""
    n, k = b.shape
    assert n % tile == 0 and k % 4 == 0
    return np.ascontiguousarray(b.reshape(n // tile, tile, k // 4, 4).transpose(0, 2, 1, 3))


def unpack_dense_weights(bp: np.ndarray) -> np.ndarray:
    nt, k4, t, r = bp.shape
    return np.ascontiguousarray(bp.transpose(0, 2, 1, 3).reshape(nt * t, k4 * r))


def pack_oihw_to_f16_weights(w: np.ndarray) -> np.ndarray:
    """OIHW fp16 -> [O/16][I/16][KH][KW][16 i][16 o]."""
    w = _pad_axis(_pad_axis(w, 0, 16), 1, 16)
    o, i, kh, kw = w.shape
    w6 = w.reshape(o // 16, 16, i // 16, 16, kh, kw)
    return np.ascontiguousarray(w6.transpose(0, 2, 4, 5, 3, 1))


def unpack_f16_weights_to_oihw(wp: np.ndarray) -> np.ndarray:
    oc, icc, kh, kw, ib, ob = wp.shape
    return np.ascontiguousarray(wp.transpose(0, 5, 1, 4, 2, 3).reshape(oc * 16, icc * 16, kh, kw))


# --------------------------------------------------------------------------
# contractions on logical tensors
# --------------------------------------------------------------------------
def _patches(x: np.ndarray, kh: int, kw: int, stride, pad) -> np.ndarray:
    """x NCHW -> view [N][C][KH][KW][OH][OW] of the zero-padded input."""
    sh, sw = stride
    ph, pw = pad
    xp = np.pad(x, ((0, 0), (0, 0), (ph, ph), (pw, pw)))
    n, c, h, w = xp.shape
    oh = (h - kh) // sh + 1
    ow = (w - kw) // sw + 1
    s = xp.strides
    return np.lib.stride_tricks.as_strided(
        xp, (n, c, kh, kw, oh, ow), (s[0], s[1], s[2], s[3], s[2] * sh, s[3] * sw), writeable=False)


def conv2d_int_nchw(x_u8: np.ndarray, w_s8: np.ndarray, stride=(1, 1), pad=(0, 0)) -> np.ndarray:
    """Exact integer conv on logical NCHW u8 x OIHW s8 -> int64 NCHW."""
    o, i, kh, kw = w_s8.shape
    p = _patches(x_u8.astype(np.int64), kh, kw, stride, pad)
    n, c, _, _, oh, ow = p.shape
    out = np.zeros((n, o, oh, ow), dtype=np.int64)
    wl = w_s8.astype(np.int64)
    for a in range(kh):
        for b in range(kw):
            out += np.einsum('nchw,oc->nohw', p[:, :, a, b], wl[:, :, a, b], optimize=True)
    return out


def requant_u8(acc: np.ndarray, bias: np.ndarray | None, shift: int = 8) -> np.ndarray:
    """q = clamp((acc + bias[oc] + 2^(shift-1)) >> shift, 0, 255), acc NCHW."""
    v = acc.astype(np.int64)
    if bias is not None:
        v = v + bias.astype(np.int64)[None, :, None, None]
    v = (v + (1 << (shift - 1))) >> shift
    return np.clip(v, 0, 255).astype(np.uint8)


def dense_int(a_u8: np.ndarray, b_s8_nk: np.ndarray) -> np.ndarray:
    """C[i][j] = sum_k A[i][k] * B[j][k], exact (poc/vnni/vnni_dense.py:60)."""
    return a_u8.astype(np.int64) @ b_s8_nk.astype(np.int64).T


def conv2d_f32_nchw(x_f16: np.ndarray, w_f16: np.ndarray, stride=(1, 1), pad=(0, 0)) -> np.ndarray:
    """fp16 inputs widened to fp32, fp32 accumulate (ops/gpu.py:41-43)."""
    o, i, kh, kw = w_f16.shape
    p = _patches(x_f16.astype(np.float32), kh, kw, stride, pad)
    n, c, _, _, oh, ow = p.shape
    out = np.zeros((n, o, oh, ow), dtype=np.float32)
    wl = w_f16.astype(np.float32)
    for a in range(kh):
        for b in range(kw):
            out += np.einsum('nchw,oc->nohw', p[:, :, a, b], wl[:, :, a, b], optimize=True).astype(np.float32)
    return out


def gemm_f32(a_f16: np.ndarray, b_f16_kn: np.ndarray) -> np.ndarray:
    return a_f16.astype(np.float32) @ b_f16_kn.astype(np.float32)
