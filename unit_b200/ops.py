"""Operator entry points with the reference's names, argument order and layouts.

Each function takes torch tensors (CUDA tensors, or host tensors which are
copied to the current device and whose result is copied back), checks the
layout contract, and calls the C ABI of ``libunit_b200.so`` with raw device
pointers on torch's current stream.  torch is used for device memory and
streams only; all arithmetic happens in the library's sm_100a kernels.

Reference counterparts (paths inside were/UNIT):

* ``conv2d_NCHWc_int8``  -- ``topi.nn.conv2d_NCHWc_int8`` as called in
  apps/cpu/kernel/conv2d.py:50-51 and scheduled by ``INTRINSICS['vnni']``
* ``dense_dotprod``      -- ``topi.x86.dense_dotprod`` as called in
  apps/cpu/kernel/int8-gemm.py:16
* ``conv2d_NCHW16c_OHWI16o`` / ``conv2d_NCHW16c_OHWI16o_compute`` --
  python/tensorizer/ops/gpu.py:8-58
* ``gemm_f16f32``        -- the tensor-core GEMM of apps/gpu/gemm.py:6-19
* ``INTRINSICS``         -- the registry of python/tensorizer/intrinsics/intrinsics.py:7-40
"""
from __future__ import annotations

import ctypes
import weakref
from typing import Optional, Sequence, Tuple, Union

import torch

from . import _lib
from ._lib import Conv3dDesc, ConvDesc, ConvPlan as _CPlan, Epilogue, check

IntPair = Union[int, Sequence[int]]


def _pair(v: IntPair) -> Tuple[int, int]:
    if isinstance(v, int):
        return (v, v)
    v = tuple(int(t) for t in v)
    if len(v) == 1:
        return (v[0], v[0])
    if len(v) == 2:
        return v
    if len(v) == 4:  # (top, left, bottom, right), symmetric only
        if v[0] != v[2] or v[1] != v[3]:
            raise ValueError('asymmetric padding is not supported')
        return (v[0], v[1])
    raise ValueError(f'bad pair {v}')


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


_TABLE_LOADED = False


def _require_cuda_lib():
    global _TABLE_LOADED
    if not torch.cuda.is_available():
        raise RuntimeError('unit_b200 operators need a CUDA device (sm_100a); there is no CPU fallback')
    L = _lib.lib()
    if not _TABLE_LOADED:
        _TABLE_LOADED = True
        from . import tile_table
        tile_table.load_default_table()   # per-shape tile overrides found by unit_b200.tune, if the file exists
    return L


def _to_device(t: torch.Tensor, dtype: torch.dtype, name: str) -> torch.Tensor:
    if t.dtype != dtype:
        raise TypeError(f'{name}: expected {dtype}, got {t.dtype}')
    if not t.is_cuda:
        t = t.cuda(non_blocking=True)
    return t.contiguous()


def device_status() -> None:
    """Synchronise the current stream and raise if a kernel flagged an error."""
    check(_lib.lib().unit_device_status(ctypes.c_void_p(_stream())), 'unit_device_status')


def launch_count() -> int:
    return int(_lib.lib().unit_launch_count())


# --------------------------------------------------------------------------
# packed weights
# --------------------------------------------------------------------------
class PackedWeights:
    """Tensor-core-ready copy of one weight tensor (device buffer + the geometry it was packed for)."""

    def __init__(self, kind: str, buf: torch.Tensor, key: tuple):
        self.kind = kind
        self.buf = buf
        self.key = key
        # the pack kernel was queued on the stream current at pack time: other streams wait for it once
        self._ready = torch.cuda.Event()
        self._ready.record()
        self._synced = {_stream()}

    def sync_to_current_stream(self) -> None:
        """Make the current stream wait for the pack kernel, once per stream.  (Not while the stream
        is being captured into a CUDA graph: a captured stream cannot wait for work outside the
        capture, and a capture is preceded by a warm-up call on that stream anyway.)"""
        st = _stream()
        if st in self._synced or torch.cuda.is_current_stream_capturing():
            return
        torch.cuda.current_stream().wait_event(self._ready)
        self._synced.add(st)

    @property
    def nbytes(self) -> int:
        return self.buf.numel()


_PACK_CACHE: dict = {}


def _cached(src: torch.Tensor, key: tuple, make) -> PackedWeights:
    from . import tile_table
    k = (id(src), src.data_ptr(), src._version, key, tile_table.version())   # the table shapes the packed form
    hit = _PACK_CACHE.get(k)
    if hit is not None and hit[0]() is src:
        return hit[1]
    pw = make()
    if len(_PACK_CACHE) > 512:
        _PACK_CACHE.clear()
    _PACK_CACHE[k] = (weakref.ref(src), pw)
    return pw


def _conv_desc(n, c_in, h, w, cb, c_out, kh, kw, stride, pad) -> ConvDesc:
    return ConvDesc(n, c_in, h, w, cb, c_out, kh, kw, stride[0], stride[1], pad[0], pad[1])


def pack_conv_weights_int8(kernel: torch.Tensor, stride: IntPair = 1, padding: IntPair = 0) -> PackedWeights:
    """kernel: s8 ``[O/16][I/cb][KH][KW][cb/4][16][4]`` (apps/cpu/kernel/conv2d.py:26,30).

    The packed form depends on the stride the convolution will use (the column-block width is
    chosen per stride) and, for NCHW4c kernels (cb = 4) and for strided kernels (whose pair form
    places the taps by the parity of the horizontal padding), on the padding as well.
    """
    L = _require_cuda_lib()
    kernel = _to_device(kernel, torch.int8, 'kernel')
    if kernel.dim() != 7 or kernel.shape[5] != 16 or kernel.shape[6] != 4 or kernel.shape[4] not in (1, 4):
        raise ValueError(f'kernel must be [O/16][I/cb][KH][KW][cb/4][16][4], got {tuple(kernel.shape)}')
    oc, icc, kh, kw, c4 = (int(s) for s in kernel.shape[:5])
    cb = c4 * 4
    stride = _pair(stride)
    padding = _pair(padding) if (cb == 4 or stride != (1, 1)) else (0, 0)
    key = ('conv_i8', oc * 16, icc * cb, cb, kh, kw, stride, padding)

    def make():
        d = _conv_desc(1, icc * cb, kh + 2 * 64, kw + 2 * 64, cb, oc * 16, kh, kw, stride, padding)
        nbytes = L.unit_packed_weights_bytes_conv_i8(ctypes.byref(d))
        if nbytes == 0:
            raise ValueError('unsupported convolution weights')
        buf = torch.empty(nbytes, dtype=torch.uint8, device=kernel.device)
        check(L.unit_pack_weights_conv_i8(ctypes.byref(d), _ptr(kernel), _ptr(buf), _stream()), 'unit_pack_weights_conv_i8')
        return PackedWeights('conv_i8', buf, key)

    with torch.cuda.device(kernel.device):
        return _cached(kernel, key, make)


def pack_conv_weights_f16(kernel: torch.Tensor) -> PackedWeights:
    """kernel: fp16 ``[O/16][I/16][KH][KW][16 i][16 o]`` (python/tensorizer/ops/gpu.py:29-31)."""
    L = _require_cuda_lib()
    kernel = _to_device(kernel, torch.float16, 'kernel')
    if kernel.dim() != 6 or kernel.shape[4] != 16 or kernel.shape[5] != 16:
        raise ValueError(f'kernel must be [O/16][I/16][KH][KW][16][16], got {tuple(kernel.shape)}')
    oc, icc, kh, kw = (int(s) for s in kernel.shape[:4])
    key = ('conv_f16', oc * 16, icc * 16, kh, kw)

    def make():
        d = _conv_desc(1, icc * 16, kh, kw, 16, oc * 16, kh, kw, (1, 1), (0, 0))
        nbytes = L.unit_packed_weights_bytes_conv_f16(ctypes.byref(d))
        if nbytes == 0:
            raise ValueError('unsupported convolution weights')
        buf = torch.empty(nbytes, dtype=torch.uint8, device=kernel.device)
        check(L.unit_pack_weights_conv_f16(ctypes.byref(d), _ptr(kernel), _ptr(buf), _stream()), 'unit_pack_weights_conv_f16')
        return PackedWeights('conv_f16', buf, key)

    with torch.cuda.device(kernel.device):
        return _cached(kernel, key, make)


def pack_dense_weights_int8(weight: torch.Tensor) -> PackedWeights:
    """weight: s8 ``[N/T][K/4][T][4]`` (apps/cpu/kernel/int8-gemm.py:11-14)."""
    L = _require_cuda_lib()
    weight = _to_device(weight, torch.int8, 'weight')
    if weight.dim() != 4 or weight.shape[3] != 4:
        raise ValueError(f'weight must be [N/T][K/4][T][4], got {tuple(weight.shape)}')
    nt, k4, t = (int(s) for s in weight.shape[:3])
    n, k = nt * t, k4 * 4
    key = ('dense_i8', n, k, t)

    def make():
        nbytes = L.unit_packed_weights_bytes_dense_i8(n, k)
        if nbytes == 0:
            raise ValueError(f'dense weights need N % 16 == 0 and K % 16 == 0, got N={n} K={k}')
        buf = torch.empty(nbytes, dtype=torch.uint8, device=weight.device)
        check(L.unit_pack_weights_dense_i8(n, k, t, _ptr(weight), _ptr(buf), _stream()), 'unit_pack_weights_dense_i8')
        return PackedWeights('dense_i8', buf, key)

    with torch.cuda.device(weight.device):
        return _cached(weight, key, make)


def pack_gemm_weights_f16(b: torch.Tensor) -> PackedWeights:
    """b: fp16 ``[K][N]`` row-major (apps/gpu/gemm.py:8)."""
    L = _require_cuda_lib()
    b = _to_device(b, torch.float16, 'b')
    if b.dim() != 2:
        raise ValueError('b must be [K][N]')
    k, n = int(b.shape[0]), int(b.shape[1])
    key = ('gemm_f16', n, k)

    def make():
        nbytes = L.unit_packed_weights_bytes_gemm_f16(n, k)
        if nbytes == 0:
            raise ValueError(f'gemm needs N % 16 == 0 and K % 8 == 0, got N={n} K={k}')
        buf = torch.empty(nbytes, dtype=torch.uint8, device=b.device)
        check(L.unit_pack_weights_gemm_f16(n, k, _ptr(b), _ptr(buf), _stream()), 'unit_pack_weights_gemm_f16')
        return PackedWeights('gemm_f16', buf, key)

    with torch.cuda.device(b.device):
        return _cached(b, key, make)


# --------------------------------------------------------------------------
# int8 path
# --------------------------------------------------------------------------
_WORKSPACES: dict = {}


_RETIRED_WORKSPACES: list = []


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Scratch buffer per (device, stream), grown on demand; calls on one stream run in order,
    so they can share it.  A buffer that has been handed out is never freed (a captured CUDA
    graph or a plan may still name it): when a larger one is needed the old one is retired,
    not dropped."""
    key = (device.index, _stream())
    buf = _WORKSPACES.get(key)
    if buf is None or buf.numel() < nbytes:
        if buf is not None:
            _RETIRED_WORKSPACES.append(buf)
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _WORKSPACES[key] = buf
    return buf



class ConvPlan:
    """A prepared int8 convolution bound to its buffers: ``run()`` is one call into the library
    with no argument checks, tile selection or tensor-map encoding (``unit_conv2d_plan_int8`` /
    ``unit_conv2d_run``).  The counterpart of calling a built TVM module repeatedly
    (poc/vnni/vnni_dense.py:40-66).  Keeps its tensors alive."""

    def __init__(self, plan: _CPlan, out: torch.Tensor, keep: tuple):
        self._plan = plan
        self._ref = ctypes.byref(plan)
        self.out = out
        self._keep = keep
        self._run = _lib.lib().unit_conv2d_run

    def run(self) -> torch.Tensor:
        rc = self._run(self._ref, torch.cuda.current_stream().cuda_stream)
        if rc:
            check(rc, 'unit_conv2d_run')
        return self.out


_PLAN_CACHE: dict = {}      # prepared launches of conv2d_NCHWc_int8 calls that named their output buffer
_PLAN_CACHE_MAX = 512


def _conv_int8_prepare(data, kernel, stride, padding, dilation, out_layout, out_dtype, bias, requant_shift, mul,
                       residual, out):
    """Shared front end of ``conv2d_NCHWc_int8`` and ``conv2d_NCHWc_int8_plan``: checks the layout
    contract and returns (library, descriptor, tensors, epilogue, out, workspace, host flag)."""
    L = _require_cuda_lib()
    if _pair(dilation) != (1, 1):
        raise ValueError('dilation other than 1 is not supported (the reference only uses 1)')
    if out_layout != 'NCHW16c':
        raise ValueError("out_layout must be 'NCHW16c'")
    if out_dtype not in ('int32', 'uint8'):
        raise ValueError("out_dtype must be 'int32' or 'uint8'")
    stride, padding = _pair(stride), _pair(padding)
    host = not data.is_cuda
    if data.dtype not in (torch.uint8, torch.int8):
        raise TypeError(f'data: expected torch.uint8 (or torch.int8 for signed activations), got {data.dtype}')
    signed = data.dtype == torch.int8
    data = _to_device(data, data.dtype, 'data')
    if data.dim() != 5 or data.shape[4] not in (4, 16):
        raise ValueError(f'data must be [N][C/cb][H][W][cb] with cb in (4, 16), got {tuple(data.shape)}')
    n, cc, h, w, cb = (int(s) for s in data.shape)
    with torch.cuda.device(data.device):
        pw = kernel if isinstance(kernel, PackedWeights) else pack_conv_weights_int8(kernel, stride, padding)
        if pw.kind != 'conv_i8':
            raise ValueError('kernel was packed for a different operator')
        pw.sync_to_current_stream()
        _, c_out, c_in, pcb, kh, kw, pstride, ppad = pw.key
        if c_in != cc * cb or pcb != cb:
            raise ValueError(f'channel mismatch: data has {cc}x{cb}, kernel expects {c_in} in blocks of {pcb}')
        if pstride != stride or ((cb == 4 or stride != (1, 1)) and ppad != padding):
            raise ValueError('weights were packed for a different stride (or, NCHW4c and strided kernels, padding)')
        requant = out_dtype == 'uint8' or requant_shift is not None or residual is not None
        shift = (8 if requant_shift is None else int(requant_shift)) if requant else 0
        if requant and int(mul) != 1:
            raise ValueError('mul applies to the int32 output only')
        d = _conv_desc(n, c_in, h, w, cb, c_out, kh, kw, stride, padding)
        if h + 2 * padding[0] < kh or w + 2 * padding[1] < kw:
            raise ValueError('kernel larger than padded input')
        oh = (h + 2 * padding[0] - kh) // stride[0] + 1
        ow = (w + 2 * padding[1] - kw) // stride[1] + 1
        if bias is not None:
            bias = _to_device(bias, torch.int32, 'bias')
            if bias.numel() != c_out:
                raise ValueError(f'bias must have {c_out} elements')
        oshape = (n, c_out // 16, oh, ow, 16)
        if residual is not None:
            residual = _to_device(residual, torch.uint8, 'residual')
            if tuple(residual.shape) != oshape:
                raise ValueError(f'residual must have the output shape {oshape}')
        odt = torch.uint8 if requant else torch.int32
        if out is None:
            out_t = torch.empty(oshape, dtype=odt, device=data.device)
        else:
            out_t = out
            if tuple(out_t.shape) != oshape or out_t.dtype != odt or not out_t.is_cuda or not out_t.is_contiguous():
                raise ValueError(f'out must be a contiguous CUDA {odt} tensor of shape {oshape}')
        ws_bytes = int(L.unit_conv2d_workspace_bytes(ctypes.byref(d))) if n > 0 else 0
        ws = _workspace(data.device, ws_bytes) if ws_bytes else None
        epi = Epilogue(None if bias is None else bias.data_ptr(), int(mul), shift, 1 if requant else 0,
                       None if residual is None else residual.data_ptr(), 1 if signed else 0)
    return L, d, (data, pw, bias, residual), epi, out_t, ws, ws_bytes, host, n


def conv2d_NCHWc_int8(data: torch.Tensor, kernel, stride: IntPair = 1, padding: IntPair = 0, dilation: IntPair = 1,
                      layout: str = 'NCHW4c', out_layout: str = 'NCHW16c', out_dtype: str = 'int32', *,
                      bias: Optional[torch.Tensor] = None, requant_shift: Optional[int] = None, mul: int = 1,
                      residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """u8 x s8 -> s32 convolution on blocked layouts.

    data   u8  ``[N][C/cb][H][W][cb]``, cb = 16 (or 4 for a 3/4-channel stem); an s8 tensor
           selects signed activations (the reference shifts them to u8 and compensates,
           apps/cpu/relay/result.log:4-6,15-21; the tensor core takes s8 x s8 as it is)
    kernel s8  ``[O/16][C/cb][KH][KW][cb/4][16][4]`` or a ``PackedWeights``
    result s32 ``[N][O/16][OH][OW][16]`` = ``(acc + bias) * mul`` (``mul = 11`` is the reference's
    fused graph operator, apps/cpu/relay/conv2d.py:21-23); with ``out_dtype='uint8'`` (or
    ``requant_shift`` / ``residual``) the fused epilogue
    ``clamp(((acc + bias + 2^(shift-1)) >> shift) + residual, 0, 255)`` gives u8 instead.
    ``layout`` is accepted for signature compatibility; the channel block is
    read from ``data``'s last dimension as the reference's compute does.
    """
    # Repeated calls on the same device buffers (the caller passes ``out``) reuse the prepared launch:
    # the checks, the tile selection and the tensor-map encoding are done once per distinct call.
    key = None
    if out is not None and data.is_cuda and isinstance(kernel, PackedWeights):
        from . import tile_table
        key = (data.data_ptr(), tuple(data.shape), data.dtype, kernel.buf.data_ptr(), kernel.key, stride, padding, dilation,
               out_layout, out_dtype, None if bias is None else (bias.data_ptr(), bias.dtype, bias.numel()), requant_shift, mul,
               None if residual is None else (residual.data_ptr(), tuple(residual.shape), residual.dtype),
               out.data_ptr(), tuple(out.shape), out.dtype, out.is_contiguous(), _stream(), tile_table.version())
        hit = _PLAN_CACHE.get(key)
        if hit is not None:
            rc = hit[1](hit[2], key[-2])
            if rc:
                check(rc, 'unit_conv2d_run')
            return out
    L, d, tensors, epi, out_t, ws, ws_bytes, host, n = _conv_int8_prepare(
        data, kernel, stride, padding, dilation, out_layout, out_dtype, bias, requant_shift, mul, residual, out)
    if n == 0:
        return out_t.cpu() if (host and out is None) else out_t
    x, pw = tensors[0], tensors[1]
    with torch.cuda.device(x.device):
        if key is not None and tensors[2] is bias and tensors[3] is residual:
            plan = _CPlan()
            check(L.unit_conv2d_plan_int8(ctypes.byref(d), _ptr(x), _ptr(pw.buf), ctypes.byref(epi), _ptr(out_t), _ptr(ws),
                                          ws_bytes, ctypes.byref(plan)), 'unit_conv2d_plan_int8')
            if len(_PLAN_CACHE) >= _PLAN_CACHE_MAX:
                _PLAN_CACHE.pop(next(iter(_PLAN_CACHE)))
            # (the entry holds no tensor: like the call itself it is valid for as long as the caller's buffers are)
            _PLAN_CACHE[key] = (plan, L.unit_conv2d_run, ctypes.byref(plan))
            check(L.unit_conv2d_run(ctypes.byref(plan), _stream()), 'unit_conv2d_run')
        else:
            check(L.unit_conv2d_int8_nchwc(ctypes.byref(d), _ptr(x), _ptr(pw.buf), ctypes.byref(epi), _ptr(out_t), _ptr(ws),
                                           ws_bytes, _stream()), 'unit_conv2d_int8_nchwc')
    return out_t.cpu() if (host and out is None) else out_t


def conv2d_NCHWc_int8_plan(data: torch.Tensor, kernel, stride: IntPair = 1, padding: IntPair = 0,
                           dilation: IntPair = 1, layout: str = 'NCHW4c', out_layout: str = 'NCHW16c',
                           out_dtype: str = 'int32', *, bias: Optional[torch.Tensor] = None,
                           requant_shift: Optional[int] = None, mul: int = 1,
                           residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> ConvPlan:
    """Same arguments as ``conv2d_NCHWc_int8`` (CUDA tensors only); returns a ``ConvPlan`` whose
    ``run()`` repeats the convolution on these buffers."""
    if not data.is_cuda:
        raise ValueError('a plan is bound to device buffers: pass CUDA tensors')
    L, d, tensors, epi, out_t, ws, ws_bytes, _host, n = _conv_int8_prepare(
        data, kernel, stride, padding, dilation, out_layout, out_dtype, bias, requant_shift, mul, residual, out)
    if n == 0:
        raise ValueError('empty batch')
    x, pw = tensors[0], tensors[1]
    plan = _CPlan()
    with torch.cuda.device(x.device):
        check(L.unit_conv2d_plan_int8(ctypes.byref(d), _ptr(x), _ptr(pw.buf), ctypes.byref(epi), _ptr(out_t), _ptr(ws),
                                      ws_bytes, ctypes.byref(plan)), 'unit_conv2d_plan_int8')
    return ConvPlan(plan, out_t, tensors + (ws,))


def _triple(v) -> Tuple[int, int, int]:
    if isinstance(v, int):
        return (v, v, v)
    v = tuple(int(t) for t in v)
    if len(v) != 3:
        raise ValueError(f'expected one or three values, got {v}')
    return v


def pack_conv3d_weights_int8(kernel: torch.Tensor, stride=1) -> PackedWeights:
    """kernel: s8 ``[O/16][I/16][KD][KH][KW][4][16][4]`` (apps/cpu/kernel/conv3d.py:41)."""
    L = _require_cuda_lib()
    kernel = _to_device(kernel, torch.int8, 'kernel')
    if kernel.dim() != 8 or tuple(kernel.shape[5:]) != (4, 16, 4):
        raise ValueError(f'kernel must be [O/16][I/16][KD][KH][KW][4][16][4], got {tuple(kernel.shape)}')
    oc, icc, kd, kh, kw = (int(s) for s in kernel.shape[:5])
    stride = _triple(stride)
    key = ('conv3d_i8', oc * 16, icc * 16, kd, kh, kw, stride)

    def make():
        d = Conv3dDesc(1, icc * 16, kd + 32, kh + 32, kw + 32, oc * 16, kd, kh, kw, stride[0], stride[1], stride[2], 0, 0, 0)
        nbytes = L.unit_packed_weights_bytes_conv3d_i8(ctypes.byref(d))
        if nbytes == 0:
            raise ValueError('unsupported convolution weights')
        buf = torch.empty(nbytes, dtype=torch.uint8, device=kernel.device)
        check(L.unit_pack_weights_conv3d_i8(ctypes.byref(d), _ptr(kernel), _ptr(buf), _stream()), 'unit_pack_weights_conv3d_i8')
        return PackedWeights('conv3d_i8', buf, key)

    with torch.cuda.device(kernel.device):
        return _cached(kernel, key, make)


def conv3d_NCDHWc_int8(data: torch.Tensor, kernel, stride=1, padding=0, out_dtype: str = 'int32', *,
                       bias: Optional[torch.Tensor] = None, requant_shift: Optional[int] = None, mul: int = 1,
                       out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """u8 (or s8) x s8 -> s32 three-dimensional convolution on ``[N][C/16][D][H][W][16]`` data with
    ``[O/16][C/16][KD][KH][KW][4][16][4]`` weights (apps/cpu/kernel/conv3d.py:39-64); result
    ``[N][O/16][OD][OH][OW][16]``.  Epilogue options as for ``conv2d_NCHWc_int8``."""
    L = _require_cuda_lib()
    stride, padding = _triple(stride), _triple(padding)
    if out_dtype not in ('int32', 'uint8'):
        raise ValueError("out_dtype must be 'int32' or 'uint8'")
    host = not data.is_cuda
    if data.dtype not in (torch.uint8, torch.int8):
        raise TypeError(f'data: expected torch.uint8 (or torch.int8), got {data.dtype}')
    signed = data.dtype == torch.int8
    data = _to_device(data, data.dtype, 'data')
    if data.dim() != 6 or data.shape[5] != 16:
        raise ValueError(f'data must be [N][C/16][D][H][W][16], got {tuple(data.shape)}')
    n, cc, dd, h, w, _ = (int(s) for s in data.shape)
    with torch.cuda.device(data.device):
        pw = kernel if isinstance(kernel, PackedWeights) else pack_conv3d_weights_int8(kernel, stride)
        if pw.kind != 'conv3d_i8':
            raise ValueError('kernel was packed for a different operator')
        pw.sync_to_current_stream()
        _, c_out, c_in, kd, kh, kw, pstride = pw.key
        if c_in != cc * 16:
            raise ValueError(f'channel mismatch: data has {cc * 16}, kernel expects {c_in}')
        if pstride != stride:
            raise ValueError('weights were packed for a different stride')
        if dd + 2 * padding[0] < kd or h + 2 * padding[1] < kh or w + 2 * padding[2] < kw:
            raise ValueError('kernel larger than padded input')
        requant = out_dtype == 'uint8' or requant_shift is not None
        shift = (8 if requant_shift is None else int(requant_shift)) if requant else 0
        if requant and int(mul) != 1:
            raise ValueError('mul applies to the int32 output only')
        od = (dd + 2 * padding[0] - kd) // stride[0] + 1
        oh = (h + 2 * padding[1] - kh) // stride[1] + 1
        ow = (w + 2 * padding[2] - kw) // stride[2] + 1
        if bias is not None:
            bias = _to_device(bias, torch.int32, 'bias')
            if bias.numel() != c_out:
                raise ValueError(f'bias must have {c_out} elements')
        oshape = (n, c_out // 16, od, oh, ow, 16)
        odt = torch.uint8 if requant else torch.int32
        if out is None:
            out_t = torch.empty(oshape, dtype=odt, device=data.device)
        else:
            out_t = out
            if tuple(out_t.shape) != oshape or out_t.dtype != odt or not out_t.is_cuda or not out_t.is_contiguous():
                raise ValueError(f'out must be a contiguous CUDA {odt} tensor of shape {oshape}')
        if n == 0:
            return out_t.cpu() if (host and out is None) else out_t
        d = Conv3dDesc(n, c_in, dd, h, w, c_out, kd, kh, kw, stride[0], stride[1], stride[2], padding[0], padding[1], padding[2])
        epi = Epilogue(None if bias is None else bias.data_ptr(), int(mul), shift, 1 if requant else 0, None, 1 if signed else 0)
        check(L.unit_conv3d_int8_ncdhwc(ctypes.byref(d), _ptr(data), _ptr(pw.buf), ctypes.byref(epi), _ptr(out_t), _stream()),
              'unit_conv3d_int8_ncdhwc')
    return out_t.cpu() if (host and out is None) else out_t


def dense_dotprod(data: torch.Tensor, weight, bias: Optional[torch.Tensor] = None, out_dtype: str = 'int32', *,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C[i][j] = sum_k u8 data[i][k] * s8 weight[j/T][k/4][j%T][k%4]  -> s32 [M][N]."""
    L = _require_cuda_lib()
    if out_dtype != 'int32':
        raise ValueError("out_dtype must be 'int32'")
    if bias is not None:
        raise ValueError('bias is not supported (the reference passes None)')
    host = not data.is_cuda
    data = _to_device(data, torch.uint8, 'data')
    if data.dim() != 2:
        raise ValueError('data must be [M][K]')
    m, k = int(data.shape[0]), int(data.shape[1])
    with torch.cuda.device(data.device):
        pw = weight if isinstance(weight, PackedWeights) else pack_dense_weights_int8(weight)
        pw.sync_to_current_stream()
        if pw.kind != 'dense_i8':
            raise ValueError('weight was packed for a different operator')
        _, n, pk, _t = pw.key
        if pk != k:
            raise ValueError(f'K mismatch: data has {k}, weight has {pk}')
        if out is None:
            out_t = torch.empty((m, n), dtype=torch.int32, device=data.device)
        else:
            out_t = out
            if tuple(out_t.shape) != (m, n) or out_t.dtype != torch.int32 or not out_t.is_cuda or not out_t.is_contiguous():
                raise ValueError('out must be a contiguous CUDA int32 [M][N] tensor')
        if m > 0:
            check(L.unit_dense_u8s8s32(m, n, k, _ptr(data), k, _ptr(pw.buf), _ptr(out_t), n, _stream()),
                  'unit_dense_u8s8s32')
    return out_t.cpu() if (host and out is None) else out_t


# --------------------------------------------------------------------------
# fp16 path
# --------------------------------------------------------------------------
def pack_data_nchwc(x: torch.Tensor, c_block: int = 16) -> torch.Tensor:
    """NCHW -> ``[N][ceil(C/cb)][H][W][cb]`` on the device (python/tensorizer/ops/gpu.py:26-28)."""
    L = _require_cuda_lib()
    if x.dim() != 4:
        raise ValueError('x must be NCHW')
    if not x.is_cuda:
        x = x.cuda(non_blocking=True)
    x = x.contiguous()
    n, c, h, w = (int(s) for s in x.shape)
    cc = (c + c_block - 1) // c_block
    y = torch.empty((n, cc, h, w, c_block), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        check(L.unit_pack_data_nchw_to_nchwc(_ptr(x), _ptr(y), n, c, h, w, c_block, x.element_size(), _stream()),
              'unit_pack_data_nchw_to_nchwc')
    return y


def unpack_data_nchwc(x: torch.Tensor, channels: Optional[int] = None) -> torch.Tensor:
    """``[N][C/cb][H][W][cb]`` -> NCHW, keeping the first ``channels`` channels."""
    L = _require_cuda_lib()
    if x.dim() != 5:
        raise ValueError('x must be [N][C/cb][H][W][cb]')
    if not x.is_cuda:
        x = x.cuda(non_blocking=True)
    x = x.contiguous()
    n, cc, h, w, cb = (int(s) for s in x.shape)
    c = cc * cb if channels is None else int(channels)
    if c < 1 or c > cc * cb or (c + cb - 1) // cb != cc:
        raise ValueError(f'channels must fill {cc} blocks of {cb} (last block partly): got {c}')
    y = torch.empty((n, c, h, w), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        check(L.unit_unpack_data_nchwc_to_nchw(_ptr(x), _ptr(y), n, c, h, w, cb, x.element_size(), _stream()),
              'unit_unpack_data_nchwc_to_nchw')
    return y


def pack_weights_oihw_int8(w: torch.Tensor, c_block: int = 16) -> torch.Tensor:
    """OIHW s8 -> the reference's ``[O/16][I/cb][KH][KW][cb/4][16][4]`` array, zero padded."""
    L = _require_cuda_lib()
    w = _to_device(w, torch.int8, 'w')
    o, i, kh, kw = (int(s) for s in w.shape)
    y = torch.empty(((o + 15) // 16, (i + c_block - 1) // c_block, kh, kw, c_block // 4, 16, 4), dtype=torch.int8,
                    device=w.device)
    with torch.cuda.device(w.device):
        check(L.unit_pack_weights_oihw_to_ref_i8(_ptr(w), _ptr(y), o, i, kh, kw, c_block, _stream()),
              'unit_pack_weights_oihw_to_ref_i8')
    return y


def pack_weights_oihw_f16(w: torch.Tensor) -> torch.Tensor:
    """OIHW fp16 -> ``[O/16][I/16][KH][KW][16 i][16 o]`` (python/tensorizer/ops/gpu.py:29-31)."""
    L = _require_cuda_lib()
    w = _to_device(w, torch.float16, 'w')
    o, i, kh, kw = (int(s) for s in w.shape)
    y = torch.empty(((o + 15) // 16, (i + 15) // 16, kh, kw, 16, 16), dtype=torch.float16, device=w.device)
    with torch.cuda.device(w.device):
        check(L.unit_pack_weights_oihw_to_ref_f16(_ptr(w), _ptr(y), o, i, kh, kw, _stream()),
              'unit_pack_weights_oihw_to_ref_f16')
    return y


def conv2d_NCHW16c_OHWI16o(a: torch.Tensor, b, stride_h: int = 1, stride_w: int = 1, out_type: str = 'float32', *,
                           padding: IntPair = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp16 x fp16 -> fp32 convolution, the tensor-core operator of the reference.

    Like the reference's compute it takes either 4-D NCHW data with OIHW
    weights (packed here first) or 5-D ``[N][C/16][H][W][16]`` data with 6-D
    ``[O/16][C/16][KH][KW][16][16]`` weights; the result is always
    ``[N][O/16][OH][OW][16]`` fp32.  The reference convolves without padding;
    ``padding`` adds implicit zero padding.
    """
    L = _require_cuda_lib()
    if out_type != 'float32':
        raise ValueError("out_type must be 'float32'")
    padding = _pair(padding)
    host = not a.is_cuda
    a = _to_device(a, torch.float16, 'a')
    if a.dim() == 4:
        if isinstance(b, PackedWeights) or b.dim() != 4:
            raise ValueError('4-D data needs 4-D OIHW weights')
        a = pack_data_nchwc(a, 16)
        b = pack_weights_oihw_f16(b if b.is_cuda else b.cuda(non_blocking=True))
    elif a.dim() != 5 or a.shape[4] != 16:
        raise ValueError('a must be NCHW or [N][C/16][H][W][16]')
    n, cc, h, w, _ = (int(s) for s in a.shape)
    with torch.cuda.device(a.device):
        pw = b if isinstance(b, PackedWeights) else pack_conv_weights_f16(b)
        pw.sync_to_current_stream()
        if pw.kind != 'conv_f16':
            raise ValueError('b was packed for a different operator')
        _, c_out, c_in, kh, kw = pw.key
        if c_in != cc * 16:
            raise ValueError(f'channel mismatch: data has {cc * 16}, weights expect {c_in}')
        if h + 2 * padding[0] < kh or w + 2 * padding[1] < kw:
            raise ValueError('kernel larger than padded input')
        d = _conv_desc(n, c_in, h, w, 16, c_out, kh, kw, (int(stride_h), int(stride_w)), padding)
        oh = (h + 2 * padding[0] - kh) // int(stride_h) + 1
        ow = (w + 2 * padding[1] - kw) // int(stride_w) + 1
        oshape = (n, c_out // 16, oh, ow, 16)
        if out is None:
            out_t = torch.empty(oshape, dtype=torch.float32, device=a.device)
        else:
            out_t = out
            if tuple(out_t.shape) != oshape or out_t.dtype != torch.float32 or not out_t.is_cuda or not out_t.is_contiguous():
                raise ValueError(f'out must be a contiguous CUDA float32 tensor of shape {oshape}')
        if n == 0:
            return out_t.cpu() if (host and out is None) else out_t
        check(L.unit_conv2d_f16f32_nchw16c(ctypes.byref(d), _ptr(a), _ptr(pw.buf), _ptr(out_t), _stream()),
              'unit_conv2d_f16f32_nchw16c')
    return out_t.cpu() if (host and out is None) else out_t


class _Attrs:
    """Minimal stand-in for the relay attrs object the reference's compute receives."""

    def __init__(self, strides=(1, 1), padding=(0, 0)):
        self._v = {'strides': tuple(strides), 'padding': tuple(padding)}

    def get_int_tuple(self, name):
        return self._v[name]


def conv2d_NCHW16c_OHWI16o_compute(attrs, inputs, out_type='float32'):
    """Same call shape as python/tensorizer/ops/gpu.py:56-58: returns a one-element list."""
    strides = attrs.get_int_tuple('strides')
    out_dtype = getattr(out_type, 'dtype', out_type)
    return [conv2d_NCHW16c_OHWI16o(inputs[0], inputs[1], strides[0], strides[1], out_dtype)]


def gemm_f16f32(a: torch.Tensor, b, *, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C[M][N] fp32 = A[M][K] fp16 . B[K][N] fp16 with fp32 accumulation."""
    L = _require_cuda_lib()
    host = not a.is_cuda
    a = _to_device(a, torch.float16, 'a')
    if a.dim() != 2:
        raise ValueError('a must be [M][K]')
    m, k = int(a.shape[0]), int(a.shape[1])
    with torch.cuda.device(a.device):
        pw = b if isinstance(b, PackedWeights) else pack_gemm_weights_f16(b)
        pw.sync_to_current_stream()
        if pw.kind != 'gemm_f16':
            raise ValueError('b was packed for a different operator')
        _, n, pk = pw.key
        if pk != k:
            raise ValueError(f'K mismatch: a has {k}, b has {pk}')
        if out is None:
            out_t = torch.empty((m, n), dtype=torch.float32, device=a.device)
        else:
            out_t = out
            if tuple(out_t.shape) != (m, n) or out_t.dtype != torch.float32 or not out_t.is_cuda or not out_t.is_contiguous():
                raise ValueError('out must be a contiguous CUDA float32 [M][N] tensor')
        if m > 0:
            check(L.unit_gemm_f16f32(m, n, k, _ptr(a), 2 * k, _ptr(pw.buf), _ptr(out_t), n, _stream()),
                  'unit_gemm_f16f32')
    return out_t.cpu() if (host and out is None) else out_t


# The reference registers its instructions in a dict keyed by instruction name
# (python/tensorizer/intrinsics/intrinsics.py:7-40).  The same keys map to the
# contraction each instruction performs and to the operators built on it here.
INTRINSICS = {
    'vnni': {
        'pattern': {'out_lanes': 16, 'reduce_lanes': 4, 'a_dtype': 'uint8', 'b_dtype': 'int8', 'out_dtype': 'int32'},
        'conv2d': conv2d_NCHWc_int8,
        'conv3d': conv3d_NCDHWc_int8,
        'dense': dense_dotprod,
    },
    'tensorcore': {
        'pattern': {'m': 16, 'n': 16, 'k': 16, 'a_dtype': 'float16', 'b_dtype': 'float16', 'out_dtype': 'float32'},
        'conv2d': conv2d_NCHW16c_OHWI16o,
        'gemm': gemm_f16f32,
    },
}
