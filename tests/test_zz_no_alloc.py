"""The allocation-free convolution entry point, through the C ABI.

Collected last on purpose: a run that stops at the first failure has already run everything
else.  Some hosts of the library cannot allocate device memory at call time (operators inside a
runtime with fully pre-planned buffers, serving loops that must not hit the synchronising
cudaMalloc); for them the library carries a fixed 8 MiB scratch array and this entry point uses
it instead of a caller workspace.  The check: same bytes out as the workspace entry point, on
two calls in a row with different inputs (the shared array keeps the first call's contents), and
a clean refusal beyond the limit.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_conv(L, fn_name, d, x, pw, bias, out, ws=None):
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
    if fn_name == 'noalloc':
        return L.unit_conv2d_u8s8_requant_nchwc_noalloc(ctypes.byref(d), p(x), p(pw), p(bias), 8, p(out), stream)
    return L.unit_conv2d_u8s8_requant_nchwc(ctypes.byref(d), p(x), p(pw), p(bias), 8, p(out), p(ws),
                                            0 if ws is None else ws.numel(), stream)


def test_noalloc_entry_point_matches_workspace_entry_point():
    assert torch.cuda.is_available()
    import unit_b200 as U
    from unit_b200 import _lib
    L = _lib.lib()
    assert L.unit_noalloc_scratch_capacity() == 8 << 20
    n, hw = 9, 64   # the folded image is 144 KB: large enough for the scratch path (tensor copies) to be taken
    d = _lib.ConvDesc(n, 4, hw, hw, 4, 64, 7, 7, 2, 2, 3, 3)
    need = L.unit_conv2d_workspace_bytes(ctypes.byref(d))
    assert 0 < need <= L.unit_noalloc_scratch_capacity()
    g = torch.Generator(device='cuda').manual_seed(5)
    w = torch.randint(-128, 128, (4, 1, 7, 7, 1, 16, 4), dtype=torch.int8, device='cuda', generator=g)
    bias = torch.randint(-2 ** 15, 2 ** 15, (64,), dtype=torch.int32, device='cuda', generator=g)
    pw = U.pack_conv_weights_int8(w, 2, 3).buf
    ws = torch.empty(need, dtype=torch.uint8, device='cuda')
    for call in range(2):  # two calls in a row, different data
        x = torch.randint(0, 256, (n, 1, hw, hw, 4), dtype=torch.uint8, device='cuda', generator=g)
        want = torch.empty((n, 4, hw // 2, hw // 2, 16), dtype=torch.uint8, device='cuda')
        got = torch.full_like(want, 7)
        assert _call_conv(L, 'workspace', d, x, pw, bias, want, ws) == 0
        assert _call_conv(L, 'noalloc', d, x, pw, bias, got) == 0
        U.device_status()
        assert torch.equal(got, want), f'call {call}: outputs differ'
    # the property the entry point exists for: a call obtains no device memory, neither from the
    # driver nor from torch's allocator
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    used0 = torch.cuda.memory_allocated()
    assert _call_conv(L, 'noalloc', d, x, pw, bias, got) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0 and torch.cuda.memory_allocated() == used0
    # a geometry that needs no scratch is forwarded unchanged
    d16 = _lib.ConvDesc(2, 32, 10, 10, 16, 32, 3, 3, 1, 1, 1, 1)
    x16 = torch.randint(0, 256, (2, 2, 10, 10, 16), dtype=torch.uint8, device='cuda', generator=g)
    w16 = torch.randint(-128, 128, (2, 2, 3, 3, 4, 16, 4), dtype=torch.int8, device='cuda', generator=g)
    pw16 = U.pack_conv_weights_int8(w16).buf
    want = torch.empty((2, 2, 10, 10, 16), dtype=torch.uint8, device='cuda')
    got = torch.empty_like(want)
    assert _call_conv(L, 'workspace', d16, x16, pw16, bias[:32].contiguous(), want) == 0
    assert _call_conv(L, 'noalloc', d16, x16, pw16, bias[:32].contiguous(), got) == 0
    U.device_status()
    assert torch.equal(got, want)


def test_noalloc_entry_point_refuses_sizes_beyond_its_scratch():
    from unit_b200 import _lib
    L = _lib.lib()
    # the documented edge: a 224 x 224 stem fits up to batch 41 (41 * 112 * 112 * 16 B <= 8 MiB < 42 * ...)
    cap = L.unit_noalloc_scratch_capacity()
    edge = lambda nb: L.unit_conv2d_workspace_bytes(ctypes.byref(_lib.ConvDesc(nb, 4, 224, 224, 4, 64, 7, 7, 2, 2, 3, 3)))
    assert edge(41) <= cap < edge(42)
    big = _lib.ConvDesc(64, 4, 224, 224, 4, 64, 7, 7, 2, 2, 3, 3)   # needs 64 * 112 * 112 * 16 B = 12.25 MiB
    assert L.unit_conv2d_workspace_bytes(ctypes.byref(big)) > L.unit_noalloc_scratch_capacity()
    buf = torch.empty(4096, dtype=torch.uint8, device='cuda')
    p = ctypes.c_void_p(buf.data_ptr())
    rc = L.unit_conv2d_u8s8_requant_nchwc_noalloc(ctypes.byref(big), p, p, None, 8, p, None)
    assert rc == -8 and L.unit_status_string(rc) == b'beyond a fixed capacity'
