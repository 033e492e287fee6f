"""Parity of the CUDA path against the oracle, through the operator entry points
(which call the C ABI).  Bit-exact for the int8 path; rel 1e-2 / abs 1e-3 for fp16."""
import numpy as np
import pytest
import torch

from oracle import np_oracle as no

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-2, 1e-3  # fp16 path tolerance stated by the task


@pytest.fixture(scope='module')
def U():
    assert torch.cuda.is_available(), 'GPU tests need a CUDA device'
    import unit_b200
    from unit_b200 import _lib
    _lib.lib()  # fails loudly if the CUDA library is missing
    return unit_b200


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def conv_case(U, oracle, rng, n, ci, h, w, co, kh, kw, s, p, cb=16, vnni=True, dist='uniform'):
    cs = (ci + cb - 1) // cb * cb
    if dist == 'uniform':
        x = rng.integers(0, 256, (n, cs // cb, h, w, cb), dtype=np.uint8)
        wt = rng.integers(-128, 128, (co // 16, cs // cb, kh, kw, cb // 4, 16, 4), dtype=np.int8)
    else:
        from unit_b200 import resnet50 as R
        x = R.synth_activations(rng, (n, cs // cb, h, w, cb))
        wt = R.synth_weights(rng, (co // 16, cs // cb, kh, kw, cb // 4, 16, 4))
    b = rng.integers(-2 ** 15, 2 ** 15, co, dtype=np.int32)
    use_vnni = vnni and oracle.host_has_vnni()
    ref = oracle.conv2d_u8s8(x, wt, (s, s), (p, p), vnni=use_vnni)
    refq = oracle.conv2d_u8s8(x, wt, (s, s), (p, p), bias=b, requant_shift=8, vnni=use_vnni)
    xd, wd, bd = dev(x), dev(wt), dev(b)
    got = U.conv2d_NCHWc_int8(xd, wd, stride=s, padding=p)
    gotq = U.conv2d_NCHWc_int8(xd, wd, stride=s, padding=p, bias=bd, out_dtype='uint8')
    U.device_status()
    assert np.array_equal(got.cpu().numpy(), ref)
    assert np.array_equal(gotq.cpu().numpy(), refq)


# ---------------------------------------------------------------------------
# golden fixtures
# ---------------------------------------------------------------------------
def test_golden_vectors(U, golden):
    g = golden
    x, w, b = dev(g['c1_x']), dev(g['c1_w']), dev(g['c1_bias'])
    assert np.array_equal(U.conv2d_NCHWc_int8(x, w, stride=1, padding=1).cpu().numpy(), g['c1_out'])
    assert np.array_equal(U.conv2d_NCHWc_int8(x, w, stride=2, padding=1).cpu().numpy(), g['c2_out'])
    assert np.array_equal(U.conv2d_NCHWc_int8(x, w, stride=1, padding=1, bias=b, out_dtype='uint8').cpu().numpy(),
                          g['c1_req'])
    assert np.array_equal(U.conv2d_NCHWc_int8(dev(g['st_x']), dev(g['st_w']), stride=2, padding=3).cpu().numpy(),
                          g['st_out'])
    assert np.array_equal(U.dense_dotprod(dev(g['d_a']), dev(g['d_bp'])).cpu().numpy(), g['d_c'])
    # small-integer fp16 inputs: exact in fp32
    assert np.array_equal(U.conv2d_NCHW16c_OHWI16o(dev(g['f_x']), dev(g['f_w']), 1, 1).cpu().numpy(), g['f_out'])
    np.testing.assert_allclose(U.gemm_f16f32(dev(g['g_a']), dev(g['g_b'])).cpu().numpy(), g['g_c'],
                               rtol=RTOL, atol=ATOL)
    U.device_status()


def test_vnni_known_answer_through_the_gpu(U):
    """poc/vnni/poc.cc's vector as a 1x1 convolution: 16 lanes x 4-way dot."""
    import json, os
    with open(os.path.join(os.path.dirname(__file__), 'golden', 'poc_vnni_kat.json')) as f:
        want = json.load(f)['d']
    a = (np.arange(64) + 1).astype(np.uint8)
    b = (64 - np.arange(64)).astype(np.int8)
    # lane x uses a[4x..4x+3] and b[4x..4x+3]: 16 pixels with 16 channels (4 real), weights per lane
    for lane in range(16):
        x = np.zeros((1, 1, 1, 1, 16), np.uint8)
        x[0, 0, 0, 0, :4] = a[4 * lane:4 * lane + 4]
        w = np.zeros((1, 1, 1, 1, 4, 16, 4), np.int8)
        w[0, 0, 0, 0, 0, lane, :] = b[4 * lane:4 * lane + 4]
        got = U.conv2d_NCHWc_int8(dev(x), dev(w)).cpu().numpy().reshape(16)
        assert got[lane] == want[lane] and got.sum() == want[lane]


# ---------------------------------------------------------------------------
# int8 convolution
# ---------------------------------------------------------------------------
@pytest.mark.parametrize('n,ci,h,w,co,kh,kw,s,p', [
    (1, 16, 1, 1, 16, 1, 1, 1, 0),        # a single pixel, a single chunk
    (1, 16, 8, 8, 16, 3, 3, 1, 1),        # odd K-column count (9): zero-padded column
    (1, 64, 56, 56, 64, 3, 3, 1, 1),      # BASELINE config 1
    (2, 64, 14, 14, 128, 3, 3, 2, 1),
    (3, 32, 13, 11, 48, 3, 3, 1, 1),      # ragged: 429 pixels, tile straddles images, N tile of 48
    (1, 48, 9, 9, 320, 1, 1, 1, 0),       # two N tiles of 160
    (2, 16, 12, 9, 16, 1, 7, 1, 0),       # 1x7 and 7x1 kernels of the reference's shape corpus
    (2, 16, 12, 9, 16, 7, 1, 1, 3),
    (1, 80, 10, 10, 64, 5, 5, 2, 2),      # K columns not a multiple of any stage size
    (5, 256, 14, 14, 512, 1, 1, 1, 0),
    (2, 512, 7, 7, 2048, 1, 1, 2, 0),     # strided 1x1 projection
    (1, 2048, 7, 7, 512, 1, 1, 1, 0),     # deepest 1x1 reduction
    (1, 512, 7, 7, 512, 3, 3, 1, 1),      # deepest 3x3 reduction (4608)
    (1, 16, 40, 40, 16, 3, 3, 1, 0),      # valid convolution (no padding), as the reference calls it
    # tensors of 128 KB and more (tensor-copy fed), ragged in every direction
    (9, 32, 23, 21, 48, 3, 3, 1, 1),      # box copies: 21-pixel rows, tiles straddle images, N tile of 48
    (5, 48, 29, 31, 320, 3, 3, 1, 1),     # box copies, three chunks, two N tiles of 160
    (3, 64, 27, 33, 64, 5, 5, 1, 2),      # 5x5 taps, 25 x 4 = 100 K columns
    (7, 16, 37, 35, 16, 1, 7, 1, 0),      # 1x7 / 7x1 on box copies
    (7, 16, 37, 35, 16, 7, 1, 1, 3),
    (2, 16, 70, 150, 32, 3, 3, 1, 1),     # rows wider than a 128-row sub-tile
    (6, 32, 31, 29, 80, 3, 3, 2, 1),      # im2col copies, odd sizes
    (4, 48, 33, 35, 64, 5, 5, 3, 2),      # stride 3
    (3, 80, 30, 30, 64, 1, 1, 2, 0),      # strided 1x1 with five chunks
    # window form (stride 1, several taps, even chunk count, enough tiles): ragged widths and heights,
    # rectangular kernels, valid and padded, wide column blocks, tiles that end inside an image
    (10, 32, 61, 47, 48, 3, 3, 1, 1),
    (6, 64, 50, 90, 320, 3, 3, 1, 1),
    (16, 32, 40, 40, 32, 1, 3, 1, 0),
    (16, 32, 40, 40, 32, 3, 1, 1, 1),
    (20, 64, 33, 35, 64, 2, 2, 1, 0),
    (12, 32, 70, 110, 16, 3, 3, 1, 1),
    # pair form (stride 2 on an even width, several taps per kernel row): padded and valid, odd heights,
    # kernels of 2 to 7 taps per row (1 to 4 pair offsets), rectangular kernels, ragged boxes, two column blocks
    (6, 32, 56, 56, 48, 3, 3, 2, 1),
    (5, 48, 31, 30, 320, 3, 3, 2, 0),
    (4, 32, 41, 58, 32, 5, 5, 2, 2),
    (8, 16, 64, 64, 16, 2, 2, 2, 0),
    (3, 32, 50, 52, 32, 4, 4, 2, 1),
    (2, 16, 100, 100, 64, 7, 7, 2, 3),
    (9, 64, 23, 22, 80, 1, 3, 2, 0),
    (3, 16, 30, 300, 32, 3, 3, 2, 1),     # output rows wider than a 128-row sub-tile
])
def test_conv_int8_bit_exact(U, oracle, n, ci, h, w, co, kh, kw, s, p):
    rng = np.random.default_rng(hash((n, ci, h, w, co, kh, kw, s, p)) % 2 ** 32)
    if kh != kw:
        # the entry point takes one stride/pad per axis; rectangular kernels use (p, p) on both
        pass
    conv_case(U, oracle, rng, n, ci, h, w, co, kh, kw, s, p)


def test_conv_int8_extremes_and_signedness(U, oracle):
    """All-255 activations against all -128 / +127 weights: u8 x s8, no saturation before the clamp."""
    x = np.full((1, 32, 6, 6, 16), 255, np.uint8)
    for val in (-128, 127):
        w = np.full((2, 32, 3, 3, 4, 16, 4), val, np.int8)
        got = U.conv2d_NCHWc_int8(dev(x), dev(w), stride=1, padding=0).cpu().numpy()
        assert (got == 255 * val * 512 * 9).all()
    U.device_status()


def test_conv_int8_impulse(U):
    x = np.zeros((1, 32, 5, 6), np.uint8)
    w = np.zeros((32, 32, 3, 3), np.int8)
    x[0, 19, 2, 3] = 7
    w[21, 19, 0, 2] = -5
    got = U.conv2d_NCHWc_int8(dev(no.pack_nchw_to_nchwc(x)), dev(no.pack_oihw_to_int8_weights(w)), stride=1, padding=1)
    got = no.unpack_nchwc_to_nchw(got.cpu().numpy())
    assert np.argwhere(got).tolist() == [[0, 21, 3, 2]] and got[0, 21, 3, 2] == -35


def test_requant_rounding_and_bias_only_s32(U, oracle):
    rng = np.random.default_rng(2)
    x = rng.integers(0, 256, (1, 1, 4, 4, 16), dtype=np.uint8)
    w = rng.integers(-128, 128, (1, 1, 1, 1, 4, 16, 4), dtype=np.int8)
    b = np.array([-1, 126, 127, 128, 383, 384, 65151, 65152, 10 ** 6, -10 ** 6, -129, -128, 0, 255, 256, 2 ** 31 - 1],
                 np.int32)
    for shift in (1, 8, 15, 31):
        got = U.conv2d_NCHWc_int8(dev(x), dev(w), bias=dev(b), requant_shift=shift).cpu().numpy()
        assert np.array_equal(got, oracle.conv2d_u8s8(x, w, bias=b, requant_shift=shift))
    got = U.conv2d_NCHWc_int8(dev(x), dev(w), bias=dev(b)).cpu().numpy()  # s32 + bias, wrapping like the oracle
    assert np.array_equal(got, oracle.conv2d_u8s8(x, w, bias=b))
    U.device_status()


def test_bias_through_the_tensor_core_and_through_the_drain(U, oracle):
    """Biases small enough enter the accumulator as one more K step of the MMA; larger ones are
    added by the drain.  Both edges of the first range, every digit pattern, and mixed blocks."""
    rng = np.random.default_rng(77)
    x = rng.integers(0, 256, (2, 3, 9, 9, 16), dtype=np.uint8)
    w = rng.integers(-128, 128, (20, 3, 3, 3, 4, 16, 4), dtype=np.int8)   # 320 channels: two column blocks
    lo, hi = -245760, 243967                                             # range of bias + rounding constant
    cases = {
        'edges_shift8': (8, np.resize(np.array([lo - 128, hi - 128, 0, -1, 1, -128, 127, lo - 127, hi - 129], np.int64), 320)),
        'all_digits': (8, np.arange(320, dtype=np.int64) * 1531 - 244000),
        'just_outside': (8, np.resize(np.array([hi - 127, 5, lo - 129, 7], np.int64), 320)),
        'second_block_outside': (8, np.concatenate([rng.integers(-2 ** 15, 2 ** 15, 160), rng.integers(-2 ** 24, 2 ** 24, 160)])),
        'shift1': (1, rng.integers(-2 ** 15, 2 ** 15, 320)),
        'shift18': (18, rng.integers(-2 ** 16, 2 ** 16, 320)),
        'shift19_rounding_too_large': (19, rng.integers(-2 ** 12, 2 ** 12, 320)),
        'huge': (8, rng.integers(-2 ** 31, 2 ** 31, 320)),
    }
    for name, (shift, b) in cases.items():
        b = np.asarray(b, np.int64).astype(np.int32)
        got = U.conv2d_NCHWc_int8(dev(x), dev(w), padding=1, bias=dev(b), requant_shift=shift).cpu().numpy()
        gots = U.conv2d_NCHWc_int8(dev(x), dev(w), padding=1, bias=dev(b)).cpu().numpy()
        U.device_status()
        assert np.array_equal(got, oracle.conv2d_u8s8(x, w, (1, 1), (1, 1), bias=b, requant_shift=shift)), name
        assert np.array_equal(gots, oracle.conv2d_u8s8(x, w, (1, 1), (1, 1), bias=b)), name
    # requantisation without a bias: only the rounding constant goes in
    got = U.conv2d_NCHWc_int8(dev(x), dev(w), padding=1, out_dtype='uint8').cpu().numpy()
    assert np.array_equal(got, oracle.conv2d_u8s8(x, w, (1, 1), (1, 1), requant_shift=8))


def test_wide_layer_bias_beyond_staged_vector(U, oracle):
    """More output channels than the kernel keeps in shared memory (2048), with ordinary and extreme biases."""
    rng = np.random.default_rng(21)
    x = rng.integers(0, 256, (1, 2, 5, 5, 16), dtype=np.uint8)
    w = rng.integers(-128, 128, (136, 2, 1, 1, 4, 16, 4), dtype=np.int8)   # 2176 output channels
    for hi in (2 ** 15, 2 ** 31 - 1):
        b = rng.integers(-hi, hi, 2176, dtype=np.int64).astype(np.int32)
        got = U.conv2d_NCHWc_int8(dev(x), dev(w), bias=dev(b), out_dtype='uint8')
        gots = U.conv2d_NCHWc_int8(dev(x), dev(w), bias=dev(b))
        U.device_status()
        assert np.array_equal(got.cpu().numpy(), oracle.conv2d_u8s8(x, w, bias=b, requant_shift=8))
        assert np.array_equal(gots.cpu().numpy(), oracle.conv2d_u8s8(x, w, bias=b))


@pytest.mark.parametrize('hw,k,p', [(64, 7, 3), (33, 7, 3), (62, 3, 1), (60, 5, 2), (18, 7, 0), (20, 4, 1), (66, 6, 2)])
def test_stem_stride2_geometries(U, oracle, hw, k, p):
    """Stride-2 NCHW4c convolutions: even images take the folded (scratch) path, odd ones the in-place gather."""
    rng = np.random.default_rng(hw * 100 + k)
    # nine images: the folded image (tensor-copy fed) is then 128 KB or more for the larger sizes; the
    # smaller ones run the in-place gather, which is checked against the same oracle
    x = rng.integers(0, 256, (9 if hw >= 26 else 3, 1, hw, hw + 2 * (hw % 2 == 0), 4), dtype=np.uint8)
    w = rng.integers(-128, 128, (2, 1, k, k, 1, 16, 4), dtype=np.int8)
    b = rng.integers(-2 ** 15, 2 ** 15, 32, dtype=np.int32)
    got = U.conv2d_NCHWc_int8(dev(x), dev(w), stride=2, padding=p)
    gotq = U.conv2d_NCHWc_int8(dev(x), dev(w), stride=2, padding=p, bias=dev(b), out_dtype='uint8')
    U.device_status()
    assert np.array_equal(got.cpu().numpy(), oracle.conv2d_u8s8(x, w, (2, 2), (p, p)))
    assert np.array_equal(gotq.cpu().numpy(), oracle.conv2d_u8s8(x, w, (2, 2), (p, p), bias=b, requant_shift=8))


@pytest.mark.parametrize('h,w,k,p', [(12, 224, 7, 3), (10, 250, 7, 3), (14, 132, 3, 1), (8, 200, 4, 1), (6, 248, 8, 3)])
def test_stem_wide_rows_one_copy_per_kernel_row(U, oracle, h, w, k, p):
    """Folded stride-2 convolutions whose output rows fill a 128-row sub-tile on their own: the taps
    of a kernel row are fetched with one copy and addressed as shifted windows."""
    rng = np.random.default_rng(h * 1000 + w + k)
    n = -(-131072 // (h * w * 4))   # enough images for the folded tensor to reach 128 KB (tensor-copy fed)
    x = rng.integers(0, 256, (n, 1, h, w, 4), dtype=np.uint8)
    wt = rng.integers(-128, 128, (4, 1, k, k, 1, 16, 4), dtype=np.int8)
    b = rng.integers(-2 ** 15, 2 ** 15, 64, dtype=np.int32)
    got = U.conv2d_NCHWc_int8(dev(x), dev(wt), stride=2, padding=p)
    gotq = U.conv2d_NCHWc_int8(dev(x), dev(wt), stride=2, padding=p, bias=dev(b), out_dtype='uint8')
    U.device_status()
    assert np.array_equal(got.cpu().numpy(), oracle.conv2d_u8s8(x, wt, (2, 2), (p, p)))
    assert np.array_equal(gotq.cpu().numpy(), oracle.conv2d_u8s8(x, wt, (2, 2), (p, p), bias=b, requant_shift=8))


def test_stem_without_workspace_through_the_c_abi(U, oracle):
    """The same stem with d_workspace = NULL: the library falls back to the in-place gather."""
    import ctypes
    from unit_b200 import _lib
    L = _lib.lib()
    rng = np.random.default_rng(77)
    x = rng.integers(0, 256, (2, 1, 32, 32, 4), dtype=np.uint8)
    w = rng.integers(-128, 128, (4, 1, 7, 7, 1, 16, 4), dtype=np.int8)
    xd, wd = dev(x), dev(w)
    pw = U.pack_conv_weights_int8(wd, 2, 3)
    d = _lib.ConvDesc(2, 4, 32, 32, 4, 64, 7, 7, 2, 2, 3, 3)
    assert L.unit_conv2d_workspace_bytes(ctypes.byref(d)) == 2 * 16 * 16 * 16
    out = torch.empty((2, 4, 16, 16, 16), dtype=torch.int32, device='cuda')
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = L.unit_conv2d_u8s8s32_nchwc(ctypes.byref(d), ctypes.c_void_p(xd.data_ptr()), ctypes.c_void_p(pw.buf.data_ptr()),
                                     None, ctypes.c_void_p(out.data_ptr()), None, 0, stream)
    assert rc == 0
    U.device_status()
    assert np.array_equal(out.cpu().numpy(), oracle.conv2d_u8s8(x, w, (2, 2), (3, 3)))


def test_stem_nchw4c(U, oracle):
    rng = np.random.default_rng(4)
    for (n, hw) in ((2, 32), (1, 224)):
        x = rng.integers(0, 256, (n, 1, hw, hw, 4), dtype=np.uint8)
        x[..., 3] = 0
        w = rng.integers(-128, 128, (4, 1, 7, 7, 1, 16, 4), dtype=np.int8)
        b = rng.integers(-2 ** 15, 2 ** 15, 64, dtype=np.int32)
        got = U.conv2d_NCHWc_int8(dev(x), dev(w), stride=2, padding=3, bias=dev(b), out_dtype='uint8')
        U.device_status()
        ref = oracle.conv2d_u8s8(x, w, (2, 2), (3, 3), bias=b, requant_shift=8, vnni=oracle.host_has_vnni())
        assert np.array_equal(got.cpu().numpy(), ref)
    # two NCHW4c chunks (8 stored channels), 3x3
    x = rng.integers(0, 256, (2, 2, 9, 9, 4), dtype=np.uint8)
    w = rng.integers(-128, 128, (2, 2, 3, 3, 1, 16, 4), dtype=np.int8)
    got = U.conv2d_NCHWc_int8(dev(x), dev(w), stride=1, padding=1)
    assert np.array_equal(got.cpu().numpy(), oracle.conv2d_u8s8(x, w, (1, 1), (1, 1)))


@pytest.mark.parametrize('batch', [1, 16])
def test_resnet50_sweep_config3(U, oracle, batch):
    """BASELINE config 3: every ResNet-50 conv shape, batch 1 and 16, fused bias + requant, bit-exact."""
    from unit_b200 import resnet50 as R
    vnni = oracle.host_has_vnni()
    if batch > 1 and not vnni:
        pytest.skip('the batch-16 sweep needs the AVX-512 VNNI oracle (the scalar oracle would take minutes)')
    for li, l in enumerate(R.LAYERS):
        x, w, b = R.make_layer_inputs(l, li, batch, config=3)
        got = U.conv2d_NCHWc_int8(dev(x), dev(w), stride=l.stride, padding=l.pad, bias=dev(b), out_dtype='uint8')
        U.device_status()
        ref = oracle.conv2d_u8s8(x, w, (l.stride, l.stride), (l.pad, l.pad), bias=b, requant_shift=8, vnni=vnni)
        assert np.array_equal(got.cpu().numpy(), ref), l.name


# ---------------------------------------------------------------------------
# int8 dense
# ---------------------------------------------------------------------------
@pytest.mark.parametrize('m,n,k,t', [
    (1, 16, 16, 16), (128, 3072, 768, 128), (100, 128, 128, 128), (300, 512, 1024, 128), (129, 48, 80, 16),
    (1024, 1024, 1024, 16),
    # swizzled A rows (K a multiple of 128 bytes) with ragged M and N, and K just off that grid (column copies)
    (257, 272, 384, 16), (5, 16, 128, 16), (700, 528, 2048, 16), (130, 64, 144, 16),
])
def test_dense_int8_bit_exact(U, oracle, m, n, k, t):
    rng = np.random.default_rng(m * 7 + n + k)
    a = rng.integers(0, 256, (m, k), dtype=np.uint8)
    b = rng.integers(-128, 128, (n, k), dtype=np.int8)
    bp = no.pack_dense_weights(b, t)
    got = U.dense_dotprod(dev(a), dev(bp))
    U.device_status()
    ref = oracle.dense_u8s8s32(a, bp, vnni=oracle.host_has_vnni())
    assert np.array_equal(got.cpu().numpy(), ref)


def test_dense_4096_config2(U, oracle):
    """BASELINE config 2: M = N = K = 4096, bit-exact."""
    rng = np.random.default_rng(2)
    a = rng.integers(0, 256, (4096, 4096), dtype=np.uint8)
    b = rng.integers(-128, 128, (4096, 4096), dtype=np.int8)
    bp = no.pack_dense_weights(b, 128)
    got = U.dense_dotprod(dev(a), dev(bp))
    U.device_status()
    if oracle.host_has_vnni():
        assert np.array_equal(got.cpu().numpy(), oracle.dense_u8s8s32(a, bp, vnni=True))
    else:  # scalar oracle on a row sample
        rows = rng.choice(4096, 64, replace=False)
        assert np.array_equal(got.cpu().numpy()[rows], oracle.dense_u8s8s32(a[rows], bp))
    # size-independent property: linearity in A over the integers (A1 + A2 with no u8 overflow)
    a1 = (a // 2).astype(np.uint8)
    a2 = (a - a1).astype(np.uint8)
    pw = U.pack_dense_weights_int8(dev(bp))
    s = U.dense_dotprod(dev(a1), pw) + U.dense_dotprod(dev(a2), pw)
    assert torch.equal(s, got)


# ---------------------------------------------------------------------------
# fp16 path
# ---------------------------------------------------------------------------
@pytest.mark.parametrize('n,ci,h,w,co,k,s,p', [
    (1, 16, 6, 6, 16, 3, 1, 0), (2, 32, 10, 10, 32, 3, 1, 1), (3, 64, 14, 14, 128, 3, 2, 1), (2, 256, 14, 14, 256, 1, 1, 0),
    (1, 1024, 14, 14, 256, 1, 1, 0), (4, 256, 14, 14, 256, 3, 1, 1),
    # strided convolutions on tensors of 128 KB and more: the im2col tensor copies
    # (the reference's strided form: python/tensorizer/ops/gpu.py:47-53)
    (8, 256, 28, 28, 256, 3, 2, 1), (8, 256, 28, 28, 512, 1, 2, 0), (5, 48, 31, 29, 80, 3, 2, 1), (3, 32, 33, 35, 32, 5, 3, 2),
    (9, 32, 23, 21, 48, 3, 1, 1),     # ragged box copies
])
def test_conv_fp16(U, oracle, n, ci, h, w, co, k, s, p):
    rng = np.random.default_rng(n + ci + co + k)
    x = rng.standard_normal((n, ci // 16, h, w, 16)).astype(np.float16)
    wt = (rng.standard_normal((co // 16, ci // 16, k, k, 16, 16)) * 0.05).astype(np.float16)
    got = U.conv2d_NCHW16c_OHWI16o(dev(x), dev(wt), s, s, padding=p)
    U.device_status()
    np.testing.assert_allclose(got.cpu().numpy(), oracle.conv2d_f16f32(x, wt, (s, s), (p, p)), rtol=RTOL, atol=ATOL)


def test_conv_fp16_config4_batch256(U, oracle):
    """BASELINE config 4: N=256, 256->256, 14x14, 3x3 pad 1.  The oracle checks a sample of images;
    the whole batch is checked through batch independence (each image equals its batch-8 result)."""
    rng = np.random.default_rng(44)
    x = rng.standard_normal((256, 16, 14, 14, 16)).astype(np.float16)
    wt = (rng.standard_normal((16, 16, 3, 3, 16, 16)) * 0.05).astype(np.float16)
    xd = dev(x)
    pw = U.pack_conv_weights_f16(dev(wt))
    got = U.conv2d_NCHW16c_OHWI16o(xd, pw, 1, 1, padding=1)
    U.device_status()
    sample = [0, 1, 127, 255]
    ref = oracle.conv2d_f16f32(x[sample], wt, (1, 1), (1, 1))
    np.testing.assert_allclose(got[sample].cpu().numpy(), ref, rtol=RTOL, atol=ATOL)
    for s0 in range(0, 256, 64):
        part = U.conv2d_NCHW16c_OHWI16o(xd[s0:s0 + 64], pw, 1, 1, padding=1)
        torch.testing.assert_close(part, got[s0:s0 + 64], rtol=RTOL, atol=ATOL)


def test_conv_fp16_accepts_nchw_and_oihw_like_the_reference(U, oracle):
    rng = np.random.default_rng(8)
    x = rng.standard_normal((2, 32, 9, 9)).astype(np.float16)
    w = (rng.standard_normal((48, 32, 3, 3)) * 0.05).astype(np.float16)
    got = U.conv2d_NCHW16c_OHWI16o(dev(x), dev(w), 1, 1)
    ref = oracle.conv2d_f16f32(no.pack_nchw_to_nchwc(x), no.pack_oihw_to_f16_weights(w))
    assert tuple(got.shape) == (2, 3, 7, 7, 16)
    np.testing.assert_allclose(got.cpu().numpy(), ref, rtol=RTOL, atol=ATOL)
    from unit_b200.ops import _Attrs
    out = U.conv2d_NCHW16c_OHWI16o_compute(_Attrs(strides=(1, 1)), [dev(x), dev(w)], 'float32')
    assert isinstance(out, list) and torch.equal(out[0], got)


@pytest.mark.parametrize('m,n,k', [(128, 768, 3072), (64, 192, 1024), (1, 16, 8), (130, 48, 72), (300, 272, 192), (70, 64, 64)])
def test_gemm_fp16(U, oracle, m, n, k):
    rng = np.random.default_rng(m + n + k)
    a = rng.standard_normal((m, k)).astype(np.float16)
    b = (rng.standard_normal((k, n)) * 0.05).astype(np.float16)
    got = U.gemm_f16f32(dev(a), dev(b))
    U.device_status()
    np.testing.assert_allclose(got.cpu().numpy(), no.gemm_f32(a, b), rtol=RTOL, atol=ATOL)


# ---------------------------------------------------------------------------
# layout kernels, host buffers, batch split, errors
# ---------------------------------------------------------------------------
def test_layout_kernels_match_numpy(U):
    rng = np.random.default_rng(6)
    x = rng.integers(0, 256, (3, 19, 5, 7), dtype=np.uint8)
    for cb in (4, 16):
        y = U.pack_data_nchwc(dev(x), cb)
        assert np.array_equal(y.cpu().numpy(), no.pack_nchw_to_nchwc(x, cb))
        assert np.array_equal(U.unpack_data_nchwc(y, 19).cpu().numpy(), x)
    # shapes whose rows are whole 4-byte words take the vectorised kernels (register transpose,
    # 16-byte stores); channel counts that do not fill the last block, every element size
    for shape, dt in (((3, 19, 6, 8), np.uint8), ((2, 37, 12, 12), np.uint8), ((2, 35, 5, 6), np.float16),
                      ((2, 21, 3, 5), np.int32), ((4, 3, 16, 16), np.uint8)):
        xv = rng.integers(0, 200, shape).astype(dt)
        for cb in (4, 16):
            yv = U.pack_data_nchwc(dev(xv), cb)
            assert np.array_equal(yv.cpu().numpy(), no.pack_nchw_to_nchwc(xv, cb)), (shape, dt, cb)
            assert np.array_equal(U.unpack_data_nchwc(yv, shape[1]).cpu().numpy(), xv), (shape, dt, cb)
    with pytest.raises(ValueError):      # fewer channels than the stored blocks could hold one block less of
        U.unpack_data_nchwc(U.pack_data_nchwc(dev(x), 4), 3)
    xf = rng.standard_normal((2, 32, 4, 4)).astype(np.float16)
    assert np.array_equal(U.pack_data_nchwc(dev(xf)).cpu().numpy(), no.pack_nchw_to_nchwc(xf))
    xi = rng.integers(-2 ** 31, 2 ** 31 - 1, (2, 16, 3, 3), dtype=np.int32)
    assert np.array_equal(U.unpack_data_nchwc(U.pack_data_nchwc(dev(xi))).cpu().numpy(), xi)
    w = rng.integers(-128, 128, (40, 19, 3, 2), dtype=np.int8)
    assert np.array_equal(U.pack_weights_oihw_int8(dev(w)).cpu().numpy(), no.pack_oihw_to_int8_weights(w))
    assert np.array_equal(U.pack_weights_oihw_int8(dev(w[:, :3]), 4).cpu().numpy(), no.pack_oihw_to_int8_weights(w[:, :3], 4))
    wf = rng.standard_normal((40, 19, 3, 2)).astype(np.float16)
    assert np.array_equal(U.pack_weights_oihw_f16(dev(wf)).cpu().numpy(), no.pack_oihw_to_f16_weights(wf))
    U.device_status()


def test_host_tensors_in_host_tensor_out(U, oracle):
    rng = np.random.default_rng(12)
    x = rng.integers(0, 256, (2, 4, 14, 14, 16), dtype=np.uint8)
    w = rng.integers(-128, 128, (4, 4, 3, 3, 4, 16, 4), dtype=np.int8)
    got = U.conv2d_NCHWc_int8(torch.from_numpy(x), torch.from_numpy(w), stride=1, padding=1)
    assert not got.is_cuda
    assert np.array_equal(got.numpy(), oracle.conv2d_u8s8(x, w, (1, 1), (1, 1)))


def test_operator_reuses_its_prepared_launch_on_the_same_buffers(U, oracle):
    """Calls that name their output buffer keep their prepared launch (unit_b200.ops._PLAN_CACHE): a repeated
    call must read the buffers' current contents, and other buffers, epilogues or shapes get launches of their own."""
    from unit_b200 import ops
    rng = np.random.default_rng(31)
    x = rng.integers(0, 256, (2, 4, 20, 20, 16), dtype=np.uint8)
    w = rng.integers(-128, 128, (4, 4, 3, 3, 4, 16, 4), dtype=np.int8)
    b = rng.integers(-2 ** 12, 2 ** 12, 64, dtype=np.int32)
    xd, bd = dev(x), dev(b)
    pw = U.pack_conv_weights_int8(dev(w), 1, 1)
    o1 = torch.empty((2, 4, 20, 20, 16), dtype=torch.int32, device='cuda')
    o2 = torch.empty_like(o1)
    o8 = torch.empty((2, 4, 20, 20, 16), dtype=torch.uint8, device='cuda')
    n0 = len(ops._PLAN_CACHE)
    for _ in range(3):
        assert U.conv2d_NCHWc_int8(xd, pw, padding=1, out=o1) is o1
    assert len(ops._PLAN_CACHE) == n0 + 1
    assert np.array_equal(o1.cpu().numpy(), oracle.conv2d_u8s8(x, w, (1, 1), (1, 1)))
    x2 = rng.integers(0, 256, x.shape, dtype=np.uint8)
    xd.copy_(dev(x2))                                   # same buffer, new contents
    U.conv2d_NCHWc_int8(xd, pw, padding=1, out=o1)
    assert len(ops._PLAN_CACHE) == n0 + 1
    assert np.array_equal(o1.cpu().numpy(), oracle.conv2d_u8s8(x2, w, (1, 1), (1, 1)))
    U.conv2d_NCHWc_int8(xd, pw, padding=1, out=o2)      # another output buffer
    U.conv2d_NCHWc_int8(xd, pw, padding=1, bias=bd, out_dtype='uint8', out=o8)   # another epilogue
    assert len(ops._PLAN_CACHE) == n0 + 3
    assert np.array_equal(o2.cpu().numpy(), o1.cpu().numpy())
    assert np.array_equal(o8.cpu().numpy(), oracle.conv2d_i8_ex(x2, w, (1, 1), (1, 1), bias=b, requant_shift=8))
    with pytest.raises(ValueError):                       # a wrong output shape is still refused
        U.conv2d_NCHWc_int8(xd, pw, padding=1, out=torch.empty((2, 4, 19, 20, 16), dtype=torch.int32, device='cuda'))
    U.device_status()


def test_batch_split_equals_whole_batch(U):
    """The multi-GPU partition: concatenating per-slice results equals the whole-batch result."""
    from unit_b200 import resnet50 as R
    from unit_b200.sharding import shard
    l = R.LAYERS[9]
    x, w, b = R.make_layer_inputs(l, 9, 24, config=5)
    xd, bd = dev(x), dev(b)
    pw = U.pack_conv_weights_int8(dev(w), l.stride, l.pad)
    whole = U.conv2d_NCHWc_int8(xd, pw, stride=l.stride, padding=l.pad, bias=bd, out_dtype='uint8')
    for world in (2, 8):
        parts = [U.conv2d_NCHWc_int8(shard(xd, r, world), pw, stride=l.stride, padding=l.pad, bias=bd, out_dtype='uint8')
                 for r in range(world)]
        assert torch.equal(torch.cat(parts), whole)
    U.device_status()


def test_large_batch_property_config5(U, oracle):
    """Full-size check (batch 256): a sample of images against the oracle, the rest by slice equality."""
    from unit_b200 import resnet50 as R
    for li in (3, 15):  # 3x3 64->64 @56 and 3x3 256->256 @14
        l = R.LAYERS[li]
        x, w, b = R.make_layer_inputs(l, li, 256, config=5)
        xd, bd = dev(x), dev(b)
        pw = U.pack_conv_weights_int8(dev(w), l.stride, l.pad)
        got = U.conv2d_NCHWc_int8(xd, pw, stride=l.stride, padding=l.pad, bias=bd, out_dtype='uint8')
        U.device_status()
        sample = [0, 100, 255]
        ref = oracle.conv2d_u8s8(x[sample], w, (l.stride, l.stride), (l.pad, l.pad), bias=b, requant_shift=8,
                                 vnni=oracle.host_has_vnni())
        assert np.array_equal(got[sample].cpu().numpy(), ref)
        for s0 in range(0, 256, 32):
            part = U.conv2d_NCHWc_int8(xd[s0:s0 + 32], pw, stride=l.stride, padding=l.pad, bias=bd, out_dtype='uint8')
            assert torch.equal(part, got[s0:s0 + 32])


def test_dependent_convolutions_back_to_back(U, oracle):
    """Each convolution's prologue may overlap the previous kernel's tail (programmatic dependent
    launch); a chain in which every layer reads the previous layer's output, launched without any
    host synchronisation in between, must still equal the oracle's chain."""
    rng = np.random.default_rng(4242)
    x = rng.integers(0, 256, (4, 4, 28, 28, 16), dtype=np.uint8)
    ws = [rng.integers(-8, 9, (4, 4, k, k, 4, 16, 4), dtype=np.int8) for k in (1, 3, 1, 3)]
    bs = [rng.integers(-2 ** 10, 2 ** 10, 64, dtype=np.int32) for _ in ws]
    ref = x
    for w, b in zip(ws, bs):
        k = w.shape[2]
        ref = oracle.conv2d_u8s8(ref, w, (1, 1), (k // 2, k // 2), bias=b, requant_shift=8)
    xd = dev(x)
    pws = [U.pack_conv_weights_int8(dev(w), 1, w.shape[2] // 2) for w in ws]
    bds = [dev(b) for b in bs]
    for rep in range(10):
        cur = xd
        for w, pw, bd in zip(ws, pws, bds):
            cur = U.conv2d_NCHWc_int8(cur, pw, stride=1, padding=w.shape[2] // 2, bias=bd, out_dtype='uint8')
        assert np.array_equal(cur.cpu().numpy(), ref), f'repetition {rep}'
    U.device_status()


def test_error_behaviour(U):
    x = torch.zeros((1, 4, 8, 8, 16), dtype=torch.uint8, device='cuda')
    w = torch.zeros((4, 4, 3, 3, 4, 16, 4), dtype=torch.int8, device='cuda')
    with pytest.raises(TypeError):
        U.conv2d_NCHWc_int8(x.to(torch.int32), w)                # (s8 data is accepted: signed activations)
    with pytest.raises(ValueError):
        U.conv2d_NCHWc_int8(x[:, :2], w)                       # channel mismatch
    with pytest.raises(ValueError):
        U.conv2d_NCHWc_int8(x, w, dilation=2)
    with pytest.raises(ValueError):
        U.conv2d_NCHWc_int8(x[:, :, :2, :2], w)                # kernel larger than input
    with pytest.raises(ValueError):
        U.conv2d_NCHWc_int8(x, w, out=torch.empty((1,), dtype=torch.int32, device='cuda'))
    with pytest.raises(ValueError):
        U.dense_dotprod(torch.zeros((4, 32), dtype=torch.uint8, device='cuda'),
                        torch.zeros((1, 16, 16, 4), dtype=torch.int8, device='cuda'))   # K mismatch
    empty = U.dense_dotprod(torch.zeros((0, 64), dtype=torch.uint8, device='cuda'),
                            torch.zeros((1, 16, 16, 4), dtype=torch.int8, device='cuda'))
    assert tuple(empty.shape) == (0, 16)
    assert tuple(U.conv2d_NCHWc_int8(x[:0], w, padding=1).shape) == (0, 4, 8, 8, 16)   # empty batch
    U.device_status()
    assert U.launch_count() > 0
