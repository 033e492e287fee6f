"""Every compiled variant of the contraction kernel is reached and checked against the oracle.

The library compiles one kernel per (operand path, epilogue, data type, sub-tiles per tile) and
picks one from the problem's geometry alone (no environment switch).  ``unit_variant_name`` lists
the compiled variants and ``unit_variant_launches`` counts launches; the cases below are chosen
from the selection rules so that each variant runs at least once, each result is compared with
the oracle (bit-exact for int8, rel 1e-2 / abs 1e-3 for fp16), and the last test fails if a
compiled variant was never launched.  Also here: the bounded-wait error path
(UNIT_ERR_DEVICE_WAIT), made to fire by the library's diagnostics hook without faulting the GPU.
"""
import ctypes
import zlib

import numpy as np
import pytest
import torch

from oracle import np_oracle as no

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-2, 1e-3


@pytest.fixture(scope='module')
def U():
    assert torch.cuda.is_available(), 'GPU tests need a CUDA device'
    import unit_b200
    from unit_b200 import _lib
    _lib.lib()
    return unit_b200


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def variant_counts():
    from unit_b200 import _lib
    L = _lib.lib()
    out = {}
    for i in range(L.unit_variant_count()):
        name = L.unit_variant_name(i)
        if name:
            out[name.decode()] = int(L.unit_variant_launches(i))
    return out


# (operand path, sub-tiles) -> geometry (n, c_in, h, w, c_out, k, stride, pad, c_block).  The selection
# rules: stride 1 on tensors >= 128 KB -> whole-row box copies; stride 2 with several taps per kernel row on an
# even width -> box copies of pixel pairs; other strides -> im2col copies; tensors
# below 128 KB, or strides the im2col descriptor cannot express (> 8) -> cp.async gather; NCHW4c
# images of odd size -> the 4-byte gather; two sub-tiles per tile once 2 x tiles >= SMs.
INT8_CASES = {
    'box_mt1': (9, 32, 23, 21, 48, 3, 1, 1, 16),
    'box_mt2': (8, 16, 56, 56, 16, 3, 1, 1, 16),
    'im2col_mt1': (4, 32, 41, 41, 32, 3, 2, 1, 16),
    'im2col_mt2': (8, 16, 113, 113, 16, 3, 2, 1, 16),
    'gather_mt1': (2, 32, 13, 11, 32, 3, 2, 1, 16),
    'gather_mt2': (32, 16, 225, 225, 16, 1, 9, 0, 16),
    'stem_gather_mt1': (2, 4, 33, 35, 32, 7, 2, 3, 4),
    'stem_gather_mt2': (8, 4, 227, 227, 16, 3, 2, 1, 4),
    # stride 1, 3x3, even chunk count, wide images, enough tiles: the window form (rows copied once per chunk,
    # every tap a shifted window); one and two sub-tiles per tile
    'win_mt1': (8, 32, 56, 56, 32, 3, 1, 1, 16),
    'win_mt2': (24, 32, 56, 56, 16, 3, 1, 1, 16),
    # few tiles and a long reduction: split-K over a thread-block cluster
    'box_splitk': (1, 256, 24, 24, 256, 3, 1, 1, 16),
    'im2col_splitk': (1, 256, 25, 25, 256, 3, 2, 1, 16),
    # stride 2 on an even width, 3x3: the pair form (dense rows of pixel pairs through the box-copy kernel)
    'pair_mt1': (4, 32, 40, 40, 32, 3, 2, 1, 16),
    'pair_mt2': (8, 16, 112, 112, 16, 3, 2, 1, 16),
    'pair_splitk': (1, 256, 24, 24, 256, 3, 2, 1, 16),
    # a tensor below 128 KB with a long reduction and few tiles (a deep layer at batch 1): the gather, split over K
    'gather_splitk': (1, 512, 7, 7, 512, 3, 1, 1, 16),
}
INT8_VARIANTS = {
    'box_mt1': 'A_CONV_BOX, {}, i8, MT=1', 'box_mt2': 'A_CONV_BOX, {}, i8, MT=2',
    'im2col_mt1': 'A_CONV_TMA, {}, i8, MT=1', 'im2col_mt2': 'A_CONV_TMA, {}, i8, MT=2',
    'gather_mt1': 'A_CONV_I8, {}, i8, MT=1', 'gather_mt2': 'A_CONV_I8, {}, i8, MT=2',
    'stem_gather_mt1': 'A_STEM_I8, {}, i8, MT=1', 'stem_gather_mt2': 'A_STEM_I8, {}, i8, MT=2',
    'win_mt1': 'A_CONV_WIN, {}, i8, MT=1', 'win_mt2': 'A_CONV_WIN, {}, i8, MT=2',
    'box_splitk': 'A_CONV_BOX, {}, i8, MT=1, split-K', 'im2col_splitk': 'A_CONV_TMA, {}, i8, MT=1, split-K',
    'pair_mt1': 'A_CONV_BOX, {}, i8, MT=1', 'pair_mt2': 'A_CONV_BOX, {}, i8, MT=2', 'pair_splitk': 'A_CONV_BOX, {}, i8, MT=1, split-K',
    'gather_splitk': 'A_CONV_I8, {}, i8, MT=1, split-K',
}


@pytest.mark.parametrize('case', sorted(INT8_CASES))
def test_int8_conv_variants_all_epilogues(U, oracle, case):
    n, ci, h, w, co, k, s, p, cb = INT8_CASES[case]
    rng = np.random.default_rng(zlib.crc32(case.encode()))
    x = rng.integers(0, 256, (n, ci // cb, h, w, cb), dtype=np.uint8)
    wt = rng.integers(-128, 128, (co // 16, ci // cb, k, k, cb // 4, 16, 4), dtype=np.int8)
    b = rng.integers(-2 ** 15, 2 ** 15, co, dtype=np.int32)
    oh, ow = (h + 2 * p - k) // s + 1, (w + 2 * p - k) // s + 1
    res = rng.integers(0, 256, (n, co // 16, oh, ow, 16), dtype=np.uint8)
    before = variant_counts()
    xd, wd, bd = dev(x), dev(wt), dev(b)
    got_raw = U.conv2d_NCHWc_int8(xd, wd, stride=s, padding=p, bias=bd)
    got_req = U.conv2d_NCHWc_int8(xd, wd, stride=s, padding=p, bias=bd, out_dtype='uint8')
    got_mul = U.conv2d_NCHWc_int8(xd, wd, stride=s, padding=p, bias=bd, mul=11)
    got_res = U.conv2d_NCHWc_int8(xd, wd, stride=s, padding=p, bias=bd, requant_shift=9, residual=dev(res))
    U.device_status()
    st, pd = (s, s), (p, p)
    assert np.array_equal(got_raw.cpu().numpy(), oracle.conv2d_i8_ex(x, wt, st, pd, bias=b)), case
    assert np.array_equal(got_req.cpu().numpy(), oracle.conv2d_i8_ex(x, wt, st, pd, bias=b, requant_shift=8)), case
    assert np.array_equal(got_mul.cpu().numpy(), oracle.conv2d_i8_ex(x, wt, st, pd, bias=b, mul=11)), case
    assert np.array_equal(got_res.cpu().numpy(),
                          oracle.conv2d_i8_ex(x, wt, st, pd, bias=b, requant_shift=9, residual=res)), case
    after = variant_counts()
    for epi in ('EPI_RAW_NCHWC', 'EPI_REQ_NCHWC', 'EPI_MUL_NCHWC', 'EPI_RES_NCHWC'):
        name = 'igemm_kernel<' + INT8_VARIANTS[case].format(epi) + '>'
        assert after[name] > before[name], f'{case}: expected {name} to run; counters moved: ' + \
            str({k_: after[k_] - before[k_] for k_ in after if after[k_] != before[k_]})


FP16_CASES = {
    'box_mt1': ((9, 16, 33, 29, 48, 3, 1, 1), 'A_CONV_BOX, EPI_RAW_NCHWC, f16, MT=1'),
    'box_mt2': ((8, 16, 56, 56, 16, 3, 1, 1), 'A_CONV_BOX, EPI_RAW_NCHWC, f16, MT=2'),
    'im2col_mt1': ((4, 32, 40, 40, 32, 3, 2, 1), 'A_CONV_TMA, EPI_RAW_NCHWC, f16, MT=1'),
    'im2col_mt2': ((8, 16, 112, 112, 16, 3, 2, 1), 'A_CONV_TMA, EPI_RAW_NCHWC, f16, MT=2'),
    'gather_mt1': ((2, 32, 13, 11, 32, 3, 2, 1), 'A_CONV_F16, EPI_RAW_NCHWC, f16, MT=1'),
    'gather_mt2': ((32, 16, 225, 225, 16, 1, 9, 0), 'A_CONV_F16, EPI_RAW_NCHWC, f16, MT=2'),
    'box_splitk': ((1, 256, 24, 24, 64, 3, 1, 1), 'A_CONV_BOX, EPI_RAW_NCHWC, f16, MT=1, split-K'),
    'im2col_splitk': ((1, 256, 24, 24, 64, 3, 2, 1), 'A_CONV_TMA, EPI_RAW_NCHWC, f16, MT=1, split-K'),
}


@pytest.mark.parametrize('case', sorted(FP16_CASES))
def test_fp16_conv_variants(U, oracle, case):
    (n, ci, h, w, co, k, s, p), variant = FP16_CASES[case]
    rng = np.random.default_rng(zlib.crc32(case.encode()))
    x = rng.standard_normal((n, ci // 16, h, w, 16)).astype(np.float16)
    wt = (rng.standard_normal((co // 16, ci // 16, k, k, 16, 16)) * 0.05).astype(np.float16)
    before = variant_counts()
    got = U.conv2d_NCHW16c_OHWI16o(dev(x), dev(wt), s, s, padding=p)
    U.device_status()
    np.testing.assert_allclose(got.cpu().numpy(), oracle.conv2d_f16f32(x, wt, (s, s), (p, p)), rtol=RTOL, atol=ATOL)
    name = f'igemm_kernel<{variant}>'
    assert variant_counts()[name] > before[name], f'{case}: expected {name} to run'


DENSE_CASES = {
    # (m, n, k): matrices of at least 128 KB arrive by tensor copies (128-byte-swizzled rows when K is a
    # multiple of 128 bytes, 16-byte columns otherwise); smaller ones by the cp.async gather
    'tma_sw128_mt1': ((10000, 64, 384), 'A_DENSE_TMA, EPI_RAW_ROWS, {}, MT=1'),
    # the reference's split-K GEMM shape (poc/tensorcore/gemm-prefetch.cu: 128 x 768 x 3072): three tiles, eight CTAs each
    'tma_splitk': ((128, 768, 3072), 'A_DENSE_TMA, EPI_RAW_ROWS, {}, MT=1, split-K'),
    'tma_cols_mt1': ((2000, 64, 144), 'A_DENSE_TMA, EPI_RAW_ROWS, {}, MT=1'),
    'tma_mt2': ((20000, 16, 128), 'A_DENSE_TMA, EPI_RAW_ROWS, {}, MT=2'),
    'gather_mt1': ((129, 48, 80), 'A_DENSE, EPI_RAW_ROWS, {}, MT=1'),
}


@pytest.mark.parametrize('case', sorted(DENSE_CASES))
def test_dense_and_gemm_variants(U, oracle, case):
    (m, n, k), variant = DENSE_CASES[case]
    rng = np.random.default_rng(zlib.crc32(case.encode()))
    before = variant_counts()
    a = rng.integers(0, 256, (m, k), dtype=np.uint8)
    b = rng.integers(-128, 128, (n, k), dtype=np.int8)
    bp = no.pack_dense_weights(b, 16)
    got = U.dense_dotprod(dev(a), dev(bp))
    af = rng.standard_normal((m, k)).astype(np.float16)
    bf = (rng.standard_normal((k, n)) * 0.05).astype(np.float16)
    gotf = U.gemm_f16f32(dev(af), dev(bf))
    U.device_status()
    assert np.array_equal(got.cpu().numpy(), oracle.dense_u8s8s32(a, bp, vnni=oracle.host_has_vnni()))
    np.testing.assert_allclose(gotf.cpu().numpy(), no.gemm_f32(af, bf), rtol=RTOL, atol=ATOL)
    after = variant_counts()
    for dt in ('i8', 'f16'):
        name = 'igemm_kernel<' + variant.format(dt) + '>'
        assert after[name] > before[name], f'{case}: expected {name} to run'


def test_tensor_map_size_boundary(U, oracle):
    """Tensors below 128 KB take the cp.async gather, tensors from 128 KB on the tensor copies: both
    sides of the boundary, for stride 1 (box copies), stride 2 with a 3x3 kernel (box copies of pixel
    pairs) and stride 2 with a 1x1 kernel (im2col copies), same results."""
    rng = np.random.default_rng(131072)
    for s, k, at in ((1, 3, 'A_CONV_BOX'), (2, 3, 'A_CONV_BOX'), (2, 1, 'A_CONV_TMA')):
        for (h, w, path) in ((64, 62, 'A_CONV_I8'), (64, 64, at)):   # 32 x 64 x 64 bytes = 131072 exactly
            x = rng.integers(0, 256, (1, 2, h, w, 16), dtype=np.uint8)
            wt = rng.integers(-128, 128, (2, 2, k, k, 4, 16, 4), dtype=np.int8)
            before = variant_counts()
            got = U.conv2d_NCHWc_int8(dev(x), dev(wt), stride=s, padding=k // 2)
            U.device_status()
            assert np.array_equal(got.cpu().numpy(), oracle.conv2d_u8s8(x, wt, (s, s), (k // 2, k // 2)))
            name = f'igemm_kernel<{path}, EPI_RAW_NCHWC, i8, MT=1>'
            assert variant_counts()[name] > before[name], (h, w, s, k, name)


@pytest.mark.parametrize('n,ci,hw,co,k,s', [
    (12, 256, 14, 256, 3, 1),     # 19 tiles -> clusters of 7
    (32, 256, 14, 256, 3, 1),     # 49 tiles -> clusters of 3 (the ResNet-50 stage-3 3x3 at batch 32)
    (44, 64, 14, 320, 1, 1),      # 68 tiles x 2 column blocks: just under the limit of half the SMs -> no split
    (32, 2048, 14, 256, 1, 1),    # clusters of 3, 1x1
    (32, 512, 7, 512, 3, 1),      # 26 tiles -> clusters of 5, two column blocks
    (1, 4096, 28, 128, 1, 1),     # 7 tiles -> clusters of 8
    (20, 512, 14, 512, 3, 2),     # im2col copies, 8 x 2 tiles
    (33, 2048, 7, 208, 1, 1),     # column block of 208: 13 groups dealt to the cluster's CTAs unevenly
])
def test_split_k_cluster_sizes_bit_exact(U, oracle, n, ci, hw, co, k, s):
    """Split-K with every cluster size: partial sums exchanged through distributed shared memory, bias
    added once, requantised by the owners of the columns; integer sums, so still bit-exact."""
    rng = np.random.default_rng(n * 131 + ci + co)
    x = rng.integers(0, 256, (n, ci // 16, hw, hw, 16), dtype=np.uint8)
    wt = rng.integers(-128, 128, (co // 16, ci // 16, k, k, 4, 16, 4), dtype=np.int8)
    p = k // 2
    for hi in (2 ** 15, 2 ** 28):     # biases that enter through the tensor core, and ones the drain adds
        b = rng.integers(-hi, hi, co, dtype=np.int64).astype(np.int32)
        got = U.conv2d_NCHWc_int8(dev(x), dev(wt), stride=s, padding=p, bias=dev(b), out_dtype='uint8')
        gots = U.conv2d_NCHWc_int8(dev(x), dev(wt), stride=s, padding=p, bias=dev(b))
        U.device_status()
        vn = oracle.host_has_vnni()
        assert np.array_equal(got.cpu().numpy(), oracle.conv2d_u8s8(x, wt, (s, s), (p, p), bias=b, requant_shift=8, vnni=vn))
        assert np.array_equal(gots.cpu().numpy(), oracle.conv2d_u8s8(x, wt, (s, s), (p, p), bias=b, vnni=vn))


def test_plan_then_run_equals_the_direct_call(U, oracle):
    rng = np.random.default_rng(9)
    x = rng.integers(0, 256, (6, 4, 40, 40, 16), dtype=np.uint8)
    wt = rng.integers(-128, 128, (4, 4, 3, 3, 4, 16, 4), dtype=np.int8)
    b = rng.integers(-2 ** 15, 2 ** 15, 64, dtype=np.int32)
    xd, bd = dev(x), dev(b)
    pw = U.pack_conv_weights_int8(dev(wt), 1, 1)
    want = oracle.conv2d_u8s8(x, wt, (1, 1), (1, 1), bias=b, requant_shift=8)
    plan = U.conv2d_NCHWc_int8_plan(xd, pw, stride=1, padding=1, bias=bd, out_dtype='uint8')
    for _ in range(2):
        plan.out.zero_()
        out = plan.run()
        U.device_status()
        assert np.array_equal(out.cpu().numpy(), want)
    # new data in the same buffers: the plan names buffers, not values
    x2 = rng.integers(0, 256, x.shape, dtype=np.uint8)
    xd.copy_(dev(x2))
    assert np.array_equal(plan.run().cpu().numpy(), oracle.conv2d_u8s8(x2, wt, (1, 1), (1, 1), bias=b, requant_shift=8))
    # a folded stem: the plan carries the pre-pass and its scratch
    xs = rng.integers(0, 256, (9, 1, 64, 64, 4), dtype=np.uint8)
    ws = rng.integers(-128, 128, (2, 1, 7, 7, 1, 16, 4), dtype=np.int8)
    plan = U.conv2d_NCHWc_int8_plan(dev(xs), dev(ws), stride=2, padding=3)
    assert np.array_equal(plan.run().cpu().numpy(), oracle.conv2d_u8s8(xs, ws, (2, 2), (3, 3)))
    U.device_status()


def test_signed_activations_match_the_reference_graph_flow(U, oracle):
    """s8 activations: the reference shifts them to u8, convolves, subtracts 128 * sum(w), adds the
    bias and multiplies by 11 (apps/cpu/relay/result.log:3-24 on x (1, 1024, 16, 16), w (2048, 1024, 1, 1));
    the library multiplies s8 x s8 directly.  Same numbers, with and without padding."""
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), 'golden', 'golden_relay_flow.npz'))   # committed vectors
    for tag, p in (('valid', 0), ('padded', 1)):
        got = U.conv2d_NCHWc_int8(dev(g['x']), dev(g['w']), padding=p, bias=dev(g['bias']), mul=11)
        assert np.array_equal(got.cpu().numpy(), g['out_' + tag]), tag
    rng = np.random.default_rng(11)
    cases = [((1, 1024, 16, 16), (2048, 1024, 1, 1), 1, 0),      # the logged shape
             ((3, 64, 30, 31), (96, 64, 3, 3), 1, 1), ((2, 32, 17, 19), (32, 32, 3, 3), 2, 1),
             ((4, 64, 40, 44), (64, 64, 3, 3), 2, 1),            # stride 2 on an even width: the pair form, signed
             ((3, 32, 38, 40), (48, 32, 5, 5), 2, 2),
             ((2, 3, 34, 34), (32, 3, 7, 7), 2, 3)]              # NCHW4c stem, folded
    for xs, wsh, s, p in cases:
        x = np.clip(rng.standard_normal(xs) * 128, -128, 127).astype(np.int8)       # the script's distribution
        w = np.clip(rng.standard_normal(wsh) * 128, -128, 127).astype(np.int8)
        b = (rng.standard_normal(wsh[0]) * 128).astype(np.int32)
        cb = 16 if xs[1] % 16 == 0 else 4
        xp, wp = no.pack_nchw_to_nchwc(x, cb), no.pack_oihw_to_int8_weights(w, cb)
        want = oracle.conv2d_s8s8_relay_flow(xp, wp, (s, s), (p, p), bias=b, mul=11)
        got = U.conv2d_NCHWc_int8(dev(xp), dev(wp), stride=s, padding=p, bias=dev(b), mul=11)
        U.device_status()
        assert np.array_equal(got.cpu().numpy(), want), (xs, wsh, s, p)
        gotq = U.conv2d_NCHWc_int8(dev(xp), dev(wp), stride=s, padding=p, bias=dev(b), requant_shift=10)
        assert np.array_equal(gotq.cpu().numpy(), oracle.conv2d_i8_ex(xp, wp, (s, s), (p, p), bias=b, requant_shift=10))


def test_bottleneck_block_chains_in_layout(U, oracle):
    """A residual block u8 NCHW16c -> u8 NCHW16c with no repack: 1x1 reduce, 3x3, 1x1 expand with the
    block's input added before the clamp (ReLU), every layer reading the previous layer's output."""
    rng = np.random.default_rng(23)
    x = rng.integers(0, 256, (4, 16, 28, 28, 16), dtype=np.uint8) * rng.integers(0, 2, (4, 16, 28, 28, 16), dtype=np.uint8)
    w1 = np.clip(np.rint(rng.normal(0, 12, (4, 16, 1, 1, 4, 16, 4))), -128, 127).astype(np.int8)
    w2 = np.clip(np.rint(rng.normal(0, 12, (4, 4, 3, 3, 4, 16, 4))), -128, 127).astype(np.int8)
    w3 = np.clip(np.rint(rng.normal(0, 12, (16, 4, 1, 1, 4, 16, 4))), -128, 127).astype(np.int8)
    b1, b2, b3 = (rng.integers(-2 ** 12, 2 ** 12, c, dtype=np.int32) for c in (64, 64, 256))
    r1 = oracle.conv2d_i8_ex(x, w1, bias=b1, requant_shift=9)
    r2 = oracle.conv2d_i8_ex(r1, w2, (1, 1), (1, 1), bias=b2, requant_shift=10)
    want = oracle.conv2d_i8_ex(r2, w3, bias=b3, requant_shift=9, residual=x)
    xd = dev(x)
    pws = [U.pack_conv_weights_int8(dev(w), 1, pad) for w, pad in ((w1, 0), (w2, 1), (w3, 0))]
    for _ in range(3):
        y1 = U.conv2d_NCHWc_int8(xd, pws[0], bias=dev(b1), requant_shift=9)
        y2 = U.conv2d_NCHWc_int8(y1, pws[1], padding=1, bias=dev(b2), requant_shift=10)
        y3 = U.conv2d_NCHWc_int8(y2, pws[2], bias=dev(b3), requant_shift=9, residual=xd)
        assert np.array_equal(y3.cpu().numpy(), want)
    U.device_status()
    assert (want == 0).mean() > 0.05 and (want == 255).mean() < 0.5   # the clamp really acts as a ReLU here


def test_bounded_wait_reports_device_wait_and_the_library_recovers(U, oracle):
    """The error path of the bounded waits.  With weight copies stalled by the diagnostics hook no
    pipeline stage ever completes; after the (shortened) limit every role gives up, the kernel
    frees its tensor memory and returns, and unit_device_status reports UNIT_ERR_DEVICE_WAIT once.
    The next call, with the hook off, runs normally."""
    from unit_b200 import _lib
    L = _lib.lib()
    rng = np.random.default_rng(3)
    for shape in ((2, 2, 12, 12, 16), (6, 4, 40, 40, 16)):    # gather-fed and tensor-copy-fed A operand
        x = rng.integers(0, 256, shape, dtype=np.uint8)
        wt = rng.integers(-128, 128, (2, shape[1], 3, 3, 4, 16, 4), dtype=np.int8)
        xd, wd = dev(x), dev(wt)
        want = oracle.conv2d_u8s8(x, wt, (1, 1), (1, 1))
        assert np.array_equal(U.conv2d_NCHWc_int8(xd, wd, padding=1).cpu().numpy(), want)
        U.device_status()
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        try:
            assert L.unit_debug_set(_lib.DEBUG_WAIT_LIMIT_NS, 2_000_000) == 0      # 2 ms
            assert L.unit_debug_set(_lib.DEBUG_STALL_WEIGHT_COPIES, 1) == 0
            U.conv2d_NCHWc_int8(xd, wd, padding=1)
            assert L.unit_device_status(stream) == -7
        finally:
            L.unit_debug_set(_lib.DEBUG_STALL_WEIGHT_COPIES, 0)
            L.unit_debug_set(_lib.DEBUG_WAIT_LIMIT_NS, 1_000_000_000)
        assert L.unit_device_status(stream) == 0                                    # reported once, then clear
        for _ in range(2):
            assert np.array_equal(U.conv2d_NCHWc_int8(xd, wd, padding=1).cpu().numpy(), want)
        U.device_status()


@pytest.mark.parametrize('n,c,d,h,w,co,k,s,p', [
    (1, 64, 10, 18, 18, 64, 3, 1, 0),      # valid, as the reference runs it: box copies over (depth, rows)
    (1, 64, 10, 18, 18, 64, 3, 1, 1),      # padded in all three dimensions
    (2, 64, 11, 19, 19, 32, 3, 2, 1),      # stride 2: im2col copies with three tap offsets; two images
    (1, 128, 8, 20, 20, 32, 1, 2, 0),      # 1x1x1, stride 2
    (1, 16, 5, 6, 7, 16, 3, 1, 1),         # small: the cp.async gather
    (1, 256, 8, 14, 14, 256, 3, 1, 0),     # long reduction (27 taps x 16 chunks), few tiles: split-K
    (1, 32, 30, 40, 24, 48, 3, 1, 1),      # depth tiles that straddle rows and slices
])
def test_conv3d_int8_bit_exact(U, oracle, n, c, d, h, w, co, k, s, p):
    """Three-dimensional convolution on NCDHW16c (apps/cpu/kernel/conv3d.py:39-64): the depth axis runs
    through the same kernel in place of the batch axis.  Bit-exact, s32 with bias and requantised."""
    rng = np.random.default_rng(n + c + d + h + co + k + s)
    x = rng.integers(0, 256, (n, c // 16, d, h, w, 16), dtype=np.uint8)
    wt = rng.integers(-128, 128, (co // 16, c // 16, k, k, k, 4, 16, 4), dtype=np.int8)
    b = rng.integers(-2 ** 15, 2 ** 15, co, dtype=np.int32)
    ref = oracle.conv3d_u8s8(x, wt, (s, s, s), (p, p, p), bias=b)
    got = U.conv3d_NCDHWc_int8(dev(x), dev(wt), stride=s, padding=p, bias=dev(b))
    U.device_status()
    assert np.array_equal(got.cpu().numpy(), ref)
    gotq = U.conv3d_NCDHWc_int8(dev(x), dev(wt), stride=s, padding=p, bias=dev(b), requant_shift=10)
    want = np.clip((ref.astype(np.int64) + 512) >> 10, 0, 255).astype(np.uint8)
    assert np.array_equal(gotq.cpu().numpy(), want)
    U.device_status()


def test_tile_table_overrides_keep_results(U, oracle):
    """Every override a tile-table entry can carry (column-block width, stage depth, sub-tiles, split-K
    limit) changes how the work is cut, never the result; the tuner's own bit-exactness check in small."""
    from unit_b200 import ops, tile_table
    rng = np.random.default_rng(404)
    x = rng.integers(0, 256, (8, 16, 14, 14, 16), dtype=np.uint8)          # 3x3 256 -> 256 @14^2: splits by default
    wt = rng.integers(-128, 128, (16, 16, 3, 3, 4, 16, 4), dtype=np.int8)
    b = rng.integers(-2 ** 15, 2 ** 15, 256, dtype=np.int32)
    want = oracle.conv2d_u8s8(x, wt, (1, 1), (1, 1), bias=b, requant_shift=8, vnni=oracle.host_has_vnni())
    key = dict(c_in=256, c_block=16, c_out=256, kh=3, kw=3, stride_h=1, stride_w=1)
    try:
        for over in ({}, dict(bn=64), dict(bn=128, kc=4), dict(bn=256, kc=6), dict(mt=2), dict(mt=1, ksplit=1), dict(ksplit=2),
                     dict(bn=128, ksplit=8)):
            entries = []
            if 'bn' in over or 'kc' in over:
                entries.append(dict(key, n=0, bn=over.get('bn', 0), kc=over.get('kc', 0)))
            entries.append(dict(key, n=8, h=14, w=14, mt=over.get('mt', 0), ksplit=over.get('ksplit', 0)))
            tile_table.set_table(entries if over else [])
            ops._PACK_CACHE.clear()
            got = U.conv2d_NCHWc_int8(dev(x), dev(wt), padding=1, bias=dev(b), out_dtype='uint8')
            U.device_status()
            assert np.array_equal(got.cpu().numpy(), want), over
    finally:
        tile_table.set_table([])
        ops._PACK_CACHE.clear()


def test_zz_every_compiled_variant_was_launched(U):
    """Runs after the cases above (same module, definition order): no compiled variant is left
    that no parity case reaches."""
    counts = variant_counts()
    assert len(counts) >= 40
    never = sorted(k for k, v in counts.items() if v == 0)
    assert not never, 'compiled variants no test reached: ' + ', '.join(never)
