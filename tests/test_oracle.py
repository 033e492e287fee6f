"""The oracle against the reference's known answers, the committed golden
vectors and the numpy definitions.  CPU only."""
import json
import os

import numpy as np
import pytest

from oracle import np_oracle as no

HERE = os.path.dirname(os.path.abspath(__file__))


def test_poc_vnni_known_answer(oracle):
    """poc/vnni/poc.cc: a[i]=i+1, b[i]=64-i, d = dpbusd(0, a, b)."""
    with open(os.path.join(HERE, 'golden', 'poc_vnni_kat.json')) as f:
        kat = json.load(f)
    a = (np.arange(64) + 1).astype(np.uint8)
    b = (64 - np.arange(64)).astype(np.int8)
    c = np.zeros(16, np.int32)
    assert oracle.vnni_dot(a, b, c).tolist() == kat['d']
    if oracle.host_has_vnni():
        assert oracle.vnni_dot(a, b, c, hw=True).tolist() == kat['d']


def test_reference_kat_binary_if_built():
    exe = os.path.join(os.path.dirname(HERE), 'oracle', '_ref', 'poc_vnni')
    if not os.path.exists(exe):
        pytest.skip('oracle/_ref/poc_vnni not built (needs the reference checkout)')
    from oracle import c_oracle
    if not c_oracle.host_has_vnni():
        pytest.skip('host has no AVX-512 VNNI')
    import subprocess
    out = subprocess.run([exe], capture_output=True, text=True, check=True).stdout.split('\n')
    with open(os.path.join(HERE, 'golden', 'poc_vnni_kat.json')) as f:
        assert [int(t) for t in out[0].split()] == json.load(f)['d']


def test_vnni_dot_signedness_and_wrap(oracle):
    """First operand unsigned, second signed, plain wrapping s32 add (vpdpbusd, not vpdpbusds)."""
    a = np.full(64, 200, np.uint8)
    b = np.full(64, -128, np.int8)
    c = np.zeros(16, np.int32)
    assert (oracle.vnni_dot(a, b, c) == -102400).all()
    c = np.full(16, np.iinfo(np.int32).min + 5, np.int32)
    want = (c.astype(np.int64) - 102400 + 2 ** 32) % 2 ** 32
    got = oracle.vnni_dot(a, b, c).astype(np.int64) % 2 ** 32
    assert (got == want).all()
    if oracle.host_has_vnni():
        assert (oracle.vnni_dot(a, b, c, hw=True) == oracle.vnni_dot(a, b, c)).all()


def test_golden_int8_conv(oracle, golden):
    g = golden
    assert np.array_equal(oracle.conv2d_u8s8(g['c1_x'], g['c1_w'], (1, 1), (1, 1)), g['c1_out'])
    assert np.array_equal(oracle.conv2d_u8s8(g['c1_x'], g['c1_w'], (2, 2), (1, 1)), g['c2_out'])
    assert np.array_equal(
        oracle.conv2d_u8s8(g['c1_x'], g['c1_w'], (1, 1), (1, 1), bias=g['c1_bias'], requant_shift=8), g['c1_req'])
    assert np.array_equal(oracle.conv2d_u8s8(g['st_x'], g['st_w'], (2, 2), (3, 3)), g['st_out'])


def test_golden_dense_and_fp16(oracle, golden):
    g = golden
    assert np.array_equal(oracle.dense_u8s8s32(g['d_a'], g['d_bp']), g['d_c'])
    # arange % 7 inputs are small integers: fp32 accumulation is exact
    assert np.array_equal(oracle.conv2d_f16f32(g['f_x'], g['f_w']), g['f_out'])
    np.testing.assert_allclose(oracle.gemm_f16f32(g['g_a'], g['g_b']), g['g_c'], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize('n,ci,h,w,co,kh,kw,s,p', [
    (1, 16, 5, 5, 16, 1, 1, 1, 0),
    (2, 32, 9, 10, 48, 3, 3, 1, 1),
    (2, 32, 9, 10, 48, 3, 3, 2, 1),
    (1, 64, 7, 7, 32, 3, 3, 1, 0),
    (1, 16, 12, 9, 16, 1, 7, 1, 0),
    (1, 16, 12, 9, 16, 7, 1, 1, 3),
    (3, 48, 8, 8, 64, 1, 1, 2, 0),
    # the blocked forms of the AVX-512 restatement: rows of 14 and more outputs (1 x 14 blocks, the
    # last one moved back when ragged), 7-wide maps (2 x 7 blocks, odd row count), with and without padding
    (2, 32, 14, 14, 32, 3, 3, 1, 1),
    (1, 16, 19, 17, 16, 3, 3, 1, 1),
    (1, 16, 33, 31, 32, 3, 3, 2, 1),
    (2, 32, 7, 7, 32, 3, 3, 1, 1),
    (1, 48, 14, 14, 16, 3, 3, 2, 1),
    (1, 16, 9, 9, 16, 3, 3, 1, 0),
    (2, 16, 30, 30, 16, 1, 1, 1, 0),
])
def test_c_oracle_equals_numpy_definition(oracle, n, ci, h, w, co, kh, kw, s, p):
    rng = np.random.default_rng(n * 1000 + ci + kh)
    x = rng.integers(0, 256, (n, ci, h, w), dtype=np.uint8)
    wt = rng.integers(-128, 128, (co, ci, kh, kw), dtype=np.int8)
    b = rng.integers(-2 ** 15, 2 ** 15, co, dtype=np.int32)
    xp, wp = no.pack_nchw_to_nchwc(x), no.pack_oihw_to_int8_weights(wt)
    ref = no.conv2d_int_nchw(x, wt, (s, s), (p, p))
    got = oracle.conv2d_u8s8(xp, wp, (s, s), (p, p))
    assert np.array_equal(no.unpack_nchwc_to_nchw(got), ref)
    q = oracle.conv2d_u8s8(xp, wp, (s, s), (p, p), bias=b, requant_shift=8)
    assert np.array_equal(no.unpack_nchwc_to_nchw(q), no.requant_u8(ref, b, 8))
    if oracle.host_has_vnni():
        assert np.array_equal(oracle.conv2d_u8s8(xp, wp, (s, s), (p, p), vnni=True), got)
        assert np.array_equal(oracle.conv2d_u8s8(xp, wp, (s, s), (p, p), bias=b, requant_shift=8, vnni=True), q)


def test_stem_layout_nchw4c(oracle):
    rng = np.random.default_rng(3)
    x = rng.integers(0, 256, (2, 3, 21, 21), dtype=np.uint8)
    wt = rng.integers(-128, 128, (64, 3, 7, 7), dtype=np.int8)
    xp, wp = no.pack_nchw_to_nchwc(x, 4), no.pack_oihw_to_int8_weights(wt, 4)
    assert xp.shape == (2, 1, 21, 21, 4) and wp.shape == (4, 1, 7, 7, 1, 16, 4)
    ref = no.conv2d_int_nchw(x, wt, (2, 2), (3, 3))
    got = oracle.conv2d_u8s8(xp, wp, (2, 2), (3, 3))
    assert np.array_equal(no.unpack_nchwc_to_nchw(got), ref)
    if oracle.host_has_vnni():
        assert np.array_equal(oracle.conv2d_u8s8(xp, wp, (2, 2), (3, 3), vnni=True), got)


def test_impulses_pin_the_index_maps(oracle):
    """One non-zero activation and one non-zero weight: the output has exactly one non-zero."""
    x = np.zeros((1, 32, 5, 6), np.uint8)
    w = np.zeros((32, 32, 3, 3), np.int8)
    x[0, 19, 2, 3] = 7
    w[21, 19, 0, 2] = -5
    got = no.unpack_nchwc_to_nchw(oracle.conv2d_u8s8(no.pack_nchw_to_nchwc(x), no.pack_oihw_to_int8_weights(w),
                                                     (1, 1), (1, 1)))
    nz = np.argwhere(got)
    # out[oh][ow] reads x[oh + kh - 1][ow + kw - 1]  ->  oh = 2 - 0 + 1, ow = 3 - 2 + 1
    assert nz.tolist() == [[0, 21, 3, 2]] and got[0, 21, 3, 2] == -35


def test_extremes_do_not_overflow_at_resnet_depth(oracle):
    """255 * -128 * 4608 taps stays inside s32 (the deepest ResNet-50 reduction)."""
    x = np.full((1, 512, 3, 3), 255, np.uint8)
    w = np.full((16, 512, 3, 3), -128, np.int8)
    got = oracle.conv2d_u8s8(no.pack_nchw_to_nchwc(x), no.pack_oihw_to_int8_weights(w), (1, 1), (0, 0))
    assert got.shape == (1, 1, 1, 1, 16) and (got == -255 * 128 * 4608).all()


def test_requant_rounding_definition(oracle):
    """q = clamp((acc + bias + 128) >> 8, 0, 255): half rounds up, negatives clamp to 0."""
    x = np.zeros((1, 16, 1, 1), np.uint8)
    x[0, 0, 0, 0] = 1
    w = np.zeros((16, 16, 1, 1), np.int8)
    w[:, 0, 0, 0] = 1  # acc = 1 for every output channel
    bias = np.array([-1, 126, 127, 128, 383, 384, 65151, 65152, 10 ** 6, -10 ** 6, -129, -128, 0, 255, 256, 639], np.int32)
    q = oracle.conv2d_u8s8(no.pack_nchw_to_nchwc(x), no.pack_oihw_to_int8_weights(w), bias=bias, requant_shift=8)
    want = np.clip((1 + bias.astype(np.int64) + 128) >> 8, 0, 255)
    assert q.reshape(-1).tolist() == want.tolist()


def test_dense_vnni_equals_scalar_and_matmul(oracle):
    rng = np.random.default_rng(5)
    a = rng.integers(0, 256, (37, 128), dtype=np.uint8)
    b = rng.integers(-128, 128, (256, 128), dtype=np.int8)
    for t in (16, 128):
        bp = no.pack_dense_weights(b, t)
        assert np.array_equal(no.unpack_dense_weights(bp), b)
        ref = no.dense_int(a, b)
        assert np.array_equal(oracle.dense_u8s8s32(a, bp), ref)
        if oracle.host_has_vnni():
            assert np.array_equal(oracle.dense_u8s8s32(a, bp, vnni=True), ref)


def test_fp16_oracle_matches_numpy(oracle):
    rng = np.random.default_rng(9)
    x = rng.standard_normal((2, 32, 8, 8)).astype(np.float16)
    w = (rng.standard_normal((48, 32, 3, 3)) * 0.05).astype(np.float16)
    got = oracle.conv2d_f16f32(no.pack_nchw_to_nchwc(x), no.pack_oihw_to_f16_weights(w), (2, 2), (1, 1))
    ref = no.conv2d_f32_nchw(x, w, (2, 2), (1, 1))
    np.testing.assert_allclose(no.unpack_nchwc_to_nchw(got), ref, rtol=1e-4, atol=1e-5)
    a = rng.standard_normal((9, 40)).astype(np.float16)
    b = rng.standard_normal((40, 16)).astype(np.float16)
    np.testing.assert_allclose(oracle.gemm_f16f32(a, b), no.gemm_f32(a, b), rtol=1e-5, atol=1e-5)


def test_layout_round_trips():
    rng = np.random.default_rng(1)
    x = rng.integers(0, 256, (2, 19, 3, 4), dtype=np.uint8)
    assert np.array_equal(no.unpack_nchwc_to_nchw(no.pack_nchw_to_nchwc(x), 19), x)
    assert np.array_equal(no.unpack_nchwc_to_nchw(no.pack_nchw_to_nchwc(x, 4), 19), x)
    w = rng.integers(-128, 128, (32, 48, 3, 2), dtype=np.int8)
    assert np.array_equal(no.unpack_int8_weights_to_oihw(no.pack_oihw_to_int8_weights(w)), w)
    wf = rng.standard_normal((32, 48, 3, 2)).astype(np.float16)
    assert np.array_equal(no.unpack_f16_weights_to_oihw(no.pack_oihw_to_f16_weights(wf)), wf)
    # the literal index expression of the reference's packed weights
    wp = no.pack_oihw_to_int8_weights(w)
    oc, ic, kh, kw = 21, 37, 2, 1
    assert wp[oc // 16, ic // 16, kh, kw, (ic % 16) // 4, oc % 16, ic % 4] == w[oc, ic, kh, kw]


@pytest.mark.parametrize('c,d,h,w,co,k,s,p', [(16, 5, 6, 7, 16, 3, 1, 1), (32, 6, 7, 5, 32, 2, 2, 0), (16, 4, 9, 9, 16, 1, 2, 0)])
def test_conv3d_oracle_is_a_sum_of_2d_convolutions_over_the_depth_taps(oracle, c, d, h, w, co, k, s, p):
    """The 3-D definition (apps/cpu/kernel/conv3d.py:60-64) against the 2-D one: output slice od is the
    sum over kd of the 2-D convolution of input slice od*s + kd - p with the kd-th slice of the kernel."""
    rng = np.random.default_rng(c + d + k)
    x = rng.integers(0, 256, (2, c // 16, d, h, w, 16), dtype=np.uint8)
    wt = rng.integers(-128, 128, (co // 16, c // 16, k, k, k, 4, 16, 4), dtype=np.int8)
    b = rng.integers(-2 ** 15, 2 ** 15, co, dtype=np.int32)
    got = oracle.conv3d_u8s8(x, wt, (s, s, s), (p, p, p), bias=b)
    od = (d + 2 * p - k) // s + 1
    assert got.shape[2] == od
    for z in range(od):
        acc = np.zeros(got[:, :, z].shape, np.int64)
        for kd in range(k):
            iz = z * s + kd - p
            if 0 <= iz < d:
                acc += oracle.conv2d_u8s8(np.ascontiguousarray(x[:, :, iz]), np.ascontiguousarray(wt[:, :, kd]), (s, s), (p, p))
        acc += b.reshape(1, -1, 1, 1, 16)
        assert np.array_equal(got[:, :, z], acc.astype(np.int32))


def test_relay_flow_restatement_matches_the_signed_definition(oracle):
    """The reference's graph for s8 activations shifts them to u8, convolves, subtracts 128 * sum(w),
    adds the bias and multiplies by 11 (apps/cpu/relay/result.log:3-24).  Its restatement must equal the
    committed vectors, which were computed from the signed definition directly; so must the general
    epilogue function the GPU kernels are compared with."""
    g = np.load(os.path.join(HERE, 'golden', 'golden_relay_flow.npz'))
    for tag, pad in (('valid', (0, 0)), ('padded', (1, 1))):
        assert np.array_equal(oracle.conv2d_s8s8_relay_flow(g['x'], g['w'], (1, 1), pad, bias=g['bias'], mul=11), g['out_' + tag])
        assert np.array_equal(oracle.conv2d_i8_ex(g['x'], g['w'], (1, 1), pad, bias=g['bias'], mul=11), g['out_' + tag])
