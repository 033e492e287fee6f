"""Regenerates the committed golden fixtures.

    python tests/golden/make_golden.py [reference checkout]

* ``poc_vnni_kat.json`` -- stdout of the reference's own known-answer program
  (poc/vnni/poc.cc, a[i] = i + 1, b[i] = 64 - i), compiled unmodified into
  ``oracle/_ref/poc_vnni`` by ``make -C oracle ref`` and run here.  Needs a
  host with AVX-512 VNNI.
* ``golden_small.npz`` -- seeded inputs and expected outputs of small cases of
  every contraction, computed with the numpy definitions on logical
  NCHW / OIHW tensors (oracle/np_oracle.py) and stored in the reference's
  blocked layouts.  The reference's own Python path needs a forked TVM that is
  not available, so these vectors come from the definition the reference
  checks itself against (exact integer matmul / convolution:
  poc/vnni/vnni_dense.py:58-67, poc/vnni/vnni_conv2d_NCHWxc.py:64-71; fp32
  accumulation: apps/gpu/conv-wdim.py:33-36,87).
"""
import json
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import np_oracle as no  # noqa: E402


def kat(ref):
    env = dict(os.environ)
    env.pop('CC', None)
    env.pop('CXX', None)
    subprocess.run(['make', '-C', os.path.join(ROOT, 'oracle'), 'ref', f'REF={ref}'], check=True, env=env)
    out = subprocess.run([os.path.join(ROOT, 'oracle', '_ref', 'poc_vnni')], check=True, capture_output=True,
                         text=True).stdout.strip().splitlines()
    hw = [int(t) for t in out[0].split()]
    scalar = [int(t) for t in out[1].split()]
    assert hw == scalar and len(hw) == 16
    with open(os.path.join(HERE, 'poc_vnni_kat.json'), 'w') as f:
        json.dump({'source': 'poc/vnni/poc.cc compiled unmodified and run', 'a': 'a[i] = i + 1, i < 64',
                   'b': 'b[i] = 64 - i, i < 64', 'c': 'zeros', 'd': hw}, f, indent=1)


def small():
    rng = np.random.default_rng(20240607)
    g = {}
    # int8 conv 3x3 s1 p1, two images, 32 -> 48 channels
    x = rng.integers(0, 256, (2, 32, 6, 7), dtype=np.uint8)
    w = rng.integers(-128, 128, (48, 32, 3, 3), dtype=np.int8)
    b = rng.integers(-2 ** 15, 2 ** 15, 48, dtype=np.int32)
    acc = no.conv2d_int_nchw(x, w, (1, 1), (1, 1))
    g['c1_x'] = no.pack_nchw_to_nchwc(x)
    g['c1_w'] = no.pack_oihw_to_int8_weights(w)
    g['c1_bias'] = b
    g['c1_out'] = no.pack_nchw_to_nchwc(acc.astype(np.int32))
    g['c1_req'] = no.pack_nchw_to_nchwc(no.requant_u8(acc, b, 8))
    # int8 conv 3x3 s2 p1
    acc = no.conv2d_int_nchw(x, w, (2, 2), (1, 1))
    g['c2_out'] = no.pack_nchw_to_nchwc(acc.astype(np.int32))
    # stem-like 7x7 s2 p3 on 3 channels (NCHW4c)
    xs = rng.integers(0, 256, (1, 3, 18, 18), dtype=np.uint8)
    ws = rng.integers(-128, 128, (16, 3, 7, 7), dtype=np.int8)
    acc = no.conv2d_int_nchw(xs, ws, (2, 2), (3, 3))
    g['st_x'] = no.pack_nchw_to_nchwc(xs, 4)
    g['st_w'] = no.pack_oihw_to_int8_weights(ws, 4)
    g['st_out'] = no.pack_nchw_to_nchwc(acc.astype(np.int32))
    # int8 dense with extreme values to pin signedness (u8 255 x s8 -128)
    a = rng.integers(0, 256, (20, 64), dtype=np.uint8)
    bm = rng.integers(-128, 128, (32, 64), dtype=np.int8)
    a[0, :] = 255
    bm[0, :] = -128
    bm[1, :] = 127
    g['d_a'] = a
    g['d_bp'] = no.pack_dense_weights(bm, 16)
    g['d_c'] = no.dense_int(a, bm).astype(np.int32)
    # fp16 conv with the reference's deterministic pattern (arange % 7), 3x3 valid
    n, c, h, wd, ko = 1, 32, 6, 6, 32
    xa = (np.arange(n * (c // 16) * h * wd * 16) % 7).astype(np.float16).reshape(n, c // 16, h, wd, 16)
    wa = (np.arange((ko // 16) * 3 * 3 * c * 16) % 7).astype(np.float16).reshape(ko // 16, c // 16, 3, 3, 16, 16)
    ref = no.conv2d_f32_nchw(no.unpack_nchwc_to_nchw(xa), no.unpack_f16_weights_to_oihw(wa), (1, 1), (0, 0))
    g['f_x'], g['f_w'], g['f_out'] = xa, wa, no.pack_nchw_to_nchwc(ref)
    # fp16 gemm
    ga = rng.standard_normal((24, 64)).astype(np.float16)
    gb = (rng.standard_normal((64, 32)) * 0.05).astype(np.float16)
    g['g_a'], g['g_b'], g['g_c'] = ga, gb, no.gemm_f32(ga, gb)
    np.savez_compressed(os.path.join(HERE, 'golden_small.npz'), **g)
    # The reference's fused graph operator on signed activations (apps/cpu/relay/conv2d.py:16-23,
    # apps/cpu/relay/result.log:3-24): multiply(add(conv2d(x s8, w s8), bias), 11) in wrapping s32, here
    # straight from the signed definition (no +128 shift), with the script's value distributions.
    r = {}
    rs = np.random.default_rng(11)
    xs8 = np.clip(rs.standard_normal((2, 32, 10, 9)) * 128, -128, 127).astype(np.int8)
    ws8 = np.clip(rs.standard_normal((48, 32, 3, 3)) * 128, -128, 127).astype(np.int8)
    bs = (rs.standard_normal(48) * 128).astype(np.int32)
    for tag, pad in (('valid', (0, 0)), ('padded', (1, 1))):
        acc = no.conv2d_int_nchw(xs8, ws8, (1, 1), pad) + bs.astype(np.int64)[None, :, None, None]
        out = ((acc * 11) & 0xFFFFFFFF).astype(np.uint32).view(np.int32)
        r['out_' + tag] = no.pack_nchw_to_nchwc(out)
    r['x'] = no.pack_nchw_to_nchwc(xs8)
    r['w'] = no.pack_oihw_to_int8_weights(ws8)
    r['bias'] = bs
    np.savez_compressed(os.path.join(HERE, 'golden_relay_flow.npz'), **r)


if __name__ == '__main__':
    # the reference checkout: first argument, else $UNIT_REFERENCE (without either only the second fixture is made)
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get('UNIT_REFERENCE', '')
    if ref and os.path.exists(os.path.join(ref, 'poc', 'vnni', 'poc.cc')):
        kat(ref)
    small()
    print('wrote fixtures')
