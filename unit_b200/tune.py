"""Tuner for the per-shape tile table (run on a B200):

    python -m unit_b200.tune [--batch B ...] [--limit N] [--out unit_b200/tile_table.json]

For every int8 convolution shape of the corpus (the reference's ``cpu-shapes.log`` shapes, valid
convolution on the pre-padded sizes, at the logged batch 1 and at the batches given) it times the
library's own choice and the candidate overrides (column-block width, sub-tiles per tile, split-K
limit) as CUDA-graph replays over several buffer sets, checks that every candidate reproduces the
default's output bit for bit, and keeps an entry where a candidate beats the default by more than
3 %.  The counterpart of the reference's tuning loops (apps/cpu/kernel/conv2d.py:56-75,
python/tensorizer/tune.py).
"""
from __future__ import annotations

import argparse
import json
import sys
import time

import torch

from . import ops, tile_table
from .resnet50 import LAYERS


def _time_case(x_sets, w, stride, pad=0, reps=16):
    """us per launch of the convolution under the table in force (weights packed under it too)."""
    ops._PACK_CACHE.clear()
    pw = ops.pack_conv_weights_int8(w, stride, pad)
    plans = [ops.conv2d_NCHWc_int8_plan(x, pw, stride=stride, padding=pad, out_dtype='uint8') for x in x_sets]
    for p in plans:
        p.run()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        for _ in range(reps):
            for p in plans:
                p.run()
    g.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(3):
        g.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / (3 * reps * len(plans)), plans[0].out.clone()


def candidates(shape, weight_side=True):
    c_out = shape['c_out']
    bns = sorted({min(256, (c_out + 15) // 16 * 16), 128, 64} & set(range(16, 257, 16)))
    bns = [b for b in bns if b <= max(64, (c_out + 15) // 16 * 16)]
    out = []
    for bn in (bns if weight_side else []) + [0]:
        for mt in (0, 1, 2):
            for ks in (0, 1, 4, 8):
                if bn == 0 and mt == 0 and ks == 0:
                    continue
                out.append({'bn': bn, 'kc': 0, 'mt': mt, 'ksplit': ks})
    return out


def tune_shape(shape, batch, sets=4, weight_side=True):
    dev = torch.device('cuda')
    g = torch.Generator(device=dev).manual_seed(shape['c_in'] * 131 + shape['c_out'])
    cc = shape['c_in'] // 16
    xs = [torch.randint(0, 256, (batch, cc, shape['h'], shape['w'], 16), dtype=torch.uint8, device=dev, generator=g)
          for _ in range(sets)]
    w = torch.randint(-128, 128, (shape['c_out'] // 16, cc, shape['kh'], shape['kw'], 4, 16, 4), dtype=torch.int8, device=dev,
                      generator=g)
    stride = (shape['stride_h'], shape['stride_w'])
    tile_table.set_table([])
    pad = shape.get('pad', 0)
    base_us, base_out = _time_case(xs, w, stride, pad)
    key = {k: shape[k] for k in ('c_in', 'c_out', 'kh', 'kw', 'stride_h', 'stride_w')}
    key['c_block'] = 16
    best = (base_us, None)
    for cand in candidates(shape, weight_side):
        # the weight-side fields (bn, kc) must sit in an entry for every input size; mt / ksplit in one for this size
        entries = []
        if cand['bn'] or cand['kc']:
            entries.append(dict(key, n=0, h=0, w=0, bn=cand['bn'], kc=cand['kc'], mt=0, ksplit=0))
        entries.append(dict(key, n=batch, h=shape['h'], w=shape['w'], bn=0, kc=0, mt=cand['mt'], ksplit=cand['ksplit']))
        try:
            tile_table.set_table(entries)
            us, out = _time_case(xs, w, stride, pad)
        except (ValueError, RuntimeError):
            continue
        if not torch.equal(out, base_out):
            raise AssertionError(f'candidate {cand} changes the result for {shape}')
        if us < best[0]:
            best = (us, entries)
    tile_table.set_table([])
    ops.device_status()
    return base_us, best


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument('--batch', type=int, action='append', default=None, help='batch sizes besides the logged 1')
    ap.add_argument('--limit', type=int, default=0, help='tune only the first N shapes (0 = all)')
    ap.add_argument('--resnet50', action='store_true', help='also the ResNet-50 sweep shapes, with their implicit padding')
    ap.add_argument('--only-resnet50', action='store_true', help='the ResNet-50 sweep shapes alone')
    ap.add_argument('--out', default=tile_table.TABLE_PATH)
    ap.add_argument('--min-gain', type=float, default=0.03)
    ap.add_argument('--size-specific-only', action='store_true',
                    help='only overrides bound to one input size (sub-tiles, split-K): packed weights keep their shape')
    ap.add_argument('--merge', default=None, help='an existing table whose entries are kept (new entries for the same key win)')
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit('the tuner needs a B200')
    shapes = [] if args.only_resnet50 else tile_table.load_corpus()
    if args.resnet50 or args.only_resnet50:
        for l in LAYERS:
            if l.c_block == 16:
                shapes.append({'n': 1, 'c_in': l.c_in, 'h': l.hw, 'w': l.hw, 'c_out': l.c_out, 'kh': l.k, 'kw': l.k,
                               'stride_h': l.stride, 'stride_w': l.stride, 'pad': l.pad})
    if args.limit:
        shapes = shapes[:args.limit]
    batches = ([] if args.only_resnet50 else [1]) + [b for b in (args.batch or []) if b != 1 or args.only_resnet50]
    entries, report = [], []
    t0 = time.time()
    for i, sh in enumerate(shapes):
        for b in batches:
            # shapes of the ResNet-50 sweep run at many batch sizes: their weight-side choice stays with the heuristic
            in_sweep = any(l.c_in == sh['c_in'] and l.c_out == sh['c_out'] and l.k == sh['kh'] and l.stride == sh['stride_h'] for l in LAYERS)
            base_us, (best_us, best_entries) = tune_shape(sh, b, weight_side=not (args.size_specific_only or in_sweep))
            gain = base_us / best_us - 1.0
            row = {'shape': {k: sh[k] for k in sh if k != 'count'}, 'batch': b, 'default_us': round(base_us, 2),
                   'best_us': round(best_us, 2), 'gain': round(gain, 3)}
            if best_entries is not None and gain > args.min_gain:
                # weight-side overrides of different batches of one shape must agree: keep the first found
                for e in best_entries:
                    if e['n'] == 0 and any(o['n'] == 0 and all(o[k] == e[k] for k in ('c_in', 'c_out', 'kh', 'kw', 'stride_h', 'stride_w'))
                                           for o in entries):
                        continue
                    entries.append(e)
                row['entries'] = best_entries
            report.append(row)
        if (i + 1) % 10 == 0:
            print(f'[tune] {i + 1}/{len(shapes)} shapes, {len(entries)} entries, {time.time() - t0:.0f} s', file=sys.stderr, flush=True)
    if args.merge:
        with open(args.merge) as f:
            old = json.load(f).get('entries', [])
        keyf = lambda e: tuple(e.get(k, 0) for k in ('c_in', 'c_out', 'kh', 'kw', 'stride_h', 'stride_w', 'n', 'h', 'w'))
        new_keys = {keyf(e) for e in entries}
        entries = [e for e in old if keyf(e) not in new_keys] + entries
    gains = [r['gain'] for r in report]
    with open(args.out, 'w') as f:
        json.dump({'device': torch.cuda.get_device_name(0), 'min_gain': args.min_gain,
                   'summary': {'cases': len(report), 'mean_gain': sum(gains) / max(1, len(gains)), 'max_gain': max(gains) if gains else 0.0,
                               'default_us': sum(r['default_us'] for r in report), 'best_us': sum(r['best_us'] for r in report)},
                   'entries': entries}, f, indent=0)
    with open(args.out + '.report.json', 'w') as f:
        json.dump(report, f, indent=0)
    print(json.dumps({'shapes': len(shapes), 'cases': len(report), 'entries': len(entries),
                      'mean_gain': sum(gains) / max(1, len(gains)), 'max_gain': max(gains) if gains else 0.0, 'out': args.out}))
    return 0


if __name__ == '__main__':
    sys.exit(main())
