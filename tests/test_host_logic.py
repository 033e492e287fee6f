"""Host-side logic: layer table, operator argument checks, batch split (gloo, 2 ranks),
bench reference arm.  CPU only."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_resnet50_table_matches_the_network():
    from unit_b200 import resnet50 as R
    assert sum(l.count for l in R.LAYERS) == 53
    assert abs(R.sweep_ops(1) / 1e9 - 8.174) < 1e-2
    assert abs(R.sweep_ops(256) / 1e9 - 2092.6) < 0.1
    cfg1 = next(l for l in R.LAYERS if l.name == 's1_3x3_64_64')
    assert cfg1.ops(1) == 2 * 56 * 56 * 64 * 64 * 9 and cfg1.out_hw == 56
    stem = R.LAYERS[0]
    assert (stem.c_block, stem.c_in_stored, stem.out_hw) == (4, 4, 112)
    for l in R.LAYERS:  # every stage hands the next one a consistent map size
        assert l.out_hw in (112, 56, 28, 14, 7)


def test_synthetic_distributions():
    from unit_b200 import resnet50 as R
    rng = np.random.default_rng(0)
    a = R.synth_activations(rng, (200000,))
    assert 0.48 < (a == 0).mean() < 0.52 and a.max() == 255 and a[a > 0].min() == 1
    w = R.synth_weights(rng, (200000,))
    assert w.dtype == np.int8 and 30 < w.astype(np.float64).std() < 34 and w.min() >= -128
    x, wt, b = R.make_layer_inputs(R.LAYERS[0], 0, 2)
    assert x.shape == (2, 1, 224, 224, 4) and (x[..., 3] == 0).all() and wt.shape == (4, 1, 7, 7, 1, 16, 4)
    assert (wt[..., 3] == 0).all() and b.shape == (64,)
    x2, _, _ = R.make_layer_inputs(R.LAYERS[0], 0, 2)
    assert np.array_equal(x, x2)  # seeded


def test_operators_fail_loudly_without_cuda():
    if torch.cuda.is_available():
        pytest.skip('a CUDA device is present')
    import unit_b200 as U
    x = torch.zeros((1, 4, 8, 8, 16), dtype=torch.uint8)
    w = torch.zeros((4, 4, 3, 3, 4, 16, 4), dtype=torch.int8)
    with pytest.raises(RuntimeError, match='no CPU fallback'):
        U.conv2d_NCHWc_int8(x, w, stride=1, padding=1)
    with pytest.raises(RuntimeError, match='no CPU fallback'):
        U.dense_dotprod(torch.zeros((8, 64), dtype=torch.uint8), torch.zeros((1, 16, 64, 4), dtype=torch.int8))


def test_missing_library_is_an_import_error(monkeypatch, tmp_path):
    from unit_b200 import _lib, build
    monkeypatch.setattr(_lib, '_LIB', None)
    monkeypatch.setattr(build, 'LIB_PATH', str(tmp_path / 'libunit_b200.so'))
    with pytest.raises(ImportError, match='no CPU or eager fallback'):
        _lib.lib()


def test_product_never_imports_the_oracle():
    for dirpath, _, files in os.walk(os.path.join(ROOT, 'unit_b200')):
        for f in files:
            if f.endswith(('.py', '.cu', '.cuh', '.h')):
                txt = open(os.path.join(dirpath, f)).read()
                assert 'oracle' not in txt.replace('# oracle', ''), f'{f} mentions the oracle'


def test_registry_and_pairs():
    import unit_b200 as U
    from unit_b200.ops import _pair
    assert set(U.INTRINSICS) == {'vnni', 'tensorcore'}
    assert U.INTRINSICS['vnni']['pattern'] == {'out_lanes': 16, 'reduce_lanes': 4, 'a_dtype': 'uint8',
                                               'b_dtype': 'int8', 'out_dtype': 'int32'}
    assert _pair(2) == (2, 2) and _pair((1, 2)) == (1, 2) and _pair((1, 2, 1, 2)) == (1, 2)
    with pytest.raises(ValueError):
        _pair((1, 2, 3, 4))


def test_batch_slice_covers_the_batch():
    from unit_b200.sharding import batch_slice
    for total in (0, 1, 7, 256):
        for world in (1, 2, 3, 8):
            parts = [batch_slice(total, r, world) for r in range(world)]
            assert parts[0][0] == 0 and parts[-1][1] == total
            assert all(parts[i][1] == parts[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in parts]
            assert max(sizes) - min(sizes) <= 1
    assert batch_slice(256, 3, 8) == (96, 128)
    with pytest.raises(ValueError):
        batch_slice(8, 2, 2)


_GLOO_WORKER = r'''
import os, sys
sys.path.insert(0, sys.argv[1])
import numpy as np, torch, torch.distributed as dist
from oracle import c_oracle as co
from unit_b200.sharding import shard
rank, world = int(os.environ['RANK']), int(os.environ['WORLD_SIZE'])
dist.init_process_group('gloo')
rng = np.random.default_rng(11)                      # same tensors on every rank
x = rng.integers(0, 256, (5, 2, 9, 9, 16), dtype=np.uint8)
w = rng.integers(-128, 128, (2, 2, 3, 3, 4, 16, 4), dtype=np.int8)
b = rng.integers(-2**15, 2**15, 32, dtype=np.int32)
mine = co.conv2d_u8s8(shard(x, rank, world), w, (1, 1), (1, 1), bias=b, requant_shift=8)   # this rank's images only
sizes = [shard(x, r, world).shape[0] for r in range(world)]
parts = [torch.empty((s,) + mine.shape[1:], dtype=torch.uint8) for s in sizes]
dist.all_gather(parts, torch.from_numpy(mine)) if len(set(sizes)) == 1 else None
if len(set(sizes)) != 1:                             # ragged split: gather by broadcast
    for r in range(world):
        if r == rank: parts[r].copy_(torch.from_numpy(mine))
        dist.broadcast(parts[r], src=r)
full = co.conv2d_u8s8(x, w, (1, 1), (1, 1), bias=b, requant_shift=8)
assert np.array_equal(torch.cat(parts).numpy(), full), 'batch split changed the result'
t = torch.tensor([float(rank + 1)], dtype=torch.float64)
dist.all_reduce(t, op=dist.ReduceOp.MAX)             # the max-over-ranks timing reduction
assert t.item() == world
dist.barrier(); dist.destroy_process_group()
sys.stdout.write('rank%d-ok\n' % rank); sys.stdout.flush()
'''


def test_batch_split_two_ranks_gloo(tmp_path):
    script = tmp_path / 'worker.py'
    script.write_text(_GLOO_WORKER)
    env = dict(os.environ, OMP_NUM_THREADS='2')
    import socket
    with socket.socket() as s:   # a free rendezvous port
        s.bind(('127.0.0.1', 0))
        port = s.getsockname()[1]
    r = subprocess.run([sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node=2',
                        '--master-addr', '127.0.0.1', '--master-port', str(port), str(script), ROOT],
                       capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert 'rank0-ok' in r.stdout and 'rank1-ok' in r.stdout


def test_bench_reference_arm_prints_the_contract_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, 'bench.py'), '--impl', 'reference', '--steps', '1',
                        '--warmup', '0'], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line['impl'] == 'reference' and line['unit'] == 'TOPS' and line['value'] > 0
    assert line['cpu_baseline']['kind'] == 'port' and line['cpu_baseline']['cores'] >= 1
    assert line['e2e']['h2d_bytes_per_step'] == 0 and line['e2e']['value'] == line['value']
    assert line['config']['workload'] == 'resnet50-int8-conv-sweep'


def test_tile_table_overrides_are_host_side_and_reversible():
    """unit_tile_table_set: an entry for every input size changes the column-block width (visible in the
    packed size, a pure host function); clearing the table restores the heuristic; bad entries are refused."""
    import ctypes
    from unit_b200 import _lib, build, tile_table
    build.build()
    L = _lib.lib()
    d = _lib.ConvDesc(1, 64, 31, 31, 16, 80, 1, 1, 2, 2, 0, 0)     # (1x1 with stride 2: one packed copy only)
    base = L.unit_packed_weights_bytes_conv_i8(ctypes.byref(d))
    assert base == 4 * 80 * 16                        # one column block of 80
    key = dict(c_in=64, c_block=16, c_out=80, kh=1, kw=1, stride_h=2, stride_w=2)
    tile_table.set_table([dict(key, n=0, bn=64)])
    assert L.unit_packed_weights_bytes_conv_i8(ctypes.byref(d)) == 4 * 96 * 16      # two blocks of 48
    tile_table.set_table([dict(key, n=4, h=31, w=31, bn=64)])                        # size-specific: weights untouched
    assert L.unit_packed_weights_bytes_conv_i8(ctypes.byref(d)) == base
    tile_table.set_table([])
    assert L.unit_packed_weights_bytes_conv_i8(ctypes.byref(d)) == base
    bad = (_lib.TileEntry * 1)()
    bad[0].c_in, bad[0].c_block, bad[0].c_out, bad[0].kh, bad[0].kw, bad[0].stride_h, bad[0].stride_w = 64, 16, 80, 1, 1, 2, 2
    bad[0].bn = 40                                                                    # not a multiple of 16
    assert L.unit_tile_table_set(bad, 1) == -2
    assert L.unit_tile_table_set(bad, 5000) == -8
    assert L.unit_tile_table_set(None, 0) == 0


def test_shape_corpus_parser_and_committed_corpus():
    from unit_b200 import tile_table
    lines = ['(1, 4, 58, 58, 16) (4, 4, 3, 3, 4, 16, 4) (1, 1) /some/model.json',
             '(1, 4, 58, 58, 16) (4, 4, 3, 3, 4, 16, 4) (1, 1)',
             '(1, 512) (8, 128, 128, 4) dense /some/model.json',
             '(1, 2, 56, 56, 12) (9, 2, 1, 1, 3, 16, 4) (1, 1)',          # channel block of 12: skipped
             '(1, 16, 14, 14, 16) (32, 16, 1, 1, 4, 16, 4) (2, 2) x', 'noise']
    shapes = tile_table.parse_shape_log(lines)
    assert shapes == [dict(n=1, c_in=64, h=58, w=58, c_out=64, kh=3, kw=3, stride_h=1, stride_w=1, count=2),
                      dict(n=1, c_in=256, h=14, w=14, c_out=512, kh=1, kw=1, stride_h=2, stride_w=2, count=1)]
    corpus = tile_table.load_corpus()
    assert len(corpus) >= 100 and all(s['c_in'] % 16 == 0 and s['c_out'] % 16 == 0 for s in corpus)
