#!/usr/bin/env python
"""Benchmark of the int8 convolution hot path: the ResNet-50 conv-layer sweep.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl unit|reference]

One *step* is one pass over all 53 convolutions of ResNet-50 (u8 activations,
s8 weights, fused bias + requantise to u8, NCHW16c) on a batch of 256 images.
With N GPUs the batch is split 256/N per GPU, weights replicated, no collective
on the data path (strong scaling).  Every convolution instance has its own
input and output buffers (about 5.6 GB per step in total at batch 256), so no
layer finds its data in L2 from an earlier launch.

Prints one JSON line (rank 0).  ``value`` is whole-job TOPS with inputs
resident in HBM; ``e2e`` is the same sweep through the Python operator with
pinned host buffers copied in and results copied out inside the timed region.
On one GPU the line also carries ``configs``: the other configurations of the
baseline (single 3x3 convolution, int8 GEMM 4096^3, the batch-1 and batch-16
sweeps, the fp16 convolution) and the tensor-core peak probe.
``--impl reference`` times the AVX-512 VNNI + OpenMP restatement of the
reference's CPU loop nest on the host cores, on the same batch-256 sweep.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

TOTAL_BATCH = 256
METRIC = 'int8 conv2d TOPS (ResNet-50 conv-layer sweep, batch 256)'
# The reference's own logged time for the config-1 shape (3x3 64->64 @56^2, batch 1) on its CPU
# (cpu-tune.log:160 of were/UNIT: 24.27 us = 9.5 TOPS; hardware inferred as Cascade Lake).
REFERENCE_LOG = {'shape': 'int8 3x3 64->64 @56^2, batch 1', 'us': 24.27, 'tops': 9.53,
                 'source': 'cpu-tune.log:160 (reference log, different hardware)'}


def _peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    try:
        with open(path) as f:
            p = json.load(f)
        return {'hbm_gbs': float(p['hbm_gbs']), 'bf16_burst': float(p['bf16_tflops']),
                'bf16_sustained': float(p.get('bf16_tflops_sustained', p['bf16_tflops'])), 'source': 'measured'}
    except Exception:
        return {'hbm_gbs': 6650.0, 'bf16_burst': 1590.0, 'bf16_sustained': 1400.0, 'source': 'fallback'}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    FIELDS = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,'
              'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,'
              'clocks_event_reasons.sw_power_cap')

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self._stop = threading.Event()
        self._thr = None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(['nvidia-smi', f'--query-gpu={self.FIELDS}', '--format=csv,noheader,nounits',
                                      '-i', str(self.gpu)], capture_output=True, text=True, timeout=5).stdout
                for line in out.strip().splitlines():
                    self.rows.append([t.strip() for t in line.split(',')])
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        self._thr = threading.Thread(target=self._run, daemon=True)
        self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._thr.join(timeout=10)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for i, n in enumerate(names):
                if len(r) > 4 + i and r[4 + i].lower().startswith('active'):
                    reasons.add(n)
        if not sm:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': [], 'samples': 0}
        return {'sm_mhz': statistics.median(sm), 'sm_max_mhz': max(mx), 'reasons': sorted(reasons),
                'samples': len(sm)}


# ---------------------------------------------------------------------------
# CPU legs (the oracle is the thing timed here, never the thing shipped)
# ---------------------------------------------------------------------------
def _host_batch(want: int) -> int:
    """The batch the CPU sweep can hold in host memory (about 16 MB per image for inputs and outputs)."""
    try:
        with open('/proc/meminfo') as f:
            avail_kb = next(int(line.split()[1]) for line in f if line.startswith('MemAvailable'))
    except Exception:
        return want
    b = want
    while b > 8 and b * 16e6 * 1.5 > avail_kb * 1024:
        b //= 2
    return b


class CpuSweep:
    """The VNNI/OpenMP restatement over the 53 convolutions, outputs preallocated (a fresh output
    array per call would be timed as page faults)."""

    def __init__(self, batch: int):
        import numpy as np
        from oracle import c_oracle as co
        from unit_b200 import resnet50 as R
        self.co, self.R, self.batch = co, R, batch
        self.vnni = co.host_has_vnni()
        co.use_all_cores()
        self.cores = int(co.lib().oracle_max_threads())
        self.data = []
        for i, l in enumerate(R.LAYERS):
            x, w, b = R.make_layer_inputs(l, i, batch, config=5)
            out = np.zeros((batch, l.c_out // 16, l.out_hw, l.out_hw, 16), np.uint8)
            self.data.append((l, x, w, b, out))
        self.ops = R.sweep_ops(batch)

    def one_pass(self) -> float:
        t0 = time.perf_counter()
        for l, x, w, b, out in self.data:
            for _ in range(l.count):
                self.co.conv2d_u8s8(x, w, (l.stride, l.stride), (l.pad, l.pad), bias=b, requant_shift=8, vnni=self.vnni,
                                    out=out)
        return time.perf_counter() - t0

    def describe(self) -> str:
        how = 'AVX-512 VNNI + OpenMP' if self.vnni else 'scalar + OpenMP'
        whole = 'the whole batch' if self.batch == TOTAL_BATCH else f'batch {self.batch} of {TOTAL_BATCH} (host memory)'
        return f'all 53 convolutions, {whole}, {how} restatement of the reference loop nest on pre-padded inputs'


def run_reference(args):
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return 0
    sweep = CpuSweep(_host_batch(TOTAL_BATCH))
    for _ in range(args.warmup):
        sweep.one_pass()
    times = [sweep.one_pass() for _ in range(args.steps)]
    dt = sum(times) / len(times)
    tops = sweep.ops / dt / 1e12
    line = {
        'impl': 'reference', 'metric': METRIC, 'value': tops, 'unit': 'TOPS', 'n_gpus': args.gpus,
        'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': dt * 1e3 * TOTAL_BATCH / sweep.batch,
        'higher_is_better': True,
        'scaling': 'strong', 'vs_baseline': None, 'dtype': 'u8*s8->s32', 'data': 'synthetic',
        'config': {'workload': 'resnet50-int8-conv-sweep', 'global_batch': TOTAL_BATCH, 'sample_batch': sweep.batch,
                   'convolutions': 53, 'epilogue': 'bias+requant(shift 8)->u8', 'layout': 'NCHW16c'},
        'cpu_baseline': {'value': tops, 'unit': 'TOPS', 'cores': sweep.cores, 'kind': 'port', 'sample': sweep.describe()},
        'reference_log': REFERENCE_LOG,
        'e2e': {'value': tops, 'unit': 'TOPS', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
    }
    print(json.dumps(line), flush=True)
    return 0


# DRAM traffic per launch, (dram__bytes_read.sum, dram__bytes_write.sum), of every layer shape at
# batch 256 on one GPU: one `ncu --metrics dram__bytes_read.sum,dram__bytes_write.sum,gpu__time_duration.sum
# --clock-control none -k regex:igemm -s <3 x count> -c 1 python bench.py --layer <name> --steps 1
# --warmup 3 --kernels-only` per layer (profiles/igemm_resnet50_dram_traffic_b256.md).  Writes still
# in L2 when the kernel ends are not in the write figure.
NCU_DRAM_B256 = {
    'stem_7x7s2_3_64': (51.5e6, 145.4e6),
    's1_1x1_64_64': (51.5e6, 7.7e6),
    's1_1x1_256_64': (205.6e6, 33.5e6),
    's1_3x3_64_64': (51.5e6, 8.3e6),
    's1_1x1_64_256': (51.5e6, 145.1e6),
    's1_proj_64_256': (51.5e6, 144.9e6),
    's2_1x1_256_128': (205.6e6, 65.8e6),
    's2_3x3s2_128_128': (103.0e6, 10.1e6),
    's2_1x1_512_128': (102.9e6, 6.0e6),
    's2_3x3_128_128': (25.9e6, 0.0e6),
    's2_1x1_128_512': (25.8e6, 42.3e6),
    's2_proj_s2_256_512': (103.0e6, 53.4e6),
    's3_1x1_512_256': (103.0e6, 22.4e6),
    's3_3x3s2_256_256': (52.2e6, 0.3e6),
    's3_1x1_1024_256': (51.7e6, 0.1e6),
    's3_3x3_256_256': (13.5e6, 0.0e6),
    's3_1x1_256_1024': (13.2e6, 1.3e6),
    's3_proj_s2_512_1024': (59.3e6, 11.7e6),
    's4_1x1_1024_512': (52.0e6, 1.8e6),
    's4_3x3s2_512_512': (28.9e6, 0.0e6),
    's4_1x1_2048_512': (26.8e6, 0.0e6),
    's4_3x3_512_512': (8.8e6, 0.0e6),
    's4_1x1_512_2048': (7.5e6, 0.0e6),
    's4_proj_s2_1024_2048': (38.9e6, 0.5e6),
}


def ncu_traffic(name, batch):
    """DRAM bytes of one launch from the ncu capture (only valid at the captured batch)."""
    if batch != TOTAL_BATCH or name not in NCU_DRAM_B256:
        return None
    r, w = NCU_DRAM_B256[name]
    return r + w


def tensor_peak(torch, gpu_index, f16: bool, seconds: float = 0.6):
    """The tensor-core issue-rate probe (unit_tensor_peak), run back to back for `seconds` so that the
    figure is the sustained one under the power cap; clocks sampled beside it."""
    from unit_b200 import _lib
    L = _lib.lib()
    best = None
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    out = ctypes.c_double(0.0)
    for n, issuers in ((256, 1), (256, 2), (128, 4)):
        rc = L.unit_tensor_peak(1 if f16 else 0, n, issuers, 2000, ctypes.byref(out), stream)   # warm-up
        if rc != 0:
            return {'error': f'unit_tensor_peak status {rc}'}
        vals = []
        with ClockSampler(gpu_index) as cs:
            t_end = time.time() + seconds
            while time.time() < t_end:
                rc = L.unit_tensor_peak(1 if f16 else 0, n, issuers, 40000, ctypes.byref(out), stream)
                if rc != 0:
                    return {'error': f'unit_tensor_peak status {rc}'}
                vals.append(out.value / 1e12)
        tail = vals[len(vals) // 2:] or vals
        rec = {'n': n, 'issuers': issuers, 'burst': max(vals), 'sustained': statistics.median(tail),
               'sm_mhz': cs.summary()['sm_mhz'], 'launches': len(vals)}
        if best is None or rec['sustained'] > best['sustained']:
            best = rec
    return best


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
def build_instances(torch, U, R, dev, layer_set, batch, rank, config=5):
    """Packed weights shared per shape; own activations / outputs / plan per convolution instance."""
    gen = torch.Generator(device=dev)
    instances, per_layer = [], []
    for l in layer_set:
        li = R.LAYERS.index(l)
        cb, cs = l.c_block, l.c_in_stored
        gen.manual_seed(R.layer_seed(config, li, 1) + 7919 * rank)
        w = torch.randn((l.c_out // 16, cs // cb, l.k, l.k, cb // 4, 16, 4), device=dev, generator=gen)
        w = (w * 32.0).round_().clamp_(-128, 127).to(torch.int8)
        bias = torch.randint(-2 ** 15, 2 ** 15, (l.c_out,), dtype=torch.int32, device=dev, generator=gen)
        packed = U.pack_conv_weights_int8(w, l.stride, l.pad)
        idxs = []
        for c in range(l.count):
            gen.manual_seed(R.layer_seed(config, li, 0) + 101 * c + 7919 * rank)
            shape = (batch, cs // cb, l.hw, l.hw, cb)
            x = torch.randint(1, 256, shape, dtype=torch.uint8, device=dev, generator=gen)
            x *= torch.randint(0, 2, shape, dtype=torch.uint8, device=dev, generator=gen)
            if cs != l.c_in:
                x[..., l.c_in:] = 0
            out = torch.empty((batch, l.c_out // 16, l.out_hw, l.out_hw, 16), dtype=torch.uint8, device=dev)
            plan = U.conv2d_NCHWc_int8_plan(x, packed, stride=l.stride, padding=l.pad, bias=bias, out_dtype='uint8', out=out)
            idxs.append(len(instances))
            instances.append((l, x, packed, bias, out, plan))
        per_layer.append((l, idxs))
        del w
    return instances, per_layer


def capture_graph(torch, U, fn, warm: int = 1, branches=None):
    """Captures fn() (library launches on the current stream) into a CUDA graph; returns
    (graph, launches per replay).  fn runs once on the capture stream first (one-off set-up of the
    library and of the operators' per-stream scratch must not fall inside a capture).
    `branches`: a list of callables instead of fn, captured as parallel branches of the graph (work
    without data dependencies between the branches)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())

    def body():
        if not branches:
            fn()
            return
        streams = [torch.cuda.Stream() for _ in branches]
        for st, work in zip(streams, branches):
            st.wait_stream(side)
            with torch.cuda.stream(st):
                work()
        for st in streams:
            side.wait_stream(st)

    with torch.cuda.stream(side):
        body()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    c0 = U.launch_count()
    with torch.cuda.graph(graph, stream=side):
        body()
    n = U.launch_count() - c0
    for _ in range(warm):
        graph.replay()
    torch.cuda.synchronize()
    return graph, n


def time_ms(torch, fn, reps: int) -> float:
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps


def side_configs(torch, U, R, dev, peaks, local_rank):
    """The other configurations of the baseline, each a small record {value, unit, ms, frac, peak}
    (one GPU).  Kernels timed alone are set against the burst figures."""
    out = {}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # larger than L2
    i8_burst, f16_burst = 2.0 * peaks['bf16_burst'], peaks['bf16_burst']

    def flushed(fn, reps=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(reps):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            total += a.elapsed_time(b)
        return total / reps

    # config 1: one int8 3x3 64->64 convolution at 56^2, batch 1, s32 out
    torch.manual_seed(1)
    sets = []
    w = torch.randint(-128, 128, (4, 4, 3, 3, 4, 16, 4), dtype=torch.int8, device=dev)
    pw = U.pack_conv_weights_int8(w, 1, 1)
    for _ in range(8):
        x = torch.randint(0, 256, (1, 4, 56, 56, 16), dtype=torch.uint8, device=dev)
        o = torch.empty((1, 4, 56, 56, 16), dtype=torch.int32, device=dev)
        sets.append((x, o, U.conv2d_NCHWc_int8_plan(x, pw, stride=1, padding=1, out=o)))
    for s_ in sets:
        s_[2].run()
    torch.cuda.synchronize()
    eager_us = time_ms(torch, lambda: [s_[2].run() for s_ in sets], 50) * 1e3 / len(sets)
    op_us = time_ms(torch, lambda: [U.conv2d_NCHWc_int8(s_[0], pw, stride=1, padding=1, out=s_[1]) for s_ in sets], 25) * 1e3 / len(sets)
    g, nl = capture_graph(torch, U, lambda: [s_[2].run() for s_ in sets for _ in range(16)])
    graph_us = time_ms(torch, g.replay, 20) * 1e3 / nl
    ops1 = 2.0 * 56 * 56 * 64 * 64 * 9
    out['config1_conv3x3_64_b1'] = {
        'value': eager_us, 'unit': 'us per call (prepared plan, eager launches, 8 buffer sets in turn)',
        'us_python_operator': op_us, 'us_in_cuda_graph': graph_us, 'tops_in_cuda_graph': ops1 / graph_us / 1e6,
        'reference_log_us': REFERENCE_LOG['us'], 'bound': 'launch latency (roofline time 0.13 us)'}
    del sets, g

    # config 2: int8 GEMM 4096^3
    a = torch.randint(0, 256, (4096, 4096), dtype=torch.uint8, device=dev)
    wq = torch.randint(-128, 128, (32, 1024, 128, 4), dtype=torch.int8, device=dev)
    pwd = U.pack_dense_weights_int8(wq)
    c = torch.empty((4096, 4096), dtype=torch.int32, device=dev)
    ms = flushed(lambda: U.dense_dotprod(a, pwd, out=c))
    v = 2.0 * 4096 ** 3 / ms / 1e9
    out['config2_int8_gemm_4096'] = {'value': v, 'unit': 'TOPS', 'ms': ms, 'frac': v / i8_burst, 'peak': i8_burst,
                                     'l2': 'flushed before every call'}
    del a, wq, pwd, c

    # config 4 and the fp16 GEMM
    x = torch.randn((256, 16, 14, 14, 16), dtype=torch.float16, device=dev)
    wf = torch.randn((16, 16, 3, 3, 16, 16), dtype=torch.float16, device=dev) * 0.05
    pwf = U.pack_conv_weights_f16(wf)
    of = U.conv2d_NCHW16c_OHWI16o(x, pwf, 1, 1, padding=1)
    ms = flushed(lambda: U.conv2d_NCHW16c_OHWI16o(x, pwf, 1, 1, padding=1, out=of))
    v = 2.0 * 256 * 14 * 14 * 256 * 256 * 9 / ms / 1e9
    out['config4_fp16_conv_b256'] = {'value': v, 'unit': 'TFLOP/s', 'ms': ms, 'frac': v / f16_burst, 'peak': f16_burst,
                                     'l2': 'flushed before every call'}
    del x, wf, pwf, of
    a = torch.randn((4096, 4096), dtype=torch.float16, device=dev)
    b = torch.randn((4096, 4096), dtype=torch.float16, device=dev) * 0.05
    pwg = U.pack_gemm_weights_f16(b)
    c = torch.empty((4096, 4096), dtype=torch.float32, device=dev)
    ms = flushed(lambda: U.gemm_f16f32(a, pwg, out=c))
    v = 2.0 * 4096 ** 3 / ms / 1e9
    out['fp16_gemm_4096'] = {'value': v, 'unit': 'TFLOP/s', 'ms': ms, 'frac': v / f16_burst, 'peak': f16_burst,
                             'l2': 'flushed before every call'}
    del a, b, pwg, c

    # config 3: the sweep at batch 1 and 16, as a replayed CUDA graph of the 54 launches.  The sweep's
    # convolutions do not depend on one another, and at these sizes most of them fill a fraction of the
    # SMs: six parallel branches of the graph let them share the GPU (the single chain is reported beside it)
    for bsz in (1, 16):
        inst, _ = build_instances(torch, U, R, dev, R.LAYERS, bsz, 0, config=3)
        g, nl = capture_graph(torch, U, lambda: [i[5].run() for i in inst], warm=3)
        ms_chain = time_ms(torch, g.replay, 20)
        del g
        lanes = [inst[k::6] for k in range(6)]
        g, nl = capture_graph(torch, U, lambda: [i[5].run() for i in inst], warm=1,
                              branches=[(lambda ls=ls: [i[5].run() for i in ls]) for ls in lanes])
        ms = time_ms(torch, g.replay, 20)
        eager_ms = time_ms(torch, lambda: [i[5].run() for i in inst], 5)
        ops = R.sweep_ops(bsz)
        out[f'config3_sweep_b{bsz}'] = {'value': ops / ms / 1e9, 'unit': 'TOPS', 'ms': ms, 'launches': nl,
                                        'us_per_launch': ms * 1e3 / nl, 'ms_single_chain': ms_chain, 'ms_eager_plans': eager_ms,
                                        'launch_mode': 'cuda graph replay, six parallel branches'}
        del inst, g

    # int8 conv3d: the reference's workload list (apps/cpu/kernel/conv3d.py:13-25, depth 16, valid
    # convolution on pre-padded sizes; the 4-channel stem of that list needs NCDHW4c and is left out),
    # one launch each, L2 flushed; the reference's own CPU log beside it (apps/cpu/kernel/res, GOPS
    # counted as in conv3d.py:92: one operation per 4-byte group multiply-accumulate)
    workloads = [(256, 16, 16, 256, 3, 1), (512, 9, 9, 512, 3, 1), (128, 30, 30, 128, 3, 1), (64, 56, 56, 128, 1, 2),
                 (64, 58, 58, 64, 3, 1), (128, 28, 28, 256, 1, 2), (256, 16, 16, 512, 3, 2), (64, 58, 58, 128, 3, 2),
                 (128, 30, 30, 256, 3, 2), (256, 14, 14, 512, 1, 2)]
    rows, t_sum, ops_sum = [], 0.0, 0.0
    for ic, h, w_, oc, k, st in workloads:
        x3 = torch.randint(0, 256, (1, ic // 16, 16, h, w_, 16), dtype=torch.uint8, device=dev)
        w3 = torch.randint(-128, 128, (oc // 16, ic // 16, k, k, k, 4, 16, 4), dtype=torch.int8, device=dev)
        pw3 = U.pack_conv3d_weights_int8(w3, st)
        o3 = U.conv3d_NCDHWc_int8(x3, pw3, stride=st)
        ms3 = flushed(lambda: U.conv3d_NCDHWc_int8(x3, pw3, stride=st, out=o3), reps=10)
        ops3 = 2.0 * o3.numel() * ic * k ** 3
        rows.append([f'{ic}x16x{h}x{w_}->{oc} k{k} s{st}', round(ms3 * 1e3, 2), round(ops3 / ms3 / 1e9, 1)])
        t_sum += ms3
        ops_sum += ops3
        del x3, w3, pw3, o3
    out['conv3d_reference_workloads'] = {'value': ops_sum / t_sum / 1e9, 'unit': 'TOPS over the ten workloads', 'ms': t_sum,
                                         'rows': rows, 'row_format': '[workload, us, TOPS]',
                                         'reference_log': 'apps/cpu/kernel/res: 797-1170 us for the 3x3x3 stride-1 workloads on its CPU'}

    # the reference's own fused graph operator on signed activations, multiply(add(conv2d(x s8, w s8), bias), 11)
    # in s32 (apps/cpu/relay/conv2d.py:16-23), on its logged shape (apps/cpu/relay/result.log:3: 1x1 1024->2048
    # at 16x16), at the logged batch 1 and at batch 256; one launch each (the tensor core takes s8 x s8 as it is)
    gen = torch.Generator(device=dev).manual_seed(78)
    wr = torch.randint(-128, 128, (128, 64, 1, 1, 4, 16, 4), dtype=torch.int8, device=dev, generator=gen)
    br = torch.randint(-2 ** 14, 2 ** 14, (2048,), dtype=torch.int32, device=dev, generator=gen)
    pwr = U.pack_conv_weights_int8(wr, 1, 0)
    relay_rows = {}
    for nb_ in (1, 256):
        xr = torch.randint(-128, 128, (nb_, 64, 16, 16, 16), dtype=torch.int8, device=dev, generator=gen)
        orr = torch.empty((nb_, 128, 16, 16, 16), dtype=torch.int32, device=dev)
        plr = U.conv2d_NCHWc_int8_plan(xr, pwr, bias=br, mul=11, out=orr)
        ms_r = flushed(plr.run, 10)
        relay_rows[f'b{nb_}'] = {'us': ms_r * 1e3, 'tops': 2.0 * nb_ * 256 * 2048 * 1024 / ms_r / 1e9}
        del plr, xr, orr
    out['relay_flow_s8_1x1_1024_2048'] = {'value': relay_rows['b256']['tops'], 'unit': 'TOPS at batch 256', 'ms': relay_rows['b256']['us'] / 1e3,
                                          'us_b1': relay_rows['b1']['us'], 'tops_b1': relay_rows['b1']['tops'],
                                          'what': '(conv(x s8, w s8) + bias) * 11 in s32, 1x1 1024->2048 at 16x16, L2 flushed'}
    del wr, pwr

    # a residual block chained in layout (u8 NCHW16c in, u8 NCHW16c out, no repack between the layers; the
    # reference's graph flow, apps/cpu/relay/result.log:30-36): the first bottleneck of ResNet-50's stage 1 at
    # batch 256: 1x1 256->64, 3x3 64->64, 1x1 64->256 with the block's input added before the clamp (ReLU);
    # every layer reads the previous one's output; one captured graph of the three launches, L2 flushed
    nb, hw = 256, 56
    gen = torch.Generator(device=dev).manual_seed(77)
    xb = torch.randint(0, 256, (nb, 16, hw, hw, 16), dtype=torch.uint8, device=dev, generator=gen)
    ws = [(torch.randn(shape, device=dev, generator=gen) * 12).round_().clamp_(-128, 127).to(torch.int8)
          for shape in ((4, 16, 1, 1, 4, 16, 4), (4, 4, 3, 3, 4, 16, 4), (16, 4, 1, 1, 4, 16, 4))]
    bs = [torch.randint(-2 ** 12, 2 ** 12, (c,), dtype=torch.int32, device=dev, generator=gen) for c in (64, 64, 256)]
    pws = [U.pack_conv_weights_int8(w_, 1, pad_) for w_, pad_ in zip(ws, (0, 1, 0))]
    y1 = torch.empty((nb, 4, hw, hw, 16), dtype=torch.uint8, device=dev)
    y2 = torch.empty_like(y1)
    y3 = torch.empty_like(xb)
    block = [U.conv2d_NCHWc_int8_plan(xb, pws[0], bias=bs[0], out_dtype='uint8', out=y1),
             U.conv2d_NCHWc_int8_plan(y1, pws[1], padding=1, bias=bs[1], out_dtype='uint8', out=y2),
             U.conv2d_NCHWc_int8_plan(y2, pws[2], bias=bs[2], out_dtype='uint8', residual=xb, out=y3)]
    gb, _ = capture_graph(torch, U, lambda: [pl.run() for pl in block], warm=3)
    ms_b = flushed(gb.replay, 10)
    ops_b = 2.0 * nb * hw * hw * (256 * 64 + 64 * 64 * 9 + 64 * 256)
    bytes_b = 2.0 * xb.numel() + y3.numel() + 4.0 * y1.numel()   # the input twice (conv and residual), the output, y1 and y2 written and read
    out['residual_block_chained_b256'] = {'value': ops_b / ms_b / 1e9, 'unit': 'TOPS', 'ms': ms_b, 'gbs': bytes_b / ms_b / 1e6,
                                          'layers': '1x1 256->64, 3x3 64->64, 1x1 64->256 + residual + ReLU, shift 8, 56x56, batch 256',
                                          'hbm_peak_gbs': peaks['hbm_gbs']}
    del gb, block, xb, y1, y2, y3, ws, pws

    # layout kernels (NCHW <-> NCHW16c): GB/s of bytes read + written
    xl = torch.randint(0, 256, (64, 256, 56, 56), dtype=torch.uint8, device=dev)
    yl = U.pack_data_nchwc(xl)
    # (L2 is flushed before every call: source and result together, 102 MB, would otherwise stay in it)
    ms_p = flushed(lambda: U.pack_data_nchwc(xl), 10)
    ms_u = flushed(lambda: U.unpack_data_nchwc(yl), 10)
    out['layout_kernels'] = {'nchw_to_nchw16c_gbs': 2 * xl.numel() / ms_p / 1e6, 'nchw16c_to_nchw_gbs': 2 * xl.numel() / ms_u / 1e6,
                             'tensor': 'u8 (64, 256, 56, 56), 51 MB each way', 'l2': 'flushed before every call', 'hbm_peak_gbs': peaks['hbm_gbs']}
    del xl, yl, flush

    # tensor-core peak, measured
    out['tensor_peak'] = {'i8_tops': tensor_peak(torch, local_rank, False), 'f16_tflops': tensor_peak(torch, local_rank, True),
                          'how': 'unit_tensor_peak: back-to-back tcgen05.mma 128 x n x 32 B from `issuers` threads per SM, '
                                 'operands resident in shared memory; sustained = median of the second half of 0.6 s'}
    return out


def run_unit(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit('launch with torch.distributed.run --nproc-per-node N for --gpus N')
    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device: the unit_b200 operators have no CPU fallback')
    torch.cuda.set_device(local_rank)
    dev = torch.device('cuda', local_rank)
    if world > 1:
        dist.init_process_group('nccl', device_id=dev)

    import unit_b200 as U
    from unit_b200 import resnet50 as R

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    if args.total_batch % world:
        raise SystemExit('--gpus must divide the batch')
    batch = args.total_batch // world

    layer_set = [l for l in R.LAYERS if not args.layer or l.name in args.layer]
    if not layer_set:
        raise SystemExit('no such layer; names: ' + ', '.join(l.name for l in R.LAYERS))
    instances, per_layer = build_instances(torch, U, R, dev, layer_set, batch, rank)
    U.device_status()

    def step():
        for inst in instances:
            inst[5].run()

    # ---- device-resident timing
    for _ in range(args.warmup):
        step()
    barrier()
    # One step = 54 launches of a few tens of microseconds: replay them as a CUDA graph so that
    # the host's per-call work is not what is measured.
    graph = None
    launches_per_step = None
    n_branches = max(1, args.branches)
    if not args.no_graph and not args.kernels_only:
        try:
            branches = None
            if n_branches > 1:
                # the step's convolutions are independent of one another (own buffers each): deal them to
                # parallel branches of the graph, so that one kernel's launch, prologue and tail overlap
                # another's main loop.  Contiguous runs of the sweep per branch: the early layers' full
                # grids then run beside the late layers' under-filled ones (measured against dealing the
                # layers alternately: -1.5 % at batch 256, -4 % at batch 32, -5 % at batch 64)
                per = (len(instances) + n_branches - 1) // n_branches
                lanes = [instances[k * per:(k + 1) * per] for k in range(n_branches)]
                branches = [(lambda ls=ls: [i[5].run() for i in ls]) for ls in lanes]
            graph, launches_per_step = capture_graph(torch, U, step, warm=args.warmup, branches=branches)
        except Exception as exc:  # keep measuring, say how
            print(f'[bench] CUDA graph capture failed ({exc!r}); timing eager launches', file=sys.stderr)
            graph, launches_per_step = None, None

    def timed_step():
        if graph is not None:
            graph.replay()
        else:
            step()

    barrier()
    n0 = U.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as cs_:
        e0.record()
        for _ in range(args.steps):
            timed_step()
        e1.record()
        barrier()
        launches = (launches_per_step * args.steps) if graph is not None else (U.launch_count() - n0)
        # nvidia-smi needs ~0.1 s per sample: when the timed region was shorter than a few
        # samples, keep the same load running (untimed) until the sampler has seen it
        t_end = time.time() + 1.5
        extended = False
        while len(cs_.rows) < 6 and time.time() < t_end:
            extended = True
            timed_step()
            torch.cuda.synchronize()
    ms_step = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    U.device_status()
    # the same step as one chain of launches (no parallel branches), for comparison
    ms_chain = None
    if graph is not None and n_branches > 1:
        g1, _ = capture_graph(torch, U, step, warm=args.warmup)
        barrier()
        ms_chain = max_over_ranks(time_ms(torch, g1.replay, args.steps))
        del g1
    total_ops = sum(l.ops(args.total_batch) * l.count for l in layer_set)
    value = total_ops / (ms_step * 1e-3) / 1e12
    clocks = cs_.summary()
    clocks['sampled'] = 'timed region plus the same load continued untimed' if extended else 'timed region'
    gpu_launches = int(launches)

    # ---- per-layer timing (explains the number; not part of `value`): the step's launches in
    # their order, eager through the prepared plans, an event after each layer's instances, so
    # that every launch meets the cold L2 it meets in the timed step
    peaks = _peaks()
    int8_peak = 2.0 * peaks['bf16_sustained']
    layer_rows = []
    sum_kernel_ms = 0.0
    sum_roof_ms = 0.0
    if not args.kernels_only:
        reps = max(3, min(args.steps, 10))
        acc = [0.0] * len(per_layer)
        for _ in range(reps):
            evs = [torch.cuda.Event(enable_timing=True) for _ in range(len(per_layer) + 1)]
            evs[0].record()
            for k, (l, idxs) in enumerate(per_layer):
                for i in idxs:
                    instances[i][5].run()
                evs[k + 1].record()
            torch.cuda.synchronize()
            for k in range(len(per_layer)):
                acc[k] += evs[k].elapsed_time(evs[k + 1])
        for k, (l, idxs) in enumerate(per_layer):
            ms = acc[k] / reps / len(idxs)
            ops, byts = l.ops(batch), l.bytes(batch)
            t_tensor = ops / (int8_peak * 1e12) * 1e3
            t_hbm = byts / (peaks['hbm_gbs'] * 1e9) * 1e3
            bound = 'tensor' if t_tensor >= t_hbm else 'hbm'
            roof = max(t_tensor, t_hbm)
            sum_kernel_ms += ms * len(idxs)
            sum_roof_ms += roof * len(idxs)
            layer_rows.append({'layer': l.name, 'count': l.count, 'us': round(ms * 1e3, 2),
                               'tops': round(ops / ms / 1e9, 1), 'gbs': round(byts / ms / 1e6, 1), 'bound': bound,
                               'frac': round(roof / ms, 3),
                               'traffic': ncu_traffic(l.name, batch), 'algorithmic_bytes': byts})
    else:
        sum_kernel_ms, sum_roof_ms = ms_step, None
    kernel_tops = total_ops / world / (sum_kernel_ms * 1e-3) / 1e12

    e2e_value = e2e_ms = None
    h2d = d2h = 0
    e2e_steps = 0
    # ---- end-to-end: pinned host buffers in, results out, through the Python operator
    if not args.kernels_only:
        e2e_steps = max(1, min(args.steps, args.e2e_steps))
        host_in, host_out = {}, {}
        for li, (l, idxs) in enumerate(per_layer):
            x, out = instances[idxs[0]][1], instances[idxs[0]][4]
            host_in[li] = torch.empty(x.shape, dtype=x.dtype, pin_memory=True)
            host_in[li].copy_(x)
            host_out[li] = torch.empty(out.shape, dtype=out.dtype, pin_memory=True)
            h2d += x.numel() * len(idxs)
            d2h += out.numel() * len(idxs)
        torch.cuda.synchronize()

        # Three streams: inputs up, convolutions, results down.  PCIe moves both directions at
        # once, so the step costs about max(H2D, D2H) instead of their sum; every instance has its
        # own device buffers, and the streams join at the end of a step.
        s_in, s_run, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()

        def e2e_step():
            main = torch.cuda.current_stream()
            for s_ in (s_in, s_run, s_out):
                s_.wait_stream(main)
            for li, (l, idxs) in enumerate(per_layer):
                for i in idxs:
                    _, x, packed, bias, out, _plan = instances[i]
                    with torch.cuda.stream(s_in):
                        x.copy_(host_in[li], non_blocking=True)
                        up = torch.cuda.Event()
                        up.record(s_in)
                    with torch.cuda.stream(s_run):
                        s_run.wait_event(up)
                        U.conv2d_NCHWc_int8(x, packed, stride=l.stride, padding=l.pad, bias=bias, out_dtype='uint8', out=out)
                        done = torch.cuda.Event()
                        done.record(s_run)
                    with torch.cuda.stream(s_out):
                        s_out.wait_event(done)
                        host_out[li].copy_(out, non_blocking=True)
            for s_ in (s_in, s_run, s_out):
                main.wait_stream(s_)

        e2e_step()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(e2e_steps):
            e2e_step()
        b.record()
        barrier()
        e2e_ms = max_over_ranks(a.elapsed_time(b) / e2e_steps)
        e2e_value = total_ops / (e2e_ms * 1e-3) / 1e12
        U.device_status()
        del host_in, host_out

    # ---- the other configurations and the measured tensor peak (one GPU only)
    configs = None
    single = rank == 0 and world == 1 and not args.kernels_only and not args.layer and args.total_batch == TOTAL_BATCH
    if single and not args.no_side_configs:
        del instances, graph
        instances, graph = [], None
        torch.cuda.empty_cache()
        try:
            configs = side_configs(torch, U, R, dev, peaks, local_rank)
        except Exception as exc:
            configs = {'error': repr(exc)}
        U.device_status()

    # ---- host-CPU baseline beside it (rank 0, single-GPU runs only)
    cpu = None
    if single and not args.no_cpu_baseline:
        sweep = CpuSweep(_host_batch(TOTAL_BATCH))
        sweep.one_pass()  # warm-up
        times = []
        t_start = time.perf_counter()
        while len(times) < 30 and (len(times) < 3 or time.perf_counter() - t_start < 12.0):
            times.append(sweep.one_pass())
        cpu = {'value': sweep.ops / statistics.median(times) / 1e12, 'unit': 'TOPS', 'cores': sweep.cores, 'kind': 'port',
               'sample': f'{sweep.describe()}; {len(times)} passes, median', 'reference_log': REFERENCE_LOG}

    if rank == 0:
        n_launch = sum(l.count for l in layer_set)
        peak_measured = None
        if configs and isinstance(configs.get('tensor_peak', {}).get('i8_tops'), dict) and 'sustained' in configs['tensor_peak']['i8_tops']:
            peak_measured = configs['tensor_peak']['i8_tops']['sustained']
        line = {
            'metric': METRIC, 'value': value, 'unit': 'TOPS', 'n_gpus': world, 'steps': args.steps,
            'warmup': args.warmup, 'ms_per_step': ms_step, 'higher_is_better': True, 'scaling': 'strong',
            'vs_baseline': None, 'dtype': 'u8*s8->s32', 'data': 'synthetic',
            'config': {'workload': 'resnet50-int8-conv-sweep' + ('' if not args.layer else ':' + '+'.join(args.layer)),
                       'global_batch': args.total_batch, 'per_gpu_batch': batch,
                       'convolutions': n_launch, 'epilogue': 'bias+requant(shift 8)->u8', 'layout': 'NCHW16c',
                       'parallelism': f'batch-split x{world}, weights replicated, no collective',
                       'l2': 'every convolution instance has its own buffers; %.2f GB touched per step per GPU, '
                             'larger than L2' % (sum(l.bytes(batch) * l.count for l in layer_set) / 1e9)},
            'clocks': clocks,
            'e2e': {'value': e2e_value, 'unit': 'TOPS', 'h2d_bytes_per_step': h2d * world, 'd2h_bytes_per_step': d2h * world,
                    'ms_per_step': e2e_ms, 'steps': e2e_steps},
            'gpu_launches': gpu_launches,
            'single_chain': None if ms_chain is None else {'ms_per_step': ms_chain, 'value': total_ops / (ms_chain * 1e-3) / 1e12,
                                                            'note': 'the same 54 launches captured as one chain'},
            'launch_mode': ('cuda graph: one captured step (%d kernel launches%s) replayed per timed step'
                            % (launches_per_step, '' if n_branches == 1 else
                               ', dealt to %d parallel branches: the convolutions of the sweep do not depend on one another' % n_branches))
            if launches_per_step is not None else 'eager launches of prepared plans',
            'roofline': {'bound': 'tensor', 'achieved': kernel_tops, 'peak': int8_peak, 'unit': 'TOPS',
                         'frac': kernel_tops / int8_peak,
                         # the same fraction over the timed graph replays (the step's launches overlap their tails)
                         'frac_of_step': total_ops / world / (ms_step * 1e-3) / 1e12 / int8_peak,
                         'traffic': (sum(ncu_traffic(l.name, batch) * l.count for l in layer_set) / n_launch)
                         if batch == TOTAL_BATCH else None,
                         'peak_source': f'2 x bf16_tflops_sustained of {peaks["source"]} peaks '
                                        '(dense int8 issues at twice the bf16 rate)',
                         'peak_measured': peak_measured,
                         'frac_of_peak_measured': (kernel_tops / peak_measured) if peak_measured else None,
                         'kernel': 'igemm_kernel<A_CONV_BOX|A_CONV_WIN|A_CONV_TMA, EPI_REQ_NCHWC, i8> over the contraction launches '
                                   'of one step (2 x ops / summed per-layer launch time, CUDA events)',
                         'traffic_note': 'mean DRAM bytes per launch over the 53 launches of a step (ncu, one capture per '
                                         'layer shape at batch 256); algorithmic mean %.1f MB'
                                         % (sum(l.bytes(batch) * l.count for l in layer_set) / n_launch / 1e6),
                         'mixed_bound_frac': (sum_roof_ms / sum_kernel_ms) if sum_roof_ms else None,
                         'hbm_peak_gbs': peaks['hbm_gbs'],
                         # per layer: [name, count, us per launch, bound, fraction of that bound's roofline]
                         'layers': [[r['layer'], r['count'], r['us'], r['bound'], r['frac']] for r in layer_rows]},
            'configs': configs,
            'cpu_baseline': cpu,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


def run_side_config(args):
    """One of the other configurations alone (for profiler runs), one JSON line:
    `gemm` = int8 GEMM 4096^3 (config 2), `fp16conv` = fp16 3x3 256->256 @14^2, N = 256 (config 4),
    `fp16gemm` = fp16 GEMM 4096^3, `peak` = the tensor-core peak probe, `layout` = the layout kernels."""
    import torch
    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device: the unit_b200 operators have no CPU fallback')
    import unit_b200 as U
    dev = torch.device('cuda', 0)
    torch.manual_seed(0)
    peaks = _peaks()
    if args.config == 'peak':
        print(json.dumps({'metric': 'tensor-core peak probe', 'i8_tops': tensor_peak(torch, 0, False),
                          'f16_tflops': tensor_peak(torch, 0, True)}), flush=True)
        return 0
    if args.config == 'layout':
        x = torch.randint(0, 256, (64, 256, 56, 56), dtype=torch.uint8, device=dev)
        y = U.pack_data_nchwc(x)
        ms_p = time_ms(torch, lambda: U.pack_data_nchwc(x), args.steps)
        ms_u = time_ms(torch, lambda: U.unpack_data_nchwc(y), args.steps)
        print(json.dumps({'metric': 'layout kernels, u8 (64, 256, 56, 56)', 'nchw_to_nchw16c_gbs': 2 * x.numel() / ms_p / 1e6,
                          'nchw16c_to_nchw_gbs': 2 * x.numel() / ms_u / 1e6}), flush=True)
        return 0
    if args.config == 'gemm':
        a = torch.randint(0, 256, (4096, 4096), dtype=torch.uint8, device=dev)
        w = torch.randint(-128, 128, (32, 1024, 128, 4), dtype=torch.int8, device=dev)
        pw = U.pack_dense_weights_int8(w)
        out = torch.empty((4096, 4096), dtype=torch.int32, device=dev)
        fn = lambda: U.dense_dotprod(a, pw, out=out)
        ops, unit, peak, what = 2.0 * 4096 ** 3, 'TOPS', 2.0 * peaks['bf16_burst'], 'int8 GEMM 4096^3 (u8 x s8 -> s32)'
    elif args.config == 'fp16gemm':
        a = torch.randn((4096, 4096), dtype=torch.float16, device=dev)
        b = torch.randn((4096, 4096), dtype=torch.float16, device=dev) * 0.05
        pw = U.pack_gemm_weights_f16(b)
        out = torch.empty((4096, 4096), dtype=torch.float32, device=dev)
        fn = lambda: U.gemm_f16f32(a, pw, out=out)
        ops, unit, peak, what = 2.0 * 4096 ** 3, 'TFLOP/s', peaks['bf16_burst'], 'fp16 GEMM 4096^3 (fp32 accumulate)'
    elif args.config == 'resblock':
        # the chained residual block of `configs.residual_block_chained_b256`, three launches per call
        nb, hw = 256, 56
        gen = torch.Generator(device=dev).manual_seed(77)
        xb = torch.randint(0, 256, (nb, 16, hw, hw, 16), dtype=torch.uint8, device=dev, generator=gen)
        ws = [(torch.randn(shape, device=dev, generator=gen) * 12).round_().clamp_(-128, 127).to(torch.int8)
              for shape in ((4, 16, 1, 1, 4, 16, 4), (4, 4, 3, 3, 4, 16, 4), (16, 4, 1, 1, 4, 16, 4))]
        bs = [torch.randint(-2 ** 12, 2 ** 12, (c,), dtype=torch.int32, device=dev, generator=gen) for c in (64, 64, 256)]
        pws = [U.pack_conv_weights_int8(w_, 1, pad_) for w_, pad_ in zip(ws, (0, 1, 0))]
        y1 = torch.empty((nb, 4, hw, hw, 16), dtype=torch.uint8, device=dev)
        y2, y3 = torch.empty_like(y1), torch.empty_like(xb)
        block = [U.conv2d_NCHWc_int8_plan(xb, pws[0], bias=bs[0], out_dtype='uint8', out=y1),
                 U.conv2d_NCHWc_int8_plan(y1, pws[1], padding=1, bias=bs[1], out_dtype='uint8', out=y2),
                 U.conv2d_NCHWc_int8_plan(y2, pws[2], bias=bs[2], out_dtype='uint8', residual=xb, out=y3)]
        fn = lambda: [pl.run() for pl in block]
        ops, unit, peak = 2.0 * nb * hw * hw * (256 * 64 + 64 * 64 * 9 + 64 * 256), 'TOPS', 2.0 * peaks['bf16_burst']
        what = 'residual block chained in layout: 1x1 256->64, 3x3 64->64, 1x1 64->256 + residual + ReLU @56^2, N = 256'
    elif args.config == 'relay':
        # the signed fused graph operator of `configs.relay_flow_s8_1x1_1024_2048` at batch 256
        gen = torch.Generator(device=dev).manual_seed(78)
        w = torch.randint(-128, 128, (128, 64, 1, 1, 4, 16, 4), dtype=torch.int8, device=dev, generator=gen)
        br = torch.randint(-2 ** 14, 2 ** 14, (2048,), dtype=torch.int32, device=dev, generator=gen)
        pw = U.pack_conv_weights_int8(w, 1, 0)
        x = torch.randint(-128, 128, (256, 64, 16, 16, 16), dtype=torch.int8, device=dev, generator=gen)
        out = torch.empty((256, 128, 16, 16, 16), dtype=torch.int32, device=dev)
        plr = U.conv2d_NCHWc_int8_plan(x, pw, bias=br, mul=11, out=out)
        fn = plr.run
        ops, unit, peak = 2.0 * 256 * 256 * 2048 * 1024, 'TOPS', 2.0 * peaks['bf16_burst']
        what = '(conv(x s8, w s8) + bias) * 11 in s32, 1x1 1024->2048 @16^2, N = 256'
    else:
        x = torch.randn((256, 16, 14, 14, 16), dtype=torch.float16, device=dev)
        w = torch.randn((16, 16, 3, 3, 16, 16), dtype=torch.float16, device=dev) * 0.05
        pw = U.pack_conv_weights_f16(w)
        out = U.conv2d_NCHW16c_OHWI16o(x, pw, 1, 1, padding=1)
        fn = lambda: U.conv2d_NCHW16c_OHWI16o(x, pw, 1, 1, padding=1, out=out)
        ops, unit, peak, what = 2.0 * 256 * 14 * 14 * 256 * 256 * 9, 'TFLOP/s', peaks['bf16_burst'], \
            'fp16 conv2d 3x3 256->256 @14^2, N = 256 (fp32 accumulate)'
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # larger than L2
    for _ in range(max(3, args.warmup)):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(args.steps):
        if not args.kernels_only:
            flush.zero_()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        fn()
        a1.record()
        torch.cuda.synchronize()
        total += a0.elapsed_time(a1)
    U.device_status()
    ms = total / args.steps
    value = ops / (ms * 1e-3) / 1e12
    print(json.dumps({'metric': what, 'value': value, 'unit': unit, 'n_gpus': 1, 'steps': args.steps, 'warmup': max(3, args.warmup),
                      'ms_per_step': ms, 'higher_is_better': True, 'data': 'synthetic',
                      'config': {'workload': args.config, 'l2': 'a 256 MiB buffer is rewritten before every timed call'},
                      'roofline': {'bound': 'tensor', 'achieved': value, 'peak': peak, 'unit': unit, 'frac': value / peak,
                                   'peak_source': f'{peaks["source"]} burst bf16 figure (doubled for int8)'}}), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--config', default=None, choices=['gemm', 'fp16gemm', 'fp16conv', 'peak', 'layout', 'resblock', 'relay'],
                    help='time one of the other configurations alone instead of the conv sweep (single GPU)')
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='unit', choices=['unit', 'reference'])
    ap.add_argument('--e2e-steps', type=int, default=2)
    ap.add_argument('--total-batch', type=int, default=TOTAL_BATCH,
                    help='global batch (diagnostic runs; the metric is quoted on 256)')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-side-configs', action='store_true', help='skip the `configs` records (single-GPU runs)')
    ap.add_argument('--no-graph', action='store_true', help='time eager launches instead of replaying a captured step')
    ap.add_argument('--branches', type=int, default=2,
                    help='deal the step\'s (mutually independent) convolutions to this many parallel branches of the captured graph')
    ap.add_argument('--layer', action='append', default=None,
                    help='restrict the sweep to the named layer(s) of unit_b200.resnet50.LAYERS (diagnostic runs; '
                         'the JSON line then describes that subset)')
    ap.add_argument('--kernels-only', action='store_true',
                    help='timed region only: skip the per-layer pass, the end-to-end leg, the other configurations and '
                         'the CPU baseline (for profiler runs)')
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == 'unit':
        args.warmup = 3
    if args.impl == 'reference':
        return run_reference(args)
    if args.config:
        return run_side_config(args)
    return run_unit(args)


if __name__ == '__main__':
    sys.exit(main())
