"""Benchmark of the sparse-convolution inference hot path on B200.

    python bench.py --gpus N --steps K --warmup W            # this implementation
    python bench.py --impl reference --steps K --warmup W    # reference CPU route
    python bench.py --case conv:3:128:128 --clouds 1         # one kernel, for profiling

Workload (config 4 of the baseline): MinkUNet-style int4 inference on ONE batch of 8
clouds of 120,000 voxels (LiDAR-like synthetic generator, seeded), kernel maps rebuilt in
every step ("cold"). One step = one forward pass over the batch. With N > 1 the 8 clouds
are divided over the ranks by batch element (8/4/2/1 clouds per GPU, no data-path
collective): strong scaling, value = 960,000 voxels * K / max-over-ranks time. The weak
figure (every rank a full batch of its own) is the extra key `weak_scaling`.

Prints ONE JSON line on rank 0. Timing: CUDA events on the stream the kernels are launched
on, L2 flushed between steps, max over ranks. The headline steps are CUDA-graph replays
of the whole forward pass; the per-launch roofline figures come from a second, eager pass
over the same steps.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = 'sparse-conv voxels/sec (MinkUNet int4) + kernel-map Mcoords/s per B200'
CONFIG_INDEX = 4
BATCH = 8
PER_CLOUD = 120000
WEIGHT_SEED = 20264


def load_peaks() -> dict:
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as handle:
            peaks = json.load(handle)
        peaks['source'] = 'measured'
        return peaks
    return {'hbm_gbs': 6650.0, 'bf16_tflops': 1590.0, 'bf16_tflops_sustained': 1400.0,
            'source': 'fallback'}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,'
             'clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
             'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.process = None
        self.lines: list[str] = []
        self.thread = None

    def start(self) -> None:
        try:
            self.process = subprocess.Popen(
                ['nvidia-smi', f'--query-gpu={self.QUERY}', '--format=csv,noheader,nounits',
                 '-i', str(self.gpu_index), '-lms', '100'],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.process = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self) -> None:
        for line in self.process.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.process is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        sm, sm_max, reasons = [], [], set()
        names = ('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap')
        for line in self.lines:
            parts = [p.strip() for p in line.split(',')]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max.append(float(parts[2]))
            except ValueError:
                continue
            for name, value in zip(names, parts[5:9]):
                if value.lower().startswith('active'):
                    reasons.add(name)
        return {
            'sm_mhz': statistics.median(sm) if sm else None,
            'sm_max_mhz': max(sm_max) if sm_max else None,
            'samples': len(sm),
            'reasons': sorted(reasons),
        }


# --------------------------------------------------------------------------- #
# reference CPU route (the checker, timed as a reported baseline)
# --------------------------------------------------------------------------- #


def cpu_reference_step(voxels: int, cloud_index: int = 0) -> dict:
    """One forward of the same network through the reference's own CPU code
    (oracle/_ref when it was built, else the numpy port) over the first `voxels` voxels
    of cloud `cloud_index` of the workload; voxels = PER_CLOUD is one whole cloud. Clouds
    are independent (the batch id is part of every coordinate key), so the cost per voxel
    of one whole cloud is the cost per voxel of the batch."""
    from mlx_lattice_b200 import workloads
    from oracle import pipeline, reference, restatement

    backend = reference if reference.available() else restatement
    kind = 'reference' if reference.available() else 'port'
    coords, feats = workloads.minkunet_inputs(CONFIG_INDEX, 1, PER_CLOUD, first_batch=cloud_index)
    coords, feats = coords[:voxels], feats[:voxels]
    dense = workloads.minkunet_dense_weights(WEIGHT_SEED)
    quantized = {k: pipeline.quantized_to_numpy(v) for k, v in workloads.quantize_all(dense).items()}
    timings: dict = {}
    start = time.perf_counter()
    logits = pipeline.minkunet_forward(
        backend, coords, feats, quantized, workloads.minkunet_layers(), timings)
    seconds = time.perf_counter() - start
    cores = os.cpu_count() or 1
    whole = 'one whole cloud' if voxels >= PER_CLOUD else f'the first {voxels} voxels of one cloud'
    return {
        'value': coords.shape[0] / seconds,
        'unit': 'voxels/s',
        'cores': cores if kind == 'reference' else 1,
        'kind': kind,
        'sample': f'{whole} of the workload ({coords.shape[0]} voxels, cloud {cloud_index}; 1 forward, '
                  f'kernel maps rebuilt), {seconds:.2f} s; conv {timings.get("conv", 0.0):.2f} s, '
                  f'maps {timings.get("relation", 0.0):.2f} s',
        'seconds': seconds,
        'voxels': int(coords.shape[0]),
        'checksum': float(np.abs(logits.astype(np.float32)).sum()),
    }


REFERENCE_ARM_BUDGET_S = 240.0


def run_reference_arm(args) -> None:
    """Rank 0 times the reference CPU route: one untimed pass over a small sample to page the
    library in, then whole clouds of the workload (120,000 voxels each, clouds 0, 1, ..), one
    per timed step, until `--steps` steps are done or the time budget is spent (a whole cloud
    takes tens of seconds on the host's cores)."""
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    cpu_reference_step(4000)
    seconds, voxels, last = 0.0, 0, None
    steps = 0
    while steps < max(args.steps, 1):
        last = cpu_reference_step(PER_CLOUD, cloud_index=steps % BATCH)
        seconds += last['seconds']
        voxels += last['voxels']
        steps += 1
        if seconds + last['seconds'] > REFERENCE_ARM_BUDGET_S:
            break
    value = voxels / seconds
    line = {
        'impl': 'reference',
        'metric': METRIC,
        'value': value,
        'unit': 'voxels/s',
        'n_gpus': args.gpus,
        'steps': steps,
        'steps_requested': args.steps,
        'warmup': 1,
        'ms_per_step': seconds / steps * 1e3,
        'higher_is_better': True,
        'scaling': 'strong',
        'vs_baseline': None,
        'dtype': 'f16',
        'data': 'synthetic',
        'config': {'workload': 'minkunet_int4_8x120k_lidar, one whole 120,000-voxel cloud per step '
                               '(clouds are independent: voxels/s of a cloud is voxels/s of the batch)',
                   'voxels_per_step': PER_CLOUD,
                   'time_budget_s': REFERENCE_ARM_BUDGET_S},
        'cpu_baseline': {'value': value, 'unit': 'voxels/s', 'cores': last['cores'],
                         'kind': last['kind'],
                         'sample': f'{steps} step(s) of one whole cloud each; last: ' + last['sample']},
        'e2e': {'value': value, 'unit': 'voxels/s', 'h2d_bytes_per_step': 0,
                'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------- #
# this implementation
# --------------------------------------------------------------------------- #

# DRAM bytes of a convolution launch over its algorithmic bytes, by input width: ncu captures
# (dram__bytes_read + dram__bytes_write) of the 256->256, 128->128 and 64->64 layers of the
# benchmark network at the benchmark's own size (8 LiDAR-like clouds), summarised in
# profiles/tc_conv_plan_kernel_lidar_layers.md. The excess is the repeated gather of input
# rows that fall out of L2 (each row is read once per edge) and the zero tail of the
# static-capacity output.
DRAM_OVER_ALGORITHMIC = ((256, 4.40), (128, 2.26), (0, 1.08))


def dram_over_algorithmic(c_in: int) -> float:
    return next(ratio for width, ratio in DRAM_OVER_ALGORITHMIC if c_in >= width)


def conv_algorithmic(info, counts) -> tuple[float, float]:
    """(flops, bytes) of one convolution launch: 2*E*C_in*C_out over real edges; bytes =
    active input rows * C_in * s + N_out * C_out * s + weights + 8 bytes per edge."""
    edges, n_out = counts
    c_in, c_out, k = info['c_in'], info['c_out'], info['n_kernels']
    weight_bytes = (k * c_in * c_out * info['bits'] / 8 + 2 * k * (c_in / 32) * c_out * 2
                    if info['bits'] else k * c_in * c_out * 2)
    flops = 2.0 * edges * c_in * c_out
    # input rows read: the output's own rows for a submanifold map; every edge's row for a
    # kernel-2 stride-2 map (one edge per input); at most the output rows for its transpose
    rows_in = n_out if k == 27 or edges <= n_out else min(edges, info['in_rows'])
    bytes_ = rows_in * c_in * 2 + n_out * c_out * 2 + weight_bytes + 8 * edges
    return flops, bytes_


class ConvProfile:
    """Collects per-launch CUDA-event timings of the convolution calls."""

    def __init__(self) -> None:
        self.records = []

    def __call__(self, kind, info, start, end) -> None:
        self.records.append((info, start, end))

    def layers(self, peaks: dict, steps: int) -> list[dict]:
        """Per layer shape (kernel volume, C_in, C_out, edges): launches, mean time, and the
        fraction of BOTH roofs, with the one that binds named."""
        groups: dict = {}
        for info, start, end in self.records:
            counts = tuple(info['counts'].tolist())
            key = (info['n_kernels'], info['c_in'], info['c_out'], counts[0], bool(info['tensor_cores']))
            entry = groups.setdefault(key, {'ms': 0.0, 'launches': 0, 'info': info, 'counts': counts})
            entry['ms'] += start.elapsed_time(end)
            entry['launches'] += 1
        out = []
        for (k, c_in, c_out, edges, tc), entry in groups.items():
            flops, bytes_ = conv_algorithmic(entry['info'], entry['counts'])
            ms = entry['ms'] / entry['launches']
            tflops = flops / ms / 1e9
            gbs = bytes_ / ms / 1e6
            frac_tensor = tflops / peaks['bf16_tflops_sustained']
            frac_hbm = gbs / peaks['hbm_gbs']
            # the roof a perfect kernel would hit first is the one with the longer minimum time
            t_tensor = flops / (peaks['bf16_tflops_sustained'] * 1e12)
            t_hbm = bytes_ / (peaks['hbm_gbs'] * 1e9)
            out.append({
                'layer': f'K{k} {c_in}->{c_out}', 'route': 'tcgen05' if tc else 'cuda cores',
                'edges': edges, 'out_rows': entry['counts'][1],
                'launches_per_step': entry['launches'] / steps, 'ms': ms,
                'tflops': tflops, 'frac_tensor': frac_tensor, 'gb_s': gbs, 'frac_hbm': frac_hbm,
                'bound': 'tensor' if t_tensor >= t_hbm else 'hbm',
                'frac': frac_tensor if t_tensor >= t_hbm else frac_hbm,
            })
        out.sort(key=lambda e: -e['ms'] * e['launches_per_step'])
        return out

    def summarize(self, tensor_cores: bool) -> dict:
        flops = bytes_ = ms = 0.0
        launches = 0
        for info, start, end in self.records:
            if bool(info['tensor_cores']) != tensor_cores:
                continue
            f, b = conv_algorithmic(info, info['counts'].tolist())
            flops += f
            bytes_ += b
            ms += start.elapsed_time(end)
            launches += 1
        return {'flops': flops, 'bytes': bytes_, 'ms': ms, 'launches': launches}


def event_timed(fn, steps: int, flush=None) -> list[float]:
    """CUDA-event time of `steps` calls of fn on the current stream, L2 flushed before each."""
    import torch

    times = []
    for _ in range(steps):
        if flush is not None:
            flush.zero_()
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        end.synchronize()
        times.append(start.elapsed_time(end))
    return times


def kernel_map_benchmark(device, steps: int, peaks: dict, flush) -> dict:
    """Config 2: kernel-map build only, 1,000,000 coords over batch 8 (125k each),
    LiDAR-like generator; kernel_size=3 submanifold map and kernel_size=3 stride=2 map."""
    import torch

    from mlx_lattice_b200 import _ext, synthetic

    coords = torch.from_numpy(synthetic.lidar_batch(2, 8, 125000)).to(device)
    n = coords.shape[0]
    active = torch.tensor([n], dtype=torch.int32, device=device)
    out = {}
    for name, stride in (('subm_k3', 1), ('k3_s2', 2)):
        holder = {}

        def build():
            holder['base'] = _ext.build_kernel_relation_base(coords, active, 3, stride, 0, 1)[0]

        build()
        ms = sum(event_timed(build, steps, flush)) / steps
        edges, n_out = holder['base'][5].tolist()
        slots = 1 << (4 * n - 1).bit_length()
        # HBM-class bytes of one build: coordinates read (16 B/row), table clear and insert
        # (8 B/slot, 8 B/row), the pairs (12 B/edge), row offsets, output coordinates when
        # strided; the zero tail of the three static-capacity edge arrays (27 n entries each)
        # is counted apart; the probes read 32-byte buckets from the table, which lives in
        # L2: one or two per (x, y) column of the footprint, 13.5 per output row on average
        # (the table hashes z in groups of four; ncu: 508 MB from L2 for the 1 M rows of the
        # submanifold map, coordinates and verification loads included).
        useful = n * 16 + 8 * slots + 8 * n + 12 * edges + 4 * (n + 1)
        if stride != 1:
            useful += n * 16 + 8 * slots + 8 * n + 16 * n_out
        tail = 12 * (27 * n - edges)
        probes = int(32 * 13.5 * n_out)
        out[name] = {
            'mcoords_per_s': n / ms / 1e3, 'ms': ms, 'edges': edges, 'out_rows': n_out,
            'hbm_bytes': useful, 'hbm_gb_s': useful / ms / 1e6,
            'frac_of_hbm_peak': useful / ms / 1e6 / peaks['hbm_gbs'],
            'zero_tail_bytes': tail,
            'with_zero_tail_gb_s': (useful + tail) / ms / 1e6,
            'with_zero_tail_frac_of_hbm_peak': (useful + tail) / ms / 1e6 / peaks['hbm_gbs'],
            'l2_probe_bytes': probes, 'l2_probe_gb_s': probes / ms / 1e6,
            'bound': 'instruction issue and the L2 latency of the probes (DRAM busy a few per cent: '
                     'profiles/)',
        }
        del holder
    return out


def front_end_benchmark(device, steps: int, peaks: dict) -> dict:
    """Point -> voxel front end: 2,000,000 points (8 clouds, about two points per voxel at
    voxel size 1), 4 feature channels, sparse_quantize + voxelize_features (mean)."""
    import numpy as np
    import torch

    from mlx_lattice_b200 import _ext, synthetic

    voxels = synthetic.lidar_batch(2, 8, 125000)
    rng = np.random.default_rng(77)
    reps = 2
    base = np.repeat(voxels, reps, axis=0)
    order = rng.permutation(base.shape[0])
    base = base[order]
    batch = torch.from_numpy(np.sort(base[:, 0]).astype(np.int32)).to(device)
    base = base[np.argsort(base[:, 0], kind='stable')]
    points = torch.from_numpy(
        (base[:, 1:].astype(np.float32) + rng.uniform(0.05, 0.95, size=(base.shape[0], 3)).astype(np.float32))
    ).to(device)
    feats = torch.from_numpy(rng.normal(size=(base.shape[0], 4)).astype(np.float32)).to(device)
    n = points.shape[0]
    active = torch.tensor([n], dtype=torch.int32, device=device)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)
    times = []
    count = None
    for i in range(steps + 2):
        flush.zero_()
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record()
        coords, count, inverse, counts = _ext.sparse_quantize(points, batch, active, (1.0, 1.0, 1.0), (0.0, 0.0, 0.0))
        out = _ext.voxelize_features(feats, inverse, counts, active, 'mean')
        end.record()
        torch.cuda.synchronize()
        if i >= 2:
            times.append(start.elapsed_time(end))
        del out
    ms = sum(times) / len(times)
    v = int(count.item())
    cap = 1 << (4 * n - 1).bit_length()
    # HBM-class bytes: points + batch read, table clear + insert, coords/inverse/counts out,
    # features read and voxel rows written (all at capacity n, as the contract sizes them)
    hbm = n * 16 + 8 * cap + 8 * n + n * 16 + n * 8 + n * 16 + n * 16
    return {
        'mpoints_per_s': n / ms / 1e3,
        'ms': ms,
        'points': n,
        'voxels': v,
        'hbm_algorithmic_gb_s': hbm / ms / 1e6,
        'frac_of_hbm_peak': hbm / ms / 1e6 / peaks['hbm_gbs'],
    }



def config_figures(device, steps: int, peaks: dict, flush) -> dict:
    """Event-timed figures of the other benchmark configurations (the headline is configuration 4):
    config 0 (fp32 submanifold conv, 50,000 voxels, 32->32), config 1 (int4 kernel-2 stride-2
    conv 64->128 over 4 x 200,000 voxels) and config 3 (int8 block over 16 x 60,000 voxels),
    kernel maps prebuilt (the map build is config 2's figure)."""
    import torch

    from mlx_lattice_b200 import nn, ops, synthetic, workloads
    from mlx_lattice_b200.core import SparseTensor, quantize_weight

    out = {}
    rng = np.random.default_rng(99)

    def dev(array):
        return torch.from_numpy(np.ascontiguousarray(array)).to(device)

    # ---- config 0 ----
    coords = synthetic.sphere_plane_batch(0, 1, 50000, 256)
    x = SparseTensor(dev(coords), dev(rng.normal(size=(coords.shape[0], 32)).astype(np.float32)))
    w = dev((rng.normal(size=(32, 3, 3, 3, 32)) * 0.05).astype(np.float32))
    ops.subm_conv3d(x, w, kernel_size=3)
    ms = sum(event_timed(lambda: ops.subm_conv3d(x, w, kernel_size=3), steps, flush)) / steps
    rel = x.coord_manager.submanifold_kernel_relation(x.coord_key, kernel_size=3)
    edges, n_out = rel.counts.tolist()
    bytes_ = coords.shape[0] * 32 * 4 * 2 + 27 * 32 * 32 * 4 + 8 * edges
    out['config0_subm_fp32_50k_32x32'] = {
        'ms': ms, 'edges': edges, 'mvoxels_per_s': coords.shape[0] / ms / 1e3,
        'gflops': 2.0 * edges * 32 * 32 / ms / 1e6, 'gb_s': bytes_ / ms / 1e6,
        'frac_of_hbm_peak': bytes_ / ms / 1e6 / peaks['hbm_gbs'], 'bound': 'hbm',
        'route': 'cuda cores (fp32 FMA in the reference summation order)'}

    # ---- config 1 ----
    coords = synthetic.sphere_plane_batch(1, 4, 200000, 512)
    x = SparseTensor(dev(coords), dev(rng.normal(size=(coords.shape[0], 64)).astype(np.float16)))
    dense = torch.from_numpy((rng.normal(size=(128, 2, 2, 2, 64)) * 0.05).astype(np.float16))
    q = workloads.quantized_to(quantize_weight(dense, group_size=32, bits=4), device)
    ops.conv3d(x, q, kernel_size=2, stride=2)
    ms = sum(event_timed(lambda: ops.conv3d(x, q, kernel_size=2, stride=2), steps, flush)) / steps
    rel = x.coord_manager.kernel_relation(x.coord_key, kernel_size=2, stride=2)
    edges, n_out = rel.counts.tolist()
    flops = 2.0 * edges * 64 * 128
    bytes_ = coords.shape[0] * 64 * 2 + n_out * 128 * 2 + 8 * 64 * 128 / 2 + 8 * edges
    t_tensor, t_hbm = flops / (peaks['bf16_tflops_sustained'] * 1e12), bytes_ / (peaks['hbm_gbs'] * 1e9)
    out['config1_strided_int4_4x200k_64x128'] = {
        'ms': ms, 'edges': edges, 'out_rows': n_out, 'mvoxels_per_s': coords.shape[0] / ms / 1e3,
        'tflops': flops / ms / 1e9, 'frac_tensor': flops / ms / 1e9 / peaks['bf16_tflops_sustained'],
        'gb_s': bytes_ / ms / 1e6, 'frac_of_hbm_peak': bytes_ / ms / 1e6 / peaks['hbm_gbs'],
        'bound': 'tensor' if t_tensor >= t_hbm else 'hbm'}

    # ---- config 3 ----
    coords = synthetic.lidar_batch(3, 16, 60000)
    n = coords.shape[0]
    x = SparseTensor(dev(coords), dev(rng.normal(size=(n, 96)).astype(np.float16)),
                     batch_counts=(60000,) * 16)
    dense = torch.from_numpy((rng.normal(size=(96, 3, 3, 3, 96)) * 0.05).astype(np.float16))
    qc = workloads.quantized_to(quantize_weight(dense, group_size=32, bits=8), device)
    ql = workloads.quantized_to(quantize_weight(
        torch.from_numpy((rng.normal(size=(192, 96)) * 0.1).astype(np.float16)), group_size=32, bits=8), device)
    gamma, beta = dev(rng.uniform(0.5, 1.5, 96).astype(np.float16)), dev(rng.normal(size=96).astype(np.float16))
    mean, var = dev(rng.normal(size=96).astype(np.float16) * 0.1), dev(rng.uniform(0.5, 1.5, 96).astype(np.float16))
    parts: dict = {}

    def block():
        # pooling runs in float32 (as in the reference), the linear layer in float16 again
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        marks[0].record()
        y = ops.subm_conv3d(x, qc, kernel_size=3)
        marks[1].record()
        y = ops.batch_norm(y, weight=gamma, bias=beta, mean=mean, var=var, fuse_relu=True)
        marks[2].record()
        pooled = ops.max_pool3d(y.astype(torch.float32), kernel_size=3, stride=2)
        marks[3].record()
        z = ops.linear(pooled.astype(torch.float16), ql)
        marks[4].record()
        parts['marks'] = marks
        return pooled, z

    pooled, z = block()
    n_out = int(pooled.active_rows.item())
    batch_of = pooled.coords[:n_out, 0].cpu().numpy()
    per_cloud = tuple(int(v) for v in np.bincount(batch_of, minlength=16))
    pooled_coords = pooled.coords[:n_out].contiguous()

    def whole():
        _, z = block()
        head = SparseTensor(pooled_coords, z.feats[:n_out].float(), stride=2, batch_counts=per_cloud)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        out_rows = ops.global_avg_pool(head)
        end.record()
        parts['pool'] = (start, end)
        return out_rows

    whole()
    ms = sum(event_timed(whole, steps, flush)) / steps
    torch.cuda.synchronize()
    names = ('subm_conv_int8_96x96', 'batch_norm_relu', 'max_pool_k3_s2_fp32', 'quantized_linear_96x192')
    marks = parts['marks']
    rel = x.coord_manager.submanifold_kernel_relation(x.coord_key, kernel_size=3)
    edges, _ = rel.counts.tolist()
    stage_ms = {name: marks[i].elapsed_time(marks[i + 1]) for i, name in enumerate(names)}
    stage_ms['global_avg_pool'] = parts['pool'][0].elapsed_time(parts['pool'][1])
    pool_bytes = n * 96 * 4 + n_out * 96 * 4 + 4 * 27 * n_out
    out['config3_int8_block_16x60k'] = {
        'ms': ms, 'mvoxels_per_s': n / ms / 1e3, 'conv_edges': edges, 'pooled_rows': n_out,
        'conv_tflops': 2.0 * edges * 96 * 96 / stage_ms['subm_conv_int8_96x96'] / 1e9,
        'max_pool_gb_s': pool_bytes / stage_ms['max_pool_k3_s2_fp32'] / 1e6,
        'max_pool_frac_of_hbm_peak': pool_bytes / stage_ms['max_pool_k3_s2_fp32'] / 1e6 / peaks['hbm_gbs'],
        'linear_tflops': 2.0 * n_out * 96 * 192 / stage_ms['quantized_linear_96x192'] / 1e9,
        'stage_ms': stage_ms,
        'note': 'kernel maps prebuilt and cached by the coordinate manager; stage times include the '
                'dtype casts beside them'}
    return out


def run_gpu_arm(args) -> None:
    import torch

    from mlx_lattice_b200 import _ext, _native, sharding, workloads
    from mlx_lattice_b200.core import SparseTensor

    _native.load()  # no CPU fallback: fail loudly when the extension is missing
    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    if not torch.cuda.is_available():
        raise RuntimeError('bench.py needs a CUDA device (sm_100); there is no CPU route.')
    torch.cuda.set_device(local_rank)
    device = torch.device('cuda', local_rank)
    distributed = world > 1
    if distributed:
        import torch.distributed as dist

        dist.init_process_group('nccl', device_id=device)
    peaks = load_peaks()
    steps, warmup = args.steps, max(args.warmup, 3)
    quantized = workloads.quantize_all(workloads.minkunet_dense_weights(WEIGHT_SEED))
    model = workloads.MinkUNet(quantized, device)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)

    def barrier():
        torch.cuda.synchronize()
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(value: float) -> float:
        if not distributed:
            return value
        t = torch.tensor([value], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    class Shard:
        """The clouds [first, first + count) of the workload on this GPU, their forward pass
        captured in a CUDA graph over fixed input buffers (kernel maps are rebuilt inside)."""

        def __init__(self, first: int, count: int, slots: int = 1) -> None:
            coords_np, feats_np = workloads.minkunet_inputs(CONFIG_INDEX, count, PER_CLOUD, first_batch=first)
            self.voxels = coords_np.shape[0]
            self.batch_counts = (PER_CLOUD,) * count
            self.coords_host = torch.from_numpy(coords_np).pin_memory()
            self.feats_host = torch.from_numpy(feats_np).pin_memory()
            self.inputs = [(self.coords_host.to(device), self.feats_host.to(device)) for _ in range(slots)]
            self.logits_host = [torch.empty((self.voxels, workloads.HEAD_CHANNELS), dtype=torch.float16).pin_memory()
                                for _ in range(slots)]
            self.graphs, self.outputs, self.graph_launches = [], [], 0

        def forward(self, slot: int = 0):
            # a fresh SparseTensor gets a fresh coordinate manager: every kernel map is
            # rebuilt in every step, like the reference does for a new input
            coords, feats = self.inputs[slot]
            return model(SparseTensor(coords, feats, batch_counts=self.batch_counts)).feats

        def capture(self) -> bool:
            try:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    for slot in range(len(self.inputs)):
                        self.forward(slot)
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                for slot in range(len(self.inputs)):
                    graph = torch.cuda.CUDAGraph()
                    before = _ext.launch_count()
                    with torch.cuda.graph(graph):
                        out = self.forward(slot)
                    self.graph_launches = _ext.launch_count() - before
                    self.graphs.append(graph)
                    self.outputs.append(out)
                    graph.replay()
                torch.cuda.synchronize()
                return True
            except Exception as error:  # noqa: BLE001 - fall back to eager launches, and say so
                self.graphs, self.outputs = [], []
                self.capture_error = f'{type(error).__name__}: {error}'
                return False

        def step(self, slot: int = 0):
            if self.graphs:
                self.graphs[slot].replay()
                return self.outputs[slot]
            return self.forward(slot)

    # ---- strong split: ONE 8-cloud batch, clouds divided over the ranks ----
    first, end = sharding.shard_range(BATCH, world, rank)
    shard = Shard(first, end - first, slots=2)
    for _ in range(warmup):
        shard.forward(0)
    torch.cuda.synchronize()
    _ext.check_status(device)
    graphed = False if args.no_graph else shard.capture()
    for _ in range(warmup):
        shard.step(0)
    barrier()

    # ---- timed region 1 (the headline): K steps, inputs resident, L2 flushed between steps ----
    sampler = ClockSampler(local_rank)
    sampler.start()
    wall_start = time.perf_counter()
    launches_before = _ext.launch_count()
    step_ms = event_timed(lambda: shard.step(0), steps, flush)
    barrier()
    wall = time.perf_counter() - wall_start
    launches = (shard.graph_launches * steps) if graphed else _ext.launch_count() - launches_before
    total_ms = max_over_ranks(sum(step_ms))
    value = BATCH * PER_CLOUD * steps / (total_ms / 1e3)

    # ---- timed region 2: the same K steps as eager launches with an event pair around every
    # convolution launch (the roofline figures; the events cannot sit inside a graph) ----
    profile = ConvProfile()
    _ext.profile_hook = profile
    eager_ms = event_timed(lambda: shard.forward(0), steps, flush)
    _ext.profile_hook = None
    barrier()
    eager_total_ms = max_over_ranks(sum(eager_ms))

    # ---- end to end: pinned host buffers in, logits back to the host, every step. The K
    # steps run as a two-slot software pipeline in ONE timed region: the inputs of step i+1
    # travel while step i computes, the logits of step i travel back while step i+1 computes.
    def e2e_pipelined(count: int) -> float:
        main = torch.cuda.current_stream()
        copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
        in_ready = [torch.cuda.Event() for _ in range(2)]
        consumed = [torch.cuda.Event() for _ in range(2)]
        drained = [torch.cuda.Event() for _ in range(2)]

        def prefetch(i: int) -> None:
            slot = i % 2
            with torch.cuda.stream(copy_in):
                copy_in.wait_event(consumed[slot])
                shard.inputs[slot][0].copy_(shard.coords_host, non_blocking=True)
                shard.inputs[slot][1].copy_(shard.feats_host, non_blocking=True)
                in_ready[slot].record(copy_in)

        torch.cuda.synchronize()
        start = torch.cuda.Event(enable_timing=True)
        stop = torch.cuda.Event(enable_timing=True)
        start.record(main)
        copy_in.wait_stream(main)
        copy_out.wait_stream(main)
        prefetch(0)
        for i in range(count):
            slot = i % 2
            if i + 1 < count:
                prefetch(i + 1)
            main.wait_event(in_ready[slot])
            main.wait_event(drained[slot])      # the slot's previous logits have left
            out = shard.step(slot)
            consumed[slot].record(main)
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(done)
                shard.logits_host[slot].copy_(out, non_blocking=True)
                drained[slot].record(copy_out)
        main.wait_stream(copy_out)
        stop.record(main)
        stop.synchronize()
        return start.elapsed_time(stop)

    def e2e_serial(count: int) -> float:
        def one():
            shard.inputs[0][0].copy_(shard.coords_host, non_blocking=True)
            shard.inputs[0][1].copy_(shard.feats_host, non_blocking=True)
            shard.logits_host[0].copy_(shard.step(0), non_blocking=True)
        return sum(event_timed(one, count))

    e2e_pipelined(2)
    barrier()
    e2e_ms = max_over_ranks(e2e_pipelined(steps))
    barrier()
    e2e_serial_ms = max_over_ranks(e2e_serial(steps))
    barrier()
    clocks = sampler.stop()
    _ext.check_status(device)

    # ---- weak scaling (extra key, N > 1): every rank runs a full 8-cloud batch of its own ----
    weak = None
    if distributed:
        del shard.graphs, shard.outputs
        full = Shard(rank * BATCH, BATCH)
        for _ in range(3):
            full.forward(0)
        if not args.no_graph:
            full.capture()
        for _ in range(3):
            full.step(0)
        barrier()
        weak_ms = max_over_ranks(sum(event_timed(lambda: full.step(0), steps, flush)))
        weak = {'value': BATCH * PER_CLOUD * world * steps / (weak_ms / 1e3), 'unit': 'voxels/s',
                'ms_per_step': weak_ms / steps, 'voxels_per_gpu': BATCH * PER_CLOUD,
                'note': 'every rank steps its own 8-cloud batch (clouds 8*rank .. 8*rank+7)'}
        del full
        barrier()

    if rank == 0:
        tc = profile.summarize(tensor_cores=True)
        layers = profile.layers(peaks, steps)
        peak_tf = peaks['bf16_tflops_sustained']
        achieved_tf = tc['flops'] / (tc['ms'] / 1e3) / 1e12 if tc['ms'] > 0 else 0.0
        dram = sum(dram_over_algorithmic(int(e['layer'].split()[1].split('->')[0])) * e['gb_s'] * e['ms'] * 1e6
                   * e['launches_per_step'] for e in layers if e['route'] == 'tcgen05')
        per_step_launches = tc['launches'] / steps
        roofline = {
            'bound': 'tensor',
            'kernel': 'tc_conv_plan_kernel (tcgen05 implicit GEMM, all tensor-core conv launches of the step)',
            'achieved': achieved_tf,
            'peak': peak_tf,
            'unit': 'TFLOP/s',
            'frac': achieved_tf / peak_tf,
            'peak_source': peaks['source'] + ' (dense bf16, sustained)',
            'frac_of_burst_peak': achieved_tf / peaks['bf16_tflops'],
            'traffic': dram / per_step_launches if per_step_launches else None,
            'traffic_note': 'DRAM bytes per launch, mean over the conv launches of a step: each '
                            "layer's algorithmic bytes times the dram/algorithmic ratio that ncu measured "
                            'on the 256-, 128- and 64-channel layers at this size (profiles/)',
            'algorithmic_gb_s': tc['bytes'] / (tc['ms'] / 1e3) / 1e9 if tc['ms'] > 0 else 0.0,
            'launches': tc['launches'],
            'ms_per_step_in_kernel': tc['ms'] / steps,
            'timed_in': 'the eager pass over the same K steps (an event pair per launch)',
            'layers': layers,
        }
        extra_steps = max(min(steps, 10), 3)
        kernel_map = kernel_map_benchmark(device, extra_steps, peaks, flush)
        front_end = front_end_benchmark(device, extra_steps, peaks)
        configs = config_figures(device, extra_steps, peaks, flush)
        line = {
            'metric': METRIC,
            'value': value,
            'unit': 'voxels/s',
            'n_gpus': world,
            'steps': steps,
            'warmup': warmup,
            'ms_per_step': total_ms / steps,
            'higher_is_better': True,
            'scaling': 'strong',
            'vs_baseline': None,
            'dtype': 'f16',
            'data': 'synthetic',
            'config': {
                'workload': 'minkunet_int4_8x120k_lidar',
                'global_batch': f'{BATCH} clouds x {PER_CLOUD} voxels = {BATCH * PER_CLOUD} voxels per step',
                'voxels_per_gpu': shard.voxels,
                'weights': 'int4 affine, group_size 32, N(0, 2/fan_in)',
                'kernel_maps': 'rebuilt every step (cold)',
                'l2': 'flushed between steps (256 MiB write); working set exceeds L2',
                'launch': ('one CUDA graph replay per step (the whole forward incl. kernel-map builds)'
                           if graphed else 'eager launches (' + ('--no-graph' if args.no_graph else
                           'graph capture failed: ' + getattr(shard, 'capture_error', '?')) + ')'),
                'parallelism': f'the 8 clouds sharded over {world} GPU(s) by batch element, '
                               'no data-path collective',
            },
            'eager': {'ms_per_step': eager_total_ms / steps,
                      'value': BATCH * PER_CLOUD * steps / (eager_total_ms / 1e3), 'unit': 'voxels/s',
                      'note': 'the same steps as individual launches from Python, an event pair '
                              'around every convolution'},
            'e2e': {
                'value': BATCH * PER_CLOUD * steps / (e2e_ms / 1e3),
                'unit': 'voxels/s',
                'h2d_bytes_per_step': shard.coords_host.numel() * 4 + shard.feats_host.numel() * 2,
                'd2h_bytes_per_step': shard.logits_host[0].numel() * 2,
                'ms_per_step': e2e_ms / steps,
                'pipeline': 'K steps in one timed region: H2D of step i+1 and D2H of step i overlap the '
                            'compute of their neighbour step (two input/output slots); no L2 flush inside '
                            'the region (the working set of a step exceeds L2); bytes are per rank',
                'serial_ms_per_step': e2e_serial_ms / steps,
            },
            'gpu_launches': launches,
            'gpu_launches_per_step': launches / steps,
            'roofline': roofline,
            'kernel_map': kernel_map,
            'front_end': front_end,
            'configs': configs,
            'weak_scaling': weak,
            'clocks': clocks,
            'wall_s_timed_region': wall,
        }
        if world == 1:
            cpu = cpu_reference_step(PER_CLOUD)
            line['cpu_baseline'] = {k: cpu[k] for k in ('value', 'unit', 'cores', 'kind', 'sample')}
        print(json.dumps(line))
    if distributed:
        dist.barrier()
        dist.destroy_process_group()


# --------------------------------------------------------------------------- #
# single-kernel cases: python bench.py --case <name> (the commands behind profiles/)
# --------------------------------------------------------------------------- #


def level_tensor(device, clouds: int, level: int, channels: int, per_cloud: int = PER_CLOUD,
                 config_index: int = CONFIG_INDEX):
    """Sparse tensor on the coordinates of encoder level `level` of the benchmark network
    (level 0 = input voxels, each further level one kernel-2 stride-2 downsampling) for
    `clouds` LiDAR-like clouds, with seeded N(0,1) fp16 features of `channels` channels."""
    import torch

    from mlx_lattice_b200 import ops, workloads
    from mlx_lattice_b200.core import SparseTensor

    coords_np, _ = workloads.minkunet_inputs(config_index, clouds, per_cloud)
    rng = np.random.default_rng(1234 + level)
    x = SparseTensor(torch.from_numpy(coords_np).to(device),
                     torch.zeros((coords_np.shape[0], 32), dtype=torch.float16, device=device))
    down = torch.zeros((32, 2, 2, 2, 32), dtype=torch.float16, device=device)
    for _ in range(level):
        x = ops.conv3d(x, down, kernel_size=2, stride=2)
    feats = torch.from_numpy(rng.normal(size=(x.capacity, channels)).astype(np.float16)).to(device)
    return x.replace(feats=feats)


def run_case(args) -> None:
    """One kernel of the path on a small, named input, a few times over, printing the
    event time of each repetition: `conv:<level>:<c_in>:<c_out>[:fp16]` (submanifold 3x3x3
    int4 convolution on level `level` of `--clouds` clouds), `down:<level>:<c_in>:<c_out>`
    (kernel-2 stride-2 int4 convolution from that level), `map[:stride]` (kernel map of
    `--clouds` clouds of 125,000 voxels of config 2), `pool` (max_pool3d k3 s2 over
    `--clouds` config-3 clouds of 60,000 voxels, 96 float32 channels)."""
    import torch

    from mlx_lattice_b200 import _ext, _native, ops, synthetic, workloads
    from mlx_lattice_b200.core import SparseTensor, quantize_weight

    _native.load()
    device = torch.device('cuda', 0)
    parts = args.case.split(':')
    kind = parts[0]

    def timed(fn):
        for _ in range(args.iters):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            out = fn()
            end.record()
            torch.cuda.synchronize()
            yield out, start.elapsed_time(end)

    if kind in ('conv', 'down'):
        level, c_in, c_out = int(parts[1]), int(parts[2]), int(parts[3])
        k = 3 if kind == 'conv' else 2
        rng = np.random.default_rng(5)
        dense = torch.from_numpy((rng.normal(size=(c_out, k, k, k, c_in)) * 0.05).astype(np.float16))
        if len(parts) > 4 and parts[4] == 'fp16':
            weight = dense.to(device)
        else:
            weight = workloads.quantized_to(quantize_weight(dense, group_size=32, bits=4), device)
        x = level_tensor(device, args.clouds, level, c_in)
        run = ((lambda: ops.subm_conv3d(x, weight, kernel_size=3)) if kind == 'conv'
               else (lambda: ops.conv3d(x, weight, kernel_size=2, stride=2)))
        for y, ms in timed(run):
            rel = (x.coord_manager.submanifold_kernel_relation(x.coord_key, kernel_size=3)
                   if kind == 'conv' else
                   x.coord_manager.kernel_relation(x.coord_key, kernel_size=2, stride=2))
            edges, n_out = rel.counts.tolist()
            print(f'{args.case} clouds={args.clouds} rows_in={int(x.active_rows.item())} out_rows={n_out} '
                  f'edges={edges} ms={ms:.3f} tflops={2.0 * edges * c_in * c_out / ms / 1e9:.1f}')
    elif kind == 'map':
        stride = int(parts[1]) if len(parts) > 1 else 1
        coords = torch.from_numpy(synthetic.lidar_batch(2, args.clouds, 125000)).to(device)
        n = coords.shape[0]
        active = torch.tensor([n], dtype=torch.int32, device=device)
        for (base, _, _), ms in timed(lambda: _ext.build_kernel_relation_base(coords, active, 3, stride, 0, 1)):
            print(f'{args.case} rows={n} counts={base[5].tolist()} ms={ms:.3f} mcoords_per_s={n / ms / 1e3:.0f}')
    elif kind == 'pool':
        coords_np = synthetic.lidar_batch(3, args.clouds, 60000)
        rng = np.random.default_rng(9)
        feats = torch.from_numpy(rng.normal(size=(coords_np.shape[0], 96)).astype(np.float32)).to(device)
        x = SparseTensor(torch.from_numpy(coords_np).to(device), feats)
        for y, ms in timed(lambda: ops.max_pool3d(x, kernel_size=3, stride=2)):
            print(f'{args.case} rows={x.capacity} out_rows={int(y.active_rows.item())} ms={ms:.3f}')
    else:
        raise SystemExit(f'unknown case {args.case}')
    _ext.check_status(device)


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument('--gpus', type=int, default=1)
    parser.add_argument('--steps', type=int, default=10)
    parser.add_argument('--warmup', type=int, default=3)
    parser.add_argument('--impl', default='ours', choices=('ours', 'reference'))
    parser.add_argument('--no-graph', action='store_true',
                        help='step with individual launches instead of CUDA-graph replays (the form '
                             'the ncu launch list under profiles/ is taken on)')
    parser.add_argument('--case', default=None,
                        help='run one kernel on a small named input instead of the benchmark '
                             '(see run_case); used for the ncu captures under profiles/')
    parser.add_argument('--clouds', type=int, default=1)
    parser.add_argument('--iters', type=int, default=3)
    args = parser.parse_args()
    if args.case is not None:
        run_case(args)
    elif args.impl == 'reference':
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == '__main__':
    main()
