"""Benchmark of the sparse-convolution inference hot path on B200.

    python bench.py --gpus N --steps K --warmup W            # this implementation
    python bench.py --impl reference --steps K --warmup W    # reference CPU route

Workload (config 4 of the baseline): MinkUNet-style int4 inference on 8 clouds of
120,000 voxels per GPU (LiDAR-like synthetic generator, seeded), kernel maps rebuilt
in every step ("cold"). One step = one forward pass over the batch. With N > 1 every
rank runs its own 8-cloud batch (independent clouds shard with no data-path
collective): weak scaling, value = voxels of all ranks / max-over-ranks time.

Prints ONE JSON line on rank 0 (see the keys below). Timing: CUDA events on the
stream the kernels are launched on, L2 flushed between steps, max over ranks.
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


def quantized_to_numpy(q) -> dict:
    """Package QuantizedWeight (CPU tensors) -> the dict form the oracle consumes."""
    return {
        'weight': q.weight.numpy().view(np.uint32),
        'scales': q.scales.numpy(),
        'biases': q.biases.numpy(),
        'group_size': q.group_size,
        'bits': q.bits,
        'in_channels': q.in_channels,
        'out_channels': q.out_channels,
        'kernel_size': q.kernel_size,
        'layout': q.layout,
        'storage_in_channels': q.storage_in_channels,
    }


# --------------------------------------------------------------------------- #
# reference CPU route (the checker, timed as a reported baseline)
# --------------------------------------------------------------------------- #


def cpu_reference_step(sample_voxels: int, cloud_index: int = 0) -> dict:
    """One forward of the same network through the reference's own CPU code
    (oracle/_ref when it was built, else the numpy port) on a bounded sample: the
    first `sample_voxels` voxels of one cloud of the workload."""
    import torch

    from mlx_lattice_b200 import workloads
    from oracle import pipeline, reference, restatement

    backend = reference if reference.available() else restatement
    kind = 'reference' if reference.available() else 'port'
    coords, feats = workloads.minkunet_inputs(CONFIG_INDEX, 1, PER_CLOUD, first_batch=cloud_index)
    coords, feats = coords[:sample_voxels], feats[:sample_voxels]
    dense = workloads.minkunet_dense_weights(WEIGHT_SEED)
    quantized = {k: quantized_to_numpy(v) for k, v in workloads.quantize_all(dense).items()}
    timings: dict = {}
    start = time.perf_counter()
    logits = pipeline.minkunet_forward(
        backend, coords, feats, quantized, workloads.minkunet_layers(), timings)
    seconds = time.perf_counter() - start
    cores = os.cpu_count() or 1
    return {
        'value': sample_voxels / seconds,
        'unit': 'voxels/s',
        'cores': cores if kind == 'reference' else 1,
        'kind': kind,
        'sample': f'{sample_voxels} voxels of cloud {cloud_index} (1 forward, kernel maps rebuilt), '
                  f'{seconds:.2f} s; conv {timings.get("conv", 0.0):.2f} s, '
                  f'maps {timings.get("relation", 0.0):.2f} s',
        'seconds': seconds,
        'checksum': float(np.abs(logits.astype(np.float32)).sum()),
        'torch_threads': torch.get_num_threads(),
    }


def run_reference_arm(args) -> None:
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    sample = args.cpu_sample
    times = []
    last = None
    for i in range(args.warmup + args.steps):
        last = cpu_reference_step(sample)
        if i >= args.warmup:
            times.append(last['seconds'])
    mean = sum(times) / len(times)
    value = sample / mean
    line = {
        'impl': 'reference',
        'metric': METRIC,
        'value': value,
        'unit': 'voxels/s',
        'n_gpus': args.gpus,
        'steps': args.steps,
        'warmup': args.warmup,
        'ms_per_step': mean * 1e3,
        'higher_is_better': True,
        'scaling': 'weak',
        'vs_baseline': None,
        'dtype': 'f16',
        'data': 'synthetic',
        'config': {'workload': 'minkunet_int4_8x120k_lidar (bounded sample per step)',
                   'sample_voxels': sample},
        'cpu_baseline': {'value': value, 'unit': 'voxels/s', 'cores': last['cores'],
                         'kind': last['kind'], 'sample': last['sample']},
        'e2e': {'value': value, 'unit': 'voxels/s', 'h2d_bytes_per_step': 0,
                'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------- #
# this implementation
# --------------------------------------------------------------------------- #


DRAM_READ_PER_GATHER_BYTE = 0.56  # dram__bytes_read / (E * C_in * 2), ncu, both captured cases


class ConvProfile:
    """Collects per-launch CUDA-event timings of the convolution calls."""

    def __init__(self) -> None:
        self.records = []

    def __call__(self, kind, info, start, end) -> None:
        self.records.append((info, start, end))

    def summarize(self, tensor_cores: bool) -> dict:
        """Algorithmic flops (2 * E * C_in * C_out, real edges only) and bytes of the
        launches on one route, with their summed event durations."""
        flops = 0.0
        bytes_ = 0.0
        dram = 0.0
        ms = 0.0
        launches = 0
        for info, start, end in self.records:
            if bool(info['tensor_cores']) != tensor_cores:
                continue
            counts = info['counts'].tolist()
            edges, n_out = counts[0], counts[1]
            c_in, c_out, k = info['c_in'], info['c_out'], info['n_kernels']
            flops += 2.0 * edges * c_in * c_out
            weight_bytes = (k * c_in * c_out * info['bits'] / 8 + 2 * k * (c_in / 32) * c_out * 2
                            if info['bits'] else k * c_in * c_out * 2)
            bytes_ += info['in_rows'] * c_in * 2 + n_out * c_out * 2 + weight_bytes + 8 * edges
            # DRAM bytes of a launch, from ncu captures of this kernel on two smaller cases
            # (profiles/tc_conv_plan_kernel_dense_256x256_and_128x128.md): reads are 0.56 x
            # the gathered feature bytes in both (L2 absorbs the rest), writes are the output
            dram += DRAM_READ_PER_GATHER_BYTE * edges * c_in * 2 + n_out * c_out * 2
            ms += start.elapsed_time(end)
            launches += 1
        return {'flops': flops, 'bytes': bytes_, 'dram': dram, 'ms': ms, 'launches': launches}


def kernel_map_benchmark(device, steps: int, peaks: dict) -> dict:
    """Config 2: kernel-map build only, 1,000,000 coords over batch 8 (125k each),
    LiDAR-like generator; kernel_size=3 submanifold map and kernel_size=3 stride=2 map."""
    import torch

    from mlx_lattice_b200 import _ext, synthetic

    coords_host = synthetic.lidar_batch(2, 8, 125000)
    coords = torch.from_numpy(coords_host).to(device)
    n = coords.shape[0]
    active = torch.tensor([n], dtype=torch.int32, device=device)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)
    out = {}
    for name, stride in (('subm_k3', 1), ('k3_s2', 2)):
        times = []
        counts = None
        for i in range(steps + 2):
            flush.zero_()
            start = torch.cuda.Event(enable_timing=True)
            end = torch.cuda.Event(enable_timing=True)
            start.record()
            base, _, _ = _ext.build_kernel_relation_base(coords, active, 3, stride, 0, 1)
            end.record()
            torch.cuda.synchronize()
            if i >= 2:
                times.append(start.elapsed_time(end))
            counts = base[5].tolist()
            del base
        ms = sum(times) / len(times)
        edges, n_out = counts
        cap = 1 << (4 * n - 1).bit_length()
        # algorithmic bytes per build: coord read, clear + insert of the 8-byte-slot table,
        # one 32-byte bucket per probe, edge arrays, row offsets (+ output-support pass
        # when strided)
        # the three edge arrays are outputs of static capacity n * 27 that the contract
        # defines everywhere (pairs, then a zero tail): every byte of them is written
        hbm = n * 16 + 8 * cap + 8 * n + 12 * n * 27 + 4 * (n + 1)
        if stride != 1:
            hbm += n * 16 + 8 * cap + 8 * n + 16 * n_out
        probes = 32 * 27 * n_out  # table reads, served by L2 (the table is 8 * cap bytes)
        algo = hbm + probes
        out[name] = {
            'mcoords_per_s': n / ms / 1e3,
            'ms': ms,
            'edges': edges,
            'out_rows': n_out,
            'algorithmic_gb_s': algo / ms / 1e6,
            'hbm_algorithmic_gb_s': hbm / ms / 1e6,
            'frac_of_hbm_peak': hbm / ms / 1e6 / peaks['hbm_gbs'],
        }
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


def run_gpu_arm(args) -> None:
    import torch

    from mlx_lattice_b200 import _ext, _native, workloads
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

    # ---- workload: this rank's 8 clouds (global batch ids rank*8 .. rank*8+7) ----
    coords_np, feats_np = workloads.minkunet_inputs(
        CONFIG_INDEX, BATCH, PER_CLOUD, first_batch=rank * BATCH)
    voxels = coords_np.shape[0]
    coords_host = torch.from_numpy(coords_np).pin_memory()
    feats_host = torch.from_numpy(feats_np).pin_memory()
    quantized = workloads.quantize_all(workloads.minkunet_dense_weights(WEIGHT_SEED))
    model = workloads.MinkUNet(quantized, device)
    coords_dev = coords_host.to(device)
    feats_dev = feats_host.to(device)
    logits_host = torch.empty((voxels, workloads.HEAD_CHANNELS), dtype=torch.float16).pin_memory()
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)
    batch_counts = (PER_CLOUD,) * BATCH

    def forward(coords, feats):
        # a fresh SparseTensor gets a fresh coordinate manager: every kernel map is
        # rebuilt in every step, like the reference does for a new input
        return model(SparseTensor(coords, feats, batch_counts=batch_counts)).feats

    def barrier():
        torch.cuda.synchronize()
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    def timed_steps(step_fn, steps):
        times = []
        for _ in range(steps):
            flush.zero_()
            start = torch.cuda.Event(enable_timing=True)
            end = torch.cuda.Event(enable_timing=True)
            start.record()
            step_fn()
            end.record()
            end.synchronize()
            times.append(start.elapsed_time(end))
        return times

    def resident_step():
        return forward(coords_dev, feats_dev)

    def e2e_step():
        c = coords_host.to(device, non_blocking=True)
        f = feats_host.to(device, non_blocking=True)
        logits_host.copy_(forward(c, f), non_blocking=True)

    for _ in range(max(args.warmup, 3)):
        resident_step()
    torch.cuda.synchronize()
    _ext.check_status(device)

    # ---- timed region: K resident steps, convolution launches bracketed by events ----
    profile = ConvProfile()
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    launches_before = _ext.launch_count()
    _ext.profile_hook = profile
    wall_start = time.perf_counter()
    step_ms = timed_steps(resident_step, args.steps)
    barrier()
    wall = time.perf_counter() - wall_start
    _ext.profile_hook = None
    launches = _ext.launch_count() - launches_before
    total_ms = sum(step_ms)

    # ---- the same step captured once in a CUDA graph and replayed (informational) ----
    graph_ms = None
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            resident_step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            resident_step()
        graph.replay()
        torch.cuda.synchronize()
        graph_ms = sum(timed_steps(graph.replay, args.steps)) / args.steps
        del graph
    except Exception:  # noqa: BLE001 - capture support is optional for the headline number
        graph_ms = None
    barrier()

    # ---- end to end: pinned host buffers in, logits back to the host, every step ----
    for _ in range(2):
        e2e_step()
    barrier()
    e2e_serial_ms = sum(timed_steps(e2e_step, args.steps))
    barrier()

    # The same K end-to-end steps as a software pipeline, timed as one region: the inputs
    # of step i+1 travel on a copy stream while step i computes, the logits of step i
    # travel back while step i+1 computes. Every step's H2D and D2H is inside the region.
    def e2e_pipelined(steps: int) -> float:
        main = torch.cuda.current_stream()
        copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
        dev_in = [(torch.empty_like(coords_dev), torch.empty_like(feats_dev)) for _ in range(2)]
        host_out = [torch.empty_like(logits_host).pin_memory() for _ in range(2)]
        in_ready = [torch.cuda.Event() for _ in range(2)]
        consumed = [torch.cuda.Event() for _ in range(2)]

        def prefetch(i: int) -> None:
            slot = i % 2
            with torch.cuda.stream(copy_in):
                copy_in.wait_event(consumed[slot])
                dev_in[slot][0].copy_(coords_host, non_blocking=True)
                dev_in[slot][1].copy_(feats_host, non_blocking=True)
                in_ready[slot].record(copy_in)

        flush.zero_()
        torch.cuda.synchronize()
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record(main)
        copy_in.wait_stream(main)
        copy_out.wait_stream(main)
        prefetch(0)
        for i in range(steps):
            slot = i % 2
            if i + 1 < steps:
                prefetch(i + 1)
            main.wait_event(in_ready[slot])
            out = forward(dev_in[slot][0], dev_in[slot][1])
            consumed[slot].record(main)
            step_done = torch.cuda.Event()
            step_done.record(main)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(step_done)
                host_out[slot].copy_(out, non_blocking=True)
                out.record_stream(copy_out)
        main.wait_stream(copy_out)
        end.record(main)
        end.synchronize()
        return start.elapsed_time(end)

    e2e_pipelined(2)
    barrier()
    e2e_ms = e2e_pipelined(args.steps)
    barrier()
    clocks = sampler.stop()
    _ext.check_status(device)

    if distributed:
        stats = torch.tensor([total_ms, e2e_ms, e2e_serial_ms], dtype=torch.float64, device=device)
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        total_ms, e2e_ms, e2e_serial_ms = stats.tolist()
    value = voxels * world * args.steps / (total_ms / 1e3)
    e2e_value = voxels * world * args.steps / (e2e_ms / 1e3)

    if rank == 0:
        tc = profile.summarize(tensor_cores=True)
        peak_tf = peaks['bf16_tflops_sustained']
        achieved_tf = tc['flops'] / (tc['ms'] / 1e3) / 1e12 if tc['ms'] > 0 else 0.0
        roofline = {
            'bound': 'tensor',
            'kernel': 'tc_conv_plan_kernel (tcgen05 implicit GEMM, all conv layers of the step)',
            'achieved': achieved_tf,
            'peak': peak_tf,
            'unit': 'TFLOP/s',
            'frac': achieved_tf / peak_tf,
            'peak_source': peaks['source'] + ' (dense bf16, sustained)',
            'traffic': tc['dram'] / tc['launches'] if tc['launches'] else None,
            'traffic_note': 'DRAM bytes per launch (mean over the conv launches), scaled from ncu '
                            'captures of two smaller cases by gathered bytes',
            'algorithmic_gb_s': tc['bytes'] / (tc['ms'] / 1e3) / 1e9 if tc['ms'] > 0 else 0.0,
            'launches': tc['launches'],
            'ms_per_step_in_kernel': tc['ms'] / args.steps,
        }
        kernel_map = kernel_map_benchmark(device, max(args.steps, 3), peaks)
        front_end = front_end_benchmark(device, max(args.steps, 3), peaks)
        cpu = cpu_reference_step(args.cpu_sample)
        line = {
            'metric': METRIC,
            'value': value,
            'unit': 'voxels/s',
            'n_gpus': world,
            'steps': args.steps,
            'warmup': max(args.warmup, 3),
            'ms_per_step': total_ms / args.steps,
            'higher_is_better': True,
            'scaling': 'weak',
            'vs_baseline': None,
            'dtype': 'f16',
            'data': 'synthetic',
            'config': {
                'workload': 'minkunet_int4_8x120k_lidar',
                'voxels_per_gpu': voxels,
                'weights': 'int4 affine, group_size 32, N(0, 2/fan_in)',
                'kernel_maps': 'rebuilt every step (cold)',
                'l2': 'flushed between steps (256 MiB write); working set exceeds L2',
                'parallelism': f'batch-sharded x{world}, no data-path collective',
            },
            'e2e': {
                'value': e2e_value,
                'unit': 'voxels/s',
                'h2d_bytes_per_step': coords_host.numel() * 4 + feats_host.numel() * 2,
                'd2h_bytes_per_step': logits_host.numel() * 2,
                'ms_per_step': e2e_ms / args.steps,
                'pipeline': 'K steps in one timed region: H2D of step i+1 and D2H of step i '
                            'overlap the compute of their neighbour step; no L2 flush inside the region '
                            '(the working set of a step exceeds L2)',
                'serial_ms_per_step': e2e_serial_ms / args.steps,
            },
            'gpu_launches': launches,
            'roofline': roofline,
            'kernel_map': kernel_map,
            'front_end': front_end,
            'cuda_graph_replay': None if graph_ms is None else {
                'ms_per_step': graph_ms, 'value': voxels * world / (graph_ms / 1e3), 'unit': 'voxels/s'},
            'cpu_baseline': {k: cpu[k] for k in ('value', 'unit', 'cores', 'kind', 'sample')},
            'clocks': clocks,
            'wall_s_timed_region': wall,
        }
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
    `--clouds` clouds of 125,000 voxels of config 2), `pool` (max_pool3d k3 s2 over one
    config-3 cloud, 96 channels)."""
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
        feats = torch.from_numpy(rng.normal(size=(coords_np.shape[0], 96)).astype(np.float16)).to(device)
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
    parser.add_argument('--cpu-sample', type=int, default=8000,
                        help='voxels of one cloud the CPU reference leg processes')
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
