"""The benchmark workloads: seeded inputs, weights and the MinkUNet-style network.

Channel plan (int4 affine, group size 32, fp16 activations): stem SubmConv3d 4->32;
four encoder stages [Conv3d k=2 s=2 + 2 x SubmConv3d k=3] with 32/64/128/256
channels; a mirrored decoder [transposed conv k=2 s=2 onto the saved encoder support
(`coordinates=`), channel concat with the skip tensor, 2 x SubmConv3d]; a 32->20
quantized linear head. Weights ~ N(0, 2/fan_in) from a seeded generator.
"""

from __future__ import annotations

import numpy as np
import torch

from mlx_lattice_b200 import nn, ops, synthetic
from mlx_lattice_b200.core import QuantizedWeight, SparseTensor, quantize_weight

ENCODER_CHANNELS = (32, 64, 128, 256)
STEM_CHANNELS = 32
INPUT_CHANNELS = 4
HEAD_CHANNELS = 20

# (name, kind, kernel, c_in, c_out) in execution order
def minkunet_layers() -> list[tuple[str, str, int, int, int]]:
    layers = [('stem', 'subm', 3, INPUT_CHANNELS, STEM_CHANNELS)]
    c_prev = STEM_CHANNELS
    for i, c in enumerate(ENCODER_CHANNELS, start=1):
        layers.append((f'down{i}', 'down', 2, c_prev, c))
        layers.append((f'enc{i}a', 'subm', 3, c, c))
        layers.append((f'enc{i}b', 'subm', 3, c, c))
        c_prev = c
    skips = (STEM_CHANNELS,) + ENCODER_CHANNELS[:-1]
    for i in range(len(ENCODER_CHANNELS), 0, -1):
        c_skip = skips[i - 1]
        layers.append((f'up{i}', 'up', 2, c_prev, c_skip))
        layers.append((f'dec{i}a', 'subm', 3, 2 * c_skip, c_skip))
        layers.append((f'dec{i}b', 'subm', 3, c_skip, c_skip))
        c_prev = c_skip
    layers.append(('head', 'linear', 1, c_prev, HEAD_CHANNELS))
    return layers


def minkunet_dense_weights(seed: int) -> dict[str, np.ndarray]:
    """fp16 weights: (C_out, k, k, k, C_in) for convs, (C_out, C_in) for the head,
    ~ N(0, 2 / fan_in) with fan_in = C_in * k^3."""
    rng = np.random.default_rng(seed)
    weights = {}
    for name, kind, k, c_in, c_out in minkunet_layers():
        std = np.sqrt(2.0 / (c_in * k ** 3))
        shape = (c_out, c_in) if kind == 'linear' else (c_out, k, k, k, c_in)
        weights[name] = (rng.normal(size=shape) * std).astype(np.float16)
    return weights


def quantize_all(dense: dict[str, np.ndarray], bits: int = 4, group_size: int = 32):
    """Quantise every layer with the package quantiser (on the CPU, set-up time)."""
    return {
        name: quantize_weight(torch.from_numpy(w), group_size=group_size, bits=bits)
        for name, w in dense.items()
    }


def quantized_to(q: QuantizedWeight, device) -> QuantizedWeight:
    return QuantizedWeight(
        q.weight.to(device), q.scales.to(device), q.biases.to(device), q.group_size, q.bits,
        q.in_channels, q.out_channels, q.kernel_size, q.layout,
    )


class MinkUNet:
    """Inference network assembled from the package operators."""

    def __init__(self, quantized: dict[str, QuantizedWeight], device) -> None:
        self.weights = {name: quantized_to(q, device) for name, q in quantized.items()}

    def __call__(self, x: SparseTensor) -> SparseTensor:
        w = self.weights
        skips = [ops.subm_conv3d(x, w['stem'], kernel_size=3)]
        cur = skips[0]
        stages = len(ENCODER_CHANNELS)
        for i in range(1, stages + 1):
            cur = ops.conv3d(cur, w[f'down{i}'], kernel_size=2, stride=2)
            cur = ops.subm_conv3d(cur, w[f'enc{i}a'], kernel_size=3)
            cur = ops.subm_conv3d(cur, w[f'enc{i}b'], kernel_size=3)
            if i < stages:
                skips.append(cur)
        for i in range(stages, 0, -1):
            skip = skips[i - 1]
            cur = ops.conv_transpose3d(cur, w[f'up{i}'], kernel_size=2, stride=2, coordinates=skip)
            cur = ops.sparse_cat_aligned(cur, skip, join='right')
            cur = ops.subm_conv3d(cur, w[f'dec{i}a'], kernel_size=3)
            cur = ops.subm_conv3d(cur, w[f'dec{i}b'], kernel_size=3)
        return ops.linear(cur, w['head'])


def minkunet_artifact(quantized: dict[str, QuantizedWeight], *, target_support: bool = True):
    """The network above as a lattice artifact: ``(manifest, weights)`` for
    ``artifact.save_lattice_artifact`` / ``artifact.LatticeModel``. With
    ``target_support`` the transposed convolutions name the encoder tensor they upsample
    onto (one edge per fine voxel); without it the decoder takes the reference's form, a
    plain transposed convolution followed by a right-join concatenation."""
    from mlx_lattice_b200.artifact import GraphWriter

    g = GraphWriter({'input': 'sparse_tensor'}, producer={'name': 'mlx-lattice-b200-workloads'})
    k3 = {'kernel_size': (3, 3, 3)}
    k2 = {'kernel_size': (2, 2, 2), 'stride': (2, 2, 2)}

    def conv(op, name, source, attributes):
        return g.add(f'sparse.quantized_{op}', {'input': source}, node_id=name,
                     parameters={'weight': quantized[name]}, attributes=attributes)

    cur = conv('subm_conv3d', 'stem', 'input', k3)
    skips = [cur]
    stages = len(ENCODER_CHANNELS)
    for i in range(1, stages + 1):
        cur = conv('conv3d', f'down{i}', cur, k2)
        cur = conv('subm_conv3d', f'enc{i}a', cur, k3)
        cur = conv('subm_conv3d', f'enc{i}b', cur, k3)
        if i < stages:
            skips.append(cur)
    for i in range(stages, 0, -1):
        skip = skips[i - 1]
        cur = conv('conv_transpose3d', f'up{i}', cur,
                   {**k2, 'coordinates': skip} if target_support else k2)
        cur = g.add('ops.sparse_cat_aligned', {'lhs': cur, 'rhs': skip}, node_id=f'cat{i}',
                    attributes={'join': 'right'})
        cur = conv('subm_conv3d', f'dec{i}a', cur, k3)
        cur = conv('subm_conv3d', f'dec{i}b', cur, k3)
    g.add('feature.quantized_linear', {'input': cur}, node_id='head', output='logits',
          parameters={'weight': quantized['head']})
    return g.manifest({'logits': 'sparse_tensor'}), g.weights


def minkunet_inputs(config_index: int, batch: int, per_cloud: int, first_batch: int = 0):
    """LiDAR-like coords (N, 4) int32 and xyz+intensity ~ U(0,1) fp16 features (N, 4)."""
    coords = synthetic.lidar_batch(config_index, batch, per_cloud, first_batch=first_batch)
    rng = np.random.default_rng(synthetic.cloud_seed(config_index, first_batch) + 500000)
    feats = rng.uniform(0.0, 1.0, size=(coords.shape[0], INPUT_CHANNELS)).astype(np.float16)
    return coords, feats


# --------------------------------------------------------------------------- #
# single-kernel cases (python -m mlx_lattice_b200.workloads ...), used for profiling
# --------------------------------------------------------------------------- #


def dense_cloud(rows: int, seed: int = 7) -> np.ndarray:
    """A compact cloud (~45 % occupancy of a cube, ~12 of 27 neighbours per voxel), the
    regime of the coarse U-Net levels."""
    side = int(np.ceil((rows / 0.45) ** (1.0 / 3.0)))
    rng = np.random.default_rng(seed)
    cells = rng.permutation(side ** 3)[:rows]
    xyz = np.stack([cells // (side * side), (cells // side) % side, cells % side], axis=1)
    return np.concatenate([np.zeros((rows, 1), np.int64), xyz], axis=1).astype(np.int32)


def _case_main() -> None:
    import argparse

    from mlx_lattice_b200 import _ext

    parser = argparse.ArgumentParser(description='run one kernel of the hot path repeatedly')
    parser.add_argument('case', choices=('conv', 'map'))
    parser.add_argument('--rows', type=int, default=150000)
    parser.add_argument('--cin', type=int, default=256)
    parser.add_argument('--cout', type=int, default=256)
    parser.add_argument('--bits', type=int, default=4, help='0 = fp16 weights')
    parser.add_argument('--cloud', default='dense', choices=('dense', 'lidar'))
    parser.add_argument('--stride', type=int, default=1)
    parser.add_argument('--iters', type=int, default=3)
    args = parser.parse_args()

    device = torch.device('cuda', 0)
    if args.cloud == 'dense':
        coords_np = dense_cloud(args.rows)
    else:
        coords_np = synthetic.lidar_batch(2, max(1, args.rows // 125000), min(args.rows, 125000))
    coords = torch.from_numpy(coords_np).to(device)
    n = coords.shape[0]
    if args.case == 'map':
        active = torch.tensor([n], dtype=torch.int32, device=device)
        for _ in range(args.iters):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            base, _, _ = _ext.build_kernel_relation_base(coords, active, 3, args.stride, 0, 1)
            end.record()
            torch.cuda.synchronize()
            print(f'map rows={n} stride={args.stride} counts={base[5].tolist()} '
                  f'ms={start.elapsed_time(end):.3f}')
        return
    rng = np.random.default_rng(3)
    feats = torch.from_numpy(rng.normal(size=(n, args.cin)).astype(np.float16)).to(device)
    dense = (rng.normal(size=(args.cout, 3, 3, 3, args.cin)) * 0.05).astype(np.float16)
    weight = torch.from_numpy(dense)
    if args.bits:
        weight = quantized_to(quantize_weight(weight, group_size=32, bits=args.bits), device)
    else:
        weight = weight.to(device)
    x = SparseTensor(coords, feats)
    for _ in range(args.iters):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        y = ops.subm_conv3d(x, weight, kernel_size=3)
        end.record()
        torch.cuda.synchronize()
        rel = x.coord_manager.submanifold_kernel_relation(x.coord_key, kernel_size=3)
        edges = rel.counts.tolist()[0]
        ms = start.elapsed_time(end)
        print(f'conv rows={n} cin={args.cin} cout={args.cout} bits={args.bits} edges={edges} '
              f'ms={ms:.3f} tflops={2.0 * edges * args.cin * args.cout / ms / 1e9:.1f}')
    _ext.check_status(device)
    del y


if __name__ == '__main__':
    _case_main()
