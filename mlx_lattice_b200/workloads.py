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
