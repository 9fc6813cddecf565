"""Whole-path parity: the operator/module surface (conv3d, subm_conv3d,
conv_transpose3d with coordinates=, max_pool3d, QuantizedLinear, global pooling) on
the GPU against the reference composition evaluated by the CPU oracle."""

import numpy as np
import pytest
import torch

from oracle.pipeline import quantized_to_numpy
from mlx_lattice_b200 import synthetic

pytestmark = pytest.mark.gpu


def _max_rel_err(got, want):
    want = np.asarray(want, np.float64)
    return np.abs(np.asarray(got, np.float64) - want).max() / max(np.abs(want).max(), 1e-30)


@pytest.mark.parametrize('clouds,per', [(2, 5000), (1, 120000)],
                         ids=['two_small_clouds', 'config4_one_whole_cloud'])
def test_minkunet_int4_matches_reference_composition(cuda, oracle, clouds, per):
    """Benchmark configuration 4: the MinkUNet-style int4 network against the reference composition
    evaluated by the oracle; the second case is one cloud of the benchmark batch at its
    full size (120,000 voxels; the clouds of a batch are independent)."""
    from mlx_lattice_b200 import _ext, workloads
    from mlx_lattice_b200.core import SparseTensor
    from oracle import pipeline

    coords, feats = workloads.minkunet_inputs(4, clouds, per)
    quantized = workloads.quantize_all(workloads.minkunet_dense_weights(20264))
    model = workloads.MinkUNet(quantized, cuda)
    x = SparseTensor(torch.from_numpy(coords).to(cuda), torch.from_numpy(feats).to(cuda),
                     batch_counts=(per,) * clouds)
    out = model(x)
    assert out.same_coords(x)
    logits = out.feats.cpu().numpy()
    _ext.check_status()
    want = pipeline.minkunet_forward(
        oracle, coords, feats, {k: quantized_to_numpy(v) for k, v in quantized.items()},
        workloads.minkunet_layers())
    assert logits.shape == want.shape == (clouds * per, 20)
    assert _max_rel_err(logits, want) <= 2e-3
    # deterministic: a second forward (fresh maps) is bitwise identical
    again = model(SparseTensor(torch.from_numpy(coords).to(cuda), torch.from_numpy(feats).to(cuda)))
    assert np.array_equal(again.feats.cpu().numpy(), logits)


@pytest.mark.parametrize('clouds,per', [(3, 4000), (1, 60000)],
                         ids=['three_small_clouds', 'config3_one_whole_cloud'])
def test_mixed_int8_block_config3_shape(cuda, oracle, restatement, clouds, per):
    """Benchmark configuration 3: SubmConv3d int8 96->96, BatchNorm, ReLU, max_pool3d(k3, s2),
    QuantizedLinear int8 96->192, global_avg_pool, with the dtype plumbing the reference
    allows (pooling in float32); the second case is one cloud at its full size."""
    from mlx_lattice_b200 import _ext, nn, ops
    from mlx_lattice_b200.core import SparseTensor

    rng = np.random.default_rng(20263)
    coords = synthetic.lidar_batch(3, clouds, per)
    n = coords.shape[0]
    feats = rng.normal(size=(n, 96)).astype(np.float16)
    conv = nn.SubmConv3d(96, 96, kernel_size=3, bias=False)
    conv.weight = torch.from_numpy((rng.normal(size=(96, 3, 3, 3, 96)) * 0.05).astype(np.float16))
    qconv = nn.QuantizedSubmConv3d.from_conv(conv, group_size=32, bits=8).to(cuda)
    bn = nn.BatchNorm(96, fuse_relu=True)
    bn.running_mean = torch.from_numpy((rng.normal(size=96) * 0.1).astype(np.float16))
    bn.running_var = torch.from_numpy(rng.uniform(0.5, 1.5, size=96).astype(np.float16))
    bn.weight, bn.bias = torch.ones(96, dtype=torch.float16), torch.zeros(96, dtype=torch.float16)
    bn.to(cuda)
    lin = nn.Linear(96, 192, bias=False)
    lin.weight = torch.from_numpy((rng.normal(size=(192, 96)) * 0.05).astype(np.float16))
    qlin = nn.QuantizedLinear.from_linear(lin, group_size=32, bits=8).to(cuda)

    x = SparseTensor(torch.from_numpy(coords).to(cuda), torch.from_numpy(feats).to(cuda),
                     batch_counts=(per,) * clouds)
    y = bn(qconv(x))
    pooled = ops.max_pool3d(y.astype(torch.float32), kernel_size=3, stride=2)
    z = qlin(pooled.astype(torch.float16)).astype(torch.float32)
    n_out = int(pooled.active_rows.item())
    _ext.check_status()

    # oracle
    rel = oracle.build_submanifold_kernel_relation(coords)
    q = quantized_to_numpy(qconv._quantized_weight().__class__(
        qconv.weight.cpu(), qconv.scales.cpu(), qconv.biases.cpu(), 32, 8, 96, 96, (3, 3, 3), 'dense_5d'))
    c = oracle.sparse_quantized_conv(feats, q['weight'], q['scales'], q['biases'], rel, n, 27,
                                     96, 96, 96, 32, 8)
    c = restatement.relu(restatement.batch_norm(
        c, bn.weight.cpu().numpy(), bn.bias.cpu().numpy(), bn.running_mean.cpu().numpy(),
        bn.running_var.cpu().numpy(), 1e-5))
    assert _max_rel_err(y.feats.cpu().numpy(), c) <= 2e-3
    prel = oracle.build_kernel_relation(coords, None, kernel_size=3, stride=2)
    assert int(prel['counts'][1]) == n_out
    assert np.array_equal(pooled.coords.cpu().numpy()[:n_out], prel['out_coords'][:n_out])
    # pool the GPU's own conv output so that the max is compared exactly
    p = oracle.sparse_pool(y.feats.float().cpu().numpy(), prel, input_exclusive=False,
                           reduce='max', out_capacity=n, n_kernels=27)
    assert np.array_equal(pooled.feats.cpu().numpy(), p)
    ql = quantized_to_numpy(qlin._quantized_weight().__class__(
        qlin.weight.cpu(), qlin.scales.cpu(), qlin.biases.cpu(), 32, 8, 96, 192, (1, 1, 1), 'linear'))
    want = restatement.quantized_matmul(p[:n_out].astype(np.float16), ql)
    assert _max_rel_err(z.feats.cpu().numpy()[:n_out], want) <= 2e-3
    # global average over the active rows of each cloud (batch ids are sorted)
    batch_of = prel['out_coords'][:n_out, 0]
    counts = tuple(int((batch_of == b).sum()) for b in range(clouds))
    active = SparseTensor(pooled.coords[:n_out].contiguous(), z.feats[:n_out].contiguous(),
                          stride=2, batch_counts=counts)
    g = ops.global_avg_pool(active).cpu().numpy()
    want_g = restatement.global_pool(z.feats.cpu().numpy()[:n_out], counts, 'avg')
    assert np.allclose(g, want_g, rtol=1e-5, atol=1e-5 * np.abs(want_g).max())


def test_module_surface_and_errors(cuda):
    from mlx_lattice_b200 import nn, ops
    from mlx_lattice_b200.core import SparseTensor, quantize_weight

    coords = torch.from_numpy(synthetic.sphere_plane_batch(0, 1, 3000, 64)).to(cuda)
    feats = torch.randn(3000, 32, device=cuda, dtype=torch.float16)
    x = SparseTensor(coords, feats)
    conv = nn.Conv3d(32, 64, kernel_size=2, stride=2).to(cuda, torch.float16)
    down = conv(x)
    assert down.stride == (2, 2, 2) and down.capacity == 3000 and down.channels == 64
    q = conv.to_quantized(group_size=32, bits=4)
    down_q = q(x)
    assert down_q.feats.shape == down.feats.shape
    # relation cache: the quantized conv reuses the map built for the float conv
    assert len(x.coord_manager._kernel_relations) == 1
    up = nn.ConvTranspose3d(64, 32, kernel_size=2, stride=2, bias=False).to(cuda, torch.float16)
    restored = up(down, coordinates=x)
    assert restored.same_coords(x)
    plain = up(down)
    assert plain.capacity == 8 * 3000
    with pytest.raises(ValueError, match='convolution weights must match feature dtype'):
        ops.conv3d(x, conv.weight.float(), kernel_size=2, stride=2)
    with pytest.raises(ValueError, match='subm_conv3d requires odd kernel_size'):
        ops.subm_conv3d(x, conv.weight, kernel_size=2)
    with pytest.raises(ValueError, match='pooling currently supports float32'):
        ops.max_pool3d(x)
    with pytest.raises(ValueError, match='quantized weight input channels must match'):
        ops.subm_conv3d(x, quantize_weight(torch.randn(8, 3, 3, 3, 64).half(), group_size=32))


def test_forward_pass_captures_into_a_cuda_graph(cuda):
    """No call on the path synchronises or copies from pageable host memory: a whole
    forward pass (maps, orders, plans, convolutions, head) is captured once and replayed
    with the same bits as the eager run."""
    from mlx_lattice_b200 import workloads
    from mlx_lattice_b200.core import SparseTensor

    coords_np, feats_np = workloads.minkunet_inputs(4, 2, 6000)
    model = workloads.MinkUNet(workloads.quantize_all(workloads.minkunet_dense_weights(20264)), cuda)
    coords = torch.from_numpy(coords_np).to(cuda)
    feats = torch.from_numpy(feats_np).to(cuda)

    def forward():
        return model(SparseTensor(coords, feats, batch_counts=(6000, 6000))).feats

    eager = forward()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        forward()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = forward()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(captured, eager)
    feats.mul_(2)                      # new data in the same buffers
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(captured, forward())
