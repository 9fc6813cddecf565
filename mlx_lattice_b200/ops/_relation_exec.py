"""Feature execution over a prebuilt relation (``mlx_lattice/ops/_relation_exec.py``)."""

from __future__ import annotations

import torch

from mlx_lattice_b200 import _ext
from mlx_lattice_b200.core.quantized import QuantizedWeight
from mlx_lattice_b200.core.relations import KernelRelation


def _row_order(relation: KernelRelation, uses_tensor_cores: bool):
    if not uses_tensor_cores:
        return None
    return relation.require_row_order()


def _conv_plan(relation: KernelRelation, uses_tensor_cores: bool, in_rows: int):
    """The relation's gather plan when the tensor-core route runs and the features
    have the row capacity the plan was validated against."""
    if not uses_tensor_cores or relation.n_in_capacity != in_rows:
        return None
    return relation.require_conv_plan()


def _sources(feats, relation: KernelRelation, uses_tensor_cores: bool):
    """``feats`` is one array or a pair over the same rows (an unwritten channel
    concatenation). The tensor-core route with a gather plan reads a pair in place when the
    first part's channel count is a multiple of 8; otherwise the pair is concatenated."""
    if not isinstance(feats, tuple):
        return feats, None
    first, second = feats
    in_place = (uses_tensor_cores and relation.n_in_capacity == int(first.shape[0])
                and int(first.shape[1]) % 8 == 0)
    if in_place:
        return first, second
    return _ext.concat_aligned_features(first, None, second, None), None


def _kept_fp16_weights(weight: QuantizedWeight) -> torch.Tensor:
    """The dequantised ``(K, C_out, C_in)`` fp16 form of a packed weight, made once and kept on
    the packed array (weights are constants of an inference network; a later in-place change
    of the packed array, its scales or its biases makes a new one)."""
    versions = (weight.weight._version, weight.scales._version, weight.biases._version,
                weight.scales.data_ptr(), weight.biases.data_ptr())
    kept = getattr(weight.weight, '_lattice_fp16', None)
    if kept is None or kept[0] != versions:
        kept = (versions, _ext.dequantize_conv_weights(
            weight.weight, weight.scales, weight.biases, weight.in_channels, weight.out_channels,
            weight.storage_in_channels, weight.group_size, weight.bits))
        weight.weight._lattice_fp16 = kept
    return kept[1]


def sparse_quantized_conv_features_from_relation(
    feats, weight: QuantizedWeight, relation: KernelRelation, bias=None
) -> torch.Tensor:
    """Quantized sparse convolution over a prebuilt relation (``:19-61``)."""
    if relation.n_out_capacity is None or relation.n_kernels is None:
        raise ValueError('kernel relation is missing static shape metadata.')
    if relation.n_kernels != weight.weight.shape[0]:
        raise ValueError('quantized weight kernel rows must match the relation.')
    dtype = feats[0].dtype if isinstance(feats, tuple) else feats.dtype
    tc = _ext.conv_uses_tensor_cores(
        dtype, relation.n_kernels, weight.in_channels, weight.out_channels,
        weight.bits, weight.group_size,
    )
    feats, feats2 = _sources(feats, relation, tc)
    if tc and weight.scales.dtype == torch.float16:
        # the tensor cores take fp16 operands: the packed codes are converted once, not per call
        return _ext.sparse_conv_features(
            feats, _kept_fp16_weights(weight), relation.edges.in_rows, relation.edges.out_rows,
            relation.edges.kernel_ids, relation.counts, relation.output_csr.row_offsets,
            out_capacity=relation.n_out_capacity, n_kernels=relation.n_kernels, bias=bias,
            row_order=_row_order(relation, tc), plan=_conv_plan(relation, tc, int(feats.shape[0])),
            feats2=feats2, out_major=True,
        )
    return _ext.sparse_quantized_conv_features(
        feats,
        weight.weight,
        weight.scales,
        weight.biases,
        relation.edges.in_rows,
        relation.edges.out_rows,
        relation.edges.kernel_ids,
        relation.counts,
        relation.output_csr.row_offsets,
        None,
        None,
        None,
        relation.n_out_capacity,
        relation.n_kernels,
        weight.in_channels,
        weight.out_channels,
        weight.storage_in_channels,
        weight.group_size,
        weight.bits,
        bias=bias,
        row_order=_row_order(relation, tc),
        plan=_conv_plan(relation, tc, int(feats.shape[0])),
        feats2=feats2,
    )


def sparse_conv_features_from_relation(
    feats, weight: torch.Tensor, relation: KernelRelation, bias=None
) -> torch.Tensor:
    """Float sparse convolution over a prebuilt relation (``:84-116``)."""
    if relation.n_out_capacity is None or relation.n_kernels is None:
        raise ValueError('kernel relation is missing static shape metadata.')
    c_out = int(weight.shape[2] if weight.ndim == 3 else weight.shape[0])
    pair = isinstance(feats, tuple)
    tc = _ext.conv_uses_tensor_cores(
        feats[0].dtype if pair else feats.dtype, relation.n_kernels,
        int(feats[0].shape[1] + feats[1].shape[1]) if pair else int(feats.shape[1]), c_out
    )
    feats, feats2 = _sources(feats, relation, tc)
    return _ext.sparse_conv_features(
        feats,
        weight,
        relation.edges.in_rows,
        relation.edges.out_rows,
        relation.edges.kernel_ids,
        relation.counts,
        relation.output_csr.row_offsets,
        out_capacity=relation.n_out_capacity,
        n_kernels=relation.n_kernels,
        bias=bias,
        row_order=_row_order(relation, tc),
        plan=_conv_plan(relation, tc, int(feats.shape[0])),
        feats2=feats2,
    )


def sparse_pool_features_from_relation(
    feats: torch.Tensor, relation: KernelRelation, *, input_exclusive: bool, mode: str
) -> torch.Tensor:
    """Sparse pooling over a prebuilt kernel relation (``:256-276``)."""
    if relation.n_out_capacity is None or relation.n_kernels is None:
        raise ValueError('kernel relation is missing static shape metadata.')
    return _ext.sparse_pool_features(
        feats,
        relation.edges.in_rows,
        relation.edges.out_rows,
        relation.edges.kernel_ids,
        relation.output_csr.row_offsets,
        relation.counts,
        input_exclusive,
        mode,
        relation.n_out_capacity,
        relation.n_kernels,
    )
