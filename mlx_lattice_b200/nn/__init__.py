from mlx_lattice_b200.nn._module import Module
from mlx_lattice_b200.nn.conv import Conv3d, ConvTranspose3d, SubmConv3d
from mlx_lattice_b200.nn.feature import (
    BatchNorm,
    Dropout,
    GELU,
    LayerNorm,
    LeakyReLU,
    Linear,
    ReLU,
    RMSNorm,
    Sigmoid,
    SiLU,
    Softplus,
    Tanh,
)
from mlx_lattice_b200.nn.pool import (
    AvgPool3d,
    GlobalAvgPool,
    GlobalMaxPool,
    GlobalSumPool,
    MaxPool3d,
    Pool3d,
    SumPool3d,
)
from mlx_lattice_b200.nn.quantized_conv import (
    QuantizedConv3d,
    QuantizedConvTranspose3d,
    QuantizedSubmConv3d,
)
from mlx_lattice_b200.nn.quantized_feature import QuantizedLinear

__all__ = [
    'Dropout', 'GELU', 'LayerNorm', 'LeakyReLU', 'RMSNorm', 'SiLU', 'Sigmoid', 'Softplus', 'Tanh',
    'AvgPool3d', 'BatchNorm', 'Conv3d', 'ConvTranspose3d', 'GlobalAvgPool', 'GlobalMaxPool',
    'GlobalSumPool', 'Linear', 'MaxPool3d', 'Module', 'Pool3d', 'QuantizedConv3d',
    'QuantizedConvTranspose3d', 'QuantizedLinear', 'QuantizedSubmConv3d', 'ReLU', 'SubmConv3d',
    'SumPool3d',
]
