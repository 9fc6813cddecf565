"""B200-native (sm_100a) sparse-convolution inference path with the operator and
module surface of ``mlx_lattice`` (``ops``: ``conv3d``, ``subm_conv3d``,
``max_pool3d``, ``coordinates=``; ``nn``: ``Conv3d``, ``SubmConv3d``,
``QuantizedConv3d``, ``QuantizedLinear`` ...). Arrays are CUDA ``torch.Tensor``;
all computation is in ``liblattice_b200.so`` (CUDA kernels behind a C ABI).
"""

from mlx_lattice_b200 import _native


def backend_info() -> dict:
    """``mlx_lattice.backend_info()`` (``mlx_lattice/_native.py:6-11``)."""
    from mlx_lattice_b200 import _ext

    return {'version': _ext.version(), 'capabilities': _ext.capabilities()}


__all__ = ['backend_info']
