"""The C-ABI library loads and exports every symbol the header declares, and the
ctypes signatures agree with the header's parameter counts. No compute calls."""

import ctypes
import os
import re

import pytest

from mlx_lattice_b200 import _native

HEADER = os.path.join(os.path.dirname(os.path.dirname(__file__)), 'include', 'lattice_b200.h')


def _declarations():
    text = open(HEADER).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    found = {}
    for match in re.finditer(r'\b(lat_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;', text, flags=re.S):
        name, params = match.group(1), match.group(2).strip()
        count = 0 if params in ('', 'void') else params.count(',') + 1
        found[name] = count
    return found


def test_header_declares_functions():
    decls = _declarations()
    assert len(decls) >= 30
    for required in ('lat_build_kernel_relation', 'lat_sparse_quantized_conv_features',
                     'lat_sparse_pool_features', 'lat_build_relation_grouped_view'):
        assert required in decls


def test_library_exports_every_declared_symbol():
    if not _native.library_present():
        pytest.fail('liblattice_b200.so is not built (python -m mlx_lattice_b200.build)')
    lib = ctypes.CDLL(_native.LIBRARY_PATH)
    for name in _declarations():
        assert hasattr(lib, name), f'{name} is declared in the header but not exported'


def test_ctypes_signatures_match_header():
    decls = _declarations()
    assert set(decls) == set(_native.SIGNATURES), (
        set(decls) ^ set(_native.SIGNATURES)
    )
    for name, count in decls.items():
        assert len(_native.SIGNATURES[name][1]) == count, name


def test_host_only_entry_points():
    lib = _native.load()
    assert lib.lat_version().decode().endswith('b200')
    from mlx_lattice_b200 import _ext

    assert _ext.kernel_offsets((3, 1, 1)) == ((-1, 0, 0), (0, 0, 0), (1, 0, 0))
    assert _ext.kernel_offsets(2)[:3] == ((0, 0, 0), (0, 0, 1), (0, 1, 0))
    with pytest.raises(ValueError, match='kernel_size values must be positive'):
        _ext.kernel_offsets((0, 1, 1))
    caps = _ext.capabilities()
    assert set(caps) == {'cpu', 'metal', 'cuda'} and caps['cpu'] is False


def test_vector_arguments_are_checked_on_the_host():
    """`_vec_arg` guards every optional per-channel pointer of `_ext`: a host tensor is
    refused with a ValueError (no launch is possible without a device anyway)."""
    import pytest
    import torch

    from mlx_lattice_b200 import _ext

    like = torch.zeros((4, 8), dtype=torch.float16)
    assert _ext._vec_arg(None, 'bias', 8, like) is None
    with pytest.raises(ValueError, match='bias must be a CUDA tensor'):
        _ext._vec_arg(torch.zeros(8, dtype=torch.float16), 'bias', 8, like)
    with pytest.raises(ValueError, match='bias must be a CUDA tensor'):
        _ext._vec_arg([0.0] * 8, 'bias', 8, like)
