"""Builds ``liblattice_b200.so`` (the C-ABI library) in-tree with nvcc for sm_100a.

Usage: ``python -m mlx_lattice_b200.build [--force] [--verbose]``. nvcc cross-compiles
without a GPU, so this runs on any machine with the CUDA toolkit.
"""

from __future__ import annotations

import os
import subprocess
import sys

PACKAGE_DIR = os.path.dirname(os.path.abspath(__file__))
REPO_DIR = os.path.dirname(PACKAGE_DIR)
CSRC_DIR = os.path.join(PACKAGE_DIR, 'csrc')
LIBRARY_PATH = os.path.join(PACKAGE_DIR, 'liblattice_b200.so')

SOURCES = (
    'relation.cu',
    'conv_direct.cu',
    'conv_tc.cu',
    'conv_tc_plan.cu',
    'conv_plan.cu',
    'order.cu',
    'voxelize.cu',
    'static_scratch.cu',
    'pool.cu',
    'feature.cu', 'align.cu',
    'capi.cu',
)

NVCC_FLAGS = (
    '-gencode', 'arch=compute_100a,code=sm_100a',
    '-lineinfo', '-O3', '-std=c++17',
    '-Xcompiler', '-fPIC', '-shared',
)


def _nvcc() -> str:
    for candidate in (os.environ.get('NVCC'), '/usr/local/cuda/bin/nvcc', 'nvcc'):
        if candidate and (os.path.isabs(candidate) and os.path.exists(candidate)):
            return candidate
    return 'nvcc'


def _inputs() -> list[str]:
    files = [os.path.join(CSRC_DIR, name) for name in os.listdir(CSRC_DIR)]
    files.append(os.path.join(REPO_DIR, 'include', 'lattice_b200.h'))
    return files


def is_stale() -> bool:
    if not os.path.exists(LIBRARY_PATH):
        return True
    built = os.path.getmtime(LIBRARY_PATH)
    return any(os.path.getmtime(path) > built for path in _inputs())


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile every CUDA source into one shared library; returns its path."""
    if not force and not is_stale():
        return LIBRARY_PATH
    command = [
        _nvcc(), *NVCC_FLAGS,
        *(('-Xptxas', '-v') if verbose else ()),
        '-I', os.path.join(REPO_DIR, 'include'),
        *(os.path.join(CSRC_DIR, name) for name in SOURCES),
        '-o', LIBRARY_PATH,
    ]
    result = subprocess.run(command, capture_output=True, text=True)
    if verbose or result.returncode != 0:
        sys.stderr.write(result.stdout)
        sys.stderr.write(result.stderr)
    if result.returncode != 0:
        raise RuntimeError('nvcc failed building liblattice_b200.so')
    return LIBRARY_PATH


if __name__ == '__main__':
    print(build_library(force='--force' in sys.argv, verbose='--verbose' in sys.argv))
