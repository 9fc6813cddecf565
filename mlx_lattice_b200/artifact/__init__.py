"""Lattice model artifacts (``manifest.json`` + ``weights.safetensors``) on the B200 path:
the reference's loader surface (``mlx_lattice/artifact/__init__.py``) for inference."""

from mlx_lattice_b200.artifact.export import GraphWriter
from mlx_lattice_b200.artifact.io import (
    LatticeArtifact,
    load_lattice_artifact,
    load_lattice_model,
    save_lattice_artifact,
    save_lattice_model,
)
from mlx_lattice_b200.artifact.manifest import (
    IRManifest,
    IRNode,
    IRSparseSupport,
    IRTensorSpec,
    load_manifest,
    manifest_from_dict,
    manifest_to_dict,
)
from mlx_lattice_b200.artifact.model import LatticeModel
from mlx_lattice_b200.artifact.registry import iter_operation_bindings, operation_binding

__all__ = [
    'GraphWriter', 'IRManifest', 'IRNode', 'IRSparseSupport', 'IRTensorSpec', 'LatticeArtifact',
    'LatticeModel', 'iter_operation_bindings', 'load_lattice_artifact', 'load_lattice_model',
    'load_manifest', 'manifest_from_dict', 'manifest_to_dict', 'operation_binding',
    'save_lattice_artifact', 'save_lattice_model',
]
