"""Artifact directories: ``manifest.json`` beside ``weights.safetensors``
(``mlx_lattice/artifact/io.py:22-134``)."""

from __future__ import annotations

import json
from collections.abc import Mapping
from dataclasses import dataclass
from pathlib import Path

import torch

from mlx_lattice_b200.artifact.manifest import IRManifest, load_manifest, manifest_to_dict
from mlx_lattice_b200.artifact.model import LatticeModel
from mlx_lattice_b200.artifact.tensors_file import load_tensors, save_tensors

MANIFEST_NAME = 'manifest.json'
WEIGHTS_NAME = 'weights.safetensors'


@dataclass(frozen=True, slots=True)
class LatticeArtifact:
    """A loaded artifact: the validated manifest and its tensors (on the CPU)."""

    manifest: IRManifest
    weights: dict[str, torch.Tensor]

    def model(self, device: torch.device | str | None = None) -> LatticeModel:
        return LatticeModel(self.manifest, self.weights, device=device)


def load_lattice_artifact(path: str | Path) -> LatticeArtifact:
    root = Path(path)
    if not root.is_dir():
        raise ValueError(f'lattice artifact directory does not exist: {root}')
    if not (root / MANIFEST_NAME).is_file():
        raise ValueError(f'lattice artifact is missing {MANIFEST_NAME}.')
    if not (root / WEIGHTS_NAME).is_file():
        raise ValueError(f'lattice artifact is missing {WEIGHTS_NAME}.')
    return LatticeArtifact(load_manifest(root / MANIFEST_NAME), load_tensors(root / WEIGHTS_NAME))


def load_lattice_model(path: str | Path, device: torch.device | str | None = None) -> LatticeModel:
    """The deployment entry point: artifact directory -> executable model with its weights
    on ``device`` (the current CUDA device when omitted and one is available)."""
    if device is None and torch.cuda.is_available():
        device = torch.device('cuda', torch.cuda.current_device())
    return load_lattice_artifact(path).model(device)


def save_lattice_artifact(path: str | Path, manifest: IRManifest,
                          weights: Mapping[str, torch.Tensor]) -> None:
    """Strict low-level writer: the manifest must validate against the weights."""
    LatticeModel(manifest, weights)
    root = Path(path)
    root.mkdir(parents=True, exist_ok=True)
    with (root / MANIFEST_NAME).open('w', encoding='utf-8') as file:
        json.dump(manifest_to_dict(manifest), file, indent=2)
        file.write('\n')
    save_tensors(root / WEIGHTS_NAME, dict(weights))


save_lattice_model = save_lattice_artifact
