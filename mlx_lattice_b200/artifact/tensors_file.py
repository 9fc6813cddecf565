"""``weights.safetensors`` reader and writer.

The reference stores artifact weights with ``mx.save_safetensors``
(``mlx_lattice/artifact/io.py:58-78``): the public safetensors container, i.e. an
8-byte little-endian header length, a JSON header mapping each tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end of the
header; optional ``__metadata__`` entry of strings), then the raw little-endian tensor
bytes. Packed quantised codes are ``U32``, their metadata vector ``I32``.

The file is decoded with numpy and handed over as CPU torch tensors; the model moves
them to the GPU once (``LatticeModel.to``).
"""

from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np
import torch

_NUMPY_DTYPES = {
    'BOOL': np.bool_, 'U8': np.uint8, 'I8': np.int8, 'U16': np.uint16, 'I16': np.int16,
    'U32': np.uint32, 'I32': np.int32, 'U64': np.uint64, 'I64': np.int64,
    'F16': np.float16, 'F32': np.float32, 'F64': np.float64,
}
_TAGS = {np.dtype(v): k for k, v in _NUMPY_DTYPES.items()}
_MAX_HEADER = 100 * 1024 * 1024


def _bf16_to_torch(raw: np.ndarray, shape: list[int]) -> torch.Tensor:
    return torch.from_numpy(raw.view(np.int16).copy()).view(torch.bfloat16).reshape(shape)


def load_tensors(path: str | Path) -> dict[str, torch.Tensor]:
    """All tensors of a safetensors file as CPU torch tensors (copies, not views)."""
    data = Path(path).read_bytes()
    if len(data) < 8:
        raise ValueError('weights.safetensors is truncated.')
    (header_bytes,) = struct.unpack('<Q', data[:8])
    if header_bytes > _MAX_HEADER or 8 + header_bytes > len(data):
        raise ValueError('weights.safetensors has an invalid header length.')
    try:
        header = json.loads(data[8:8 + header_bytes].decode('utf-8'))
    except (UnicodeDecodeError, json.JSONDecodeError) as exc:
        raise ValueError('weights.safetensors has an invalid header.') from exc
    if not isinstance(header, dict):
        raise ValueError('weights.safetensors must load as a tensor mapping.')
    body = memoryview(data)[8 + header_bytes:]
    tensors: dict[str, torch.Tensor] = {}
    for name, entry in header.items():
        if name == '__metadata__':
            continue
        try:
            tag, shape = entry['dtype'], [int(v) for v in entry['shape']]
            begin, end = (int(v) for v in entry['data_offsets'])
        except (KeyError, TypeError, ValueError) as exc:
            raise ValueError(f'weights.safetensors entry {name!r} is malformed.') from exc
        if not 0 <= begin <= end <= len(body):
            raise ValueError(f'weights.safetensors entry {name!r} lies outside the file.')
        count = int(np.prod(shape, dtype=np.int64)) if shape else 1
        if tag == 'BF16':
            if end - begin != 2 * count:
                raise ValueError(f'weights.safetensors entry {name!r} has a wrong byte size.')
            tensors[name] = _bf16_to_torch(np.frombuffer(body[begin:end], dtype=np.uint16), shape)
            continue
        if tag not in _NUMPY_DTYPES:
            raise ValueError(f'weights.safetensors entry {name!r} has unsupported dtype {tag!r}.')
        dtype = np.dtype(_NUMPY_DTYPES[tag]).newbyteorder('<')
        if end - begin != dtype.itemsize * count:
            raise ValueError(f'weights.safetensors entry {name!r} has a wrong byte size.')
        array = np.frombuffer(body[begin:end], dtype=dtype).astype(dtype.newbyteorder('='))
        tensors[name] = torch.from_numpy(array.reshape(shape).copy())
    return tensors


def save_tensors(path: str | Path, tensors: dict[str, torch.Tensor],
                 metadata: dict[str, str] | None = None) -> None:
    """Write tensors in name order, each aligned as the format asks (header padded with
    spaces to a multiple of 8 bytes)."""
    header: dict[str, object] = {}
    if metadata:
        header['__metadata__'] = {str(k): str(v) for k, v in metadata.items()}
    chunks: list[bytes] = []
    offset = 0
    for name in sorted(tensors):
        value = tensors[name].detach().cpu().contiguous()
        if value.dtype == torch.bfloat16:
            tag, raw = 'BF16', value.view(torch.int16).numpy().tobytes()
        else:
            array = value.numpy()
            if array.dtype not in _TAGS:
                raise ValueError(f'tensor {name!r} has unsupported dtype {value.dtype}.')
            tag, raw = _TAGS[array.dtype], array.astype(array.dtype.newbyteorder('<')).tobytes()
        header[name] = {
            'dtype': tag, 'shape': list(value.shape), 'data_offsets': [offset, offset + len(raw)],
        }
        chunks.append(raw)
        offset += len(raw)
    encoded = json.dumps(header, separators=(',', ':')).encode('utf-8')
    encoded += b' ' * (-len(encoded) % 8)
    with Path(path).open('wb') as file:
        file.write(struct.pack('<Q', len(encoded)))
        file.write(encoded)
        for raw in chunks:
            file.write(raw)
