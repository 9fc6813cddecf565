"""Drop-in for the reference's native extension module ``mlx_lattice._ext``.

Same function names, argument order and return tuples as ``native/bindings``
(``coords.cpp``, ``convolution.cpp``, ``pooling.cpp``, ``runtime.cpp``), with CUDA
``torch.Tensor`` in place of ``mx.array``. Torch only owns the device memory and
names the stream; every computation happens in ``liblattice_b200.so`` through its C
ABI. Nothing here synchronises the stream or reads device counts back, so a
sequence of calls can be captured into a CUDA graph.
"""

from __future__ import annotations

from typing import Sequence

import torch

from mlx_lattice_b200 import _native
from mlx_lattice_b200._native import FloatTriple, Triple, check

_REDUCE = {'sum': 0, 'max': 1, 'avg': 2}
_JOIN = {'inner': 0, 'left': 1, 'right': 2, 'outer': 3}

_status_words: dict[int, torch.Tensor] = {}


# --------------------------------------------------------------------------- #
# plumbing
# --------------------------------------------------------------------------- #


def _lib():
    return _native.load()


def _require_cuda(tensor: torch.Tensor, name: str) -> None:
    if not isinstance(tensor, torch.Tensor):
        raise ValueError(f'{name} must be a torch.Tensor.')
    if not tensor.is_cuda:
        raise RuntimeError(
            f'{name} must live on a CUDA device: this build has no CPU route.'
        )


def _ptr(tensor: torch.Tensor | None):
    if tensor is None or tensor.numel() == 0:
        return None
    return tensor.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _triple(values: int | Sequence[int]) -> Triple:
    if isinstance(values, int):
        values = (values, values, values)
    x, y, z = (int(v) for v in values)
    return Triple(x, y, z)


def status_word(device: torch.device | None = None) -> torch.Tensor:
    """Per-device int32 word in which kernels record run-time problems."""
    index = torch.cuda.current_device() if device is None or device.index is None else device.index
    word = _status_words.get(index)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=torch.device('cuda', index))
        _status_words[index] = word
    return word


def check_status(device: torch.device | None = None) -> None:
    """Synchronise and raise if any kernel recorded a problem since the last check."""
    word = status_word(device)
    value = int(word.item())
    if value != 0:
        word.zero_()
        reasons = [text for bit, text in _native.STATUS_BITS.items() if value & bit]
        raise RuntimeError('lattice_b200 device status: ' + '; '.join(reasons))


def _workspace(nbytes: int, device: torch.device) -> torch.Tensor:
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


def _coords_arg(coords: torch.Tensor, name: str = 'coords') -> torch.Tensor:
    _require_cuda(coords, name)
    if coords.ndim != 2 or coords.shape[1] != 4:
        raise ValueError('coords must have shape (N, 4).')
    if coords.dtype != torch.int32:
        raise ValueError('CUDA sparse kernels require int32 coordinates.')
    return coords.contiguous()


def _active_arg(active_rows: torch.Tensor) -> torch.Tensor:
    _require_cuda(active_rows, 'active_rows')
    if tuple(active_rows.shape) != (1,) or active_rows.dtype != torch.int32:
        raise ValueError('active_rows must have shape (1,) and int32 dtype.')
    return active_rows


def _i32(tensor: torch.Tensor, name: str) -> torch.Tensor:
    _require_cuda(tensor, name)
    if tensor.dtype != torch.int32:
        raise ValueError(f'{name} must be int32.')
    return tensor.contiguous()


def _dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return 0
    if dtype == torch.float16:
        return 1
    raise ValueError('convolution supports float32 and float16 tensors.')


def _vec_arg(vector, name: str, length: int, like: torch.Tensor, dtype=None):
    """Optional per-channel vector handed to a kernel as a bare pointer: CUDA tensor on the
    device of ``like``, exact length and dtype, contiguous. Returns the (contiguous) tensor
    or None; raises ValueError before anything is launched."""
    if vector is None:
        return None
    if not isinstance(vector, torch.Tensor) or not vector.is_cuda:
        raise ValueError(f'{name} must be a CUDA tensor.')
    if vector.device != like.device:
        raise ValueError(f'{name} must be on the same device as the features.')
    want = like.dtype if dtype is None else dtype
    if vector.dtype != want:
        raise ValueError(f'{name} dtype must be {want}.')
    if tuple(vector.shape) != (int(length),):
        raise ValueError(f'{name} must have shape ({int(length)},).')
    return vector.contiguous()


def _second_source(feats: torch.Tensor, feats2) -> tuple[torch.Tensor | None, int, int]:
    """Validated second feature source of a convolution: (tensor, row stride, channels)."""
    if feats2 is None:
        return None, 0, 0
    feats2, stride2 = _feats_arg(feats2)
    if feats2.device != feats.device or feats2.dtype != feats.dtype:
        raise ValueError('both feature sources must share device and dtype.')
    if feats2.shape[0] != feats.shape[0]:
        raise ValueError('both feature sources must have the same row count.')
    return feats2, stride2, int(feats2.shape[1])


def _feats_arg(feats: torch.Tensor) -> tuple[torch.Tensor, int]:
    _require_cuda(feats, 'feats')
    if feats.ndim != 2:
        raise ValueError('feats must have shape (N, C).')
    if feats.stride(1) != 1:
        feats = feats.contiguous()
    return feats, int(feats.stride(0)) if feats.shape[0] > 1 else int(feats.shape[1])


# --------------------------------------------------------------------------- #
# runtime (native/bindings/runtime.cpp:27-38)
# --------------------------------------------------------------------------- #


def launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    return int(_lib().lat_launch_count())


# Optional profiling hook: when set to a callable, every convolution call is
# bracketed by CUDA events on the current stream and reported to it as
# hook(kind, info_dict, start_event, end_event). Off (None) on the product path.
profile_hook = None


def _profiled(kind: str, info: dict, call):
    if profile_hook is None:
        return call()
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    start.record()
    out = call()
    end.record()
    profile_hook(kind, info, start, end)
    return out


def version() -> str:
    return _lib().lat_version().decode()


def capabilities() -> dict[str, bool]:
    import ctypes

    has = ctypes.c_int32(0)
    count = ctypes.c_int32(0)
    check(_lib().lat_capabilities(ctypes.byref(has), ctypes.byref(count)))
    return {'cpu': False, 'metal': False, 'cuda': bool(has.value)}


def kernel_offsets(kernel_size, dilation=1) -> tuple[tuple[int, int, int], ...]:
    import ctypes

    ks, dil = _triple(kernel_size), _triple(dilation)
    volume = max(ks.x, 0) * max(ks.y, 0) * max(ks.z, 0)
    buffer = (ctypes.c_int32 * max(3 * volume, 3))()
    check(_lib().lat_kernel_offsets_host(ks, dil, ctypes.cast(buffer, ctypes.c_void_p)))
    return tuple(
        (buffer[3 * k], buffer[3 * k + 1], buffer[3 * k + 2]) for k in range(volume)
    )


# --------------------------------------------------------------------------- #
# kernel relations (native/bindings/coords.cpp:414-589)
# --------------------------------------------------------------------------- #


def _relation_buffers(edge_capacity: int, out_capacity: int, device, with_out_coords=True):
    def new(n):
        return torch.empty(n, dtype=torch.int32, device=device)

    return (
        new(edge_capacity),
        new(edge_capacity),
        new(edge_capacity),
        new(out_capacity + 1),
        torch.empty((out_capacity, 4), dtype=torch.int32, device=device)
        if with_out_coords
        else None,
        new(2),
    )


def _views(in_rows, kernel_ids, counts, in_capacity: int, kernel_count: int):
    in_offsets, in_edges = build_relation_grouped_view(in_rows, counts, in_capacity)
    k_offsets, k_edges = build_relation_grouped_view(kernel_ids, counts, kernel_count)
    return in_offsets, in_edges, k_offsets, k_edges


def build_coord_table(coords, active_rows):
    """First-row-wins coordinate table of ``coords`` as an opaque device buffer that the
    builders taking ``source_table`` accept in place of building their own (the reference's
    GPU builders fill one per call, ``native/features/coordinates/relations.cpp:555``)."""
    coords = _coords_arg(coords)
    active_rows = _active_arg(active_rows)
    rows = int(coords.shape[0])
    device = coords.device
    lib = _lib()
    table = _workspace(lib.lat_coord_table_bytes(rows), device)
    with torch.cuda.device(device):
        check(lib.lat_build_coord_table(
            _ptr(coords), rows, _ptr(active_rows), _ptr(table), table.numel(),
            _ptr(status_word(device)), _stream(),
        ))
    return table


def build_kernel_relation_base(
    coords, active_rows, kernel_size, stride, padding, dilation, *,
    want_masks=False, want_kernel_lists=False, source_table=None,
):
    """The six contract arrays of a forward relation plus, on request, the row
    masks and the per-offset pair lists produced in the same pass. ``source_table``
    is an optional ``build_coord_table(coords, active_rows)``."""
    coords = _coords_arg(coords)
    active_rows = _active_arg(active_rows)
    ks = _triple(kernel_size)
    rows = int(coords.shape[0])
    volume = ks.x * ks.y * ks.z
    if min(ks.x, ks.y, ks.z) <= 0:
        raise ValueError('kernel_size values must be positive.')
    device = coords.device
    in_rows, out_rows, kernel_ids, row_offsets, out_coords, counts = _relation_buffers(
        rows * volume, rows, device
    )
    words = (volume + 31) // 32
    masks = torch.empty((rows, words), dtype=torch.int32, device=device) if want_masks else None
    k_offsets = torch.empty(volume + 1, dtype=torch.int32, device=device) if want_kernel_lists else None
    k_edges = torch.empty(rows * volume, dtype=torch.int32, device=device) if want_kernel_lists else None
    lib = _lib()
    nbytes = lib.lat_relation_workspace_bytes(rows, rows, volume)
    ws = _workspace(nbytes, device)
    with torch.cuda.device(device):
        check(lib.lat_build_kernel_relation(
            _ptr(coords), rows, _ptr(active_rows), ks, _triple(stride), _triple(padding),
            _triple(dilation), _ptr(in_rows), _ptr(out_rows), _ptr(kernel_ids),
            _ptr(row_offsets), _ptr(out_coords), _ptr(counts), _ptr(masks), _ptr(k_offsets),
            _ptr(k_edges), _ptr(source_table), _ptr(ws), ws.numel(),
            _ptr(status_word(device)), _stream(),
        ))
    return (in_rows, out_rows, kernel_ids, row_offsets, out_coords, counts), masks, (k_offsets, k_edges)


def build_kernel_relation(coords, active_rows, kernel_size, stride, padding, dilation):
    """``_ext.build_kernel_relation`` (``native/bindings/coords.cpp:414-479``):
    returns the 10-tuple (in_rows, out_rows, kernel_ids, output_row_offsets,
    out_coords, counts, in_row_offsets, in_edge_ids, kernel_row_offsets,
    kernel_edge_ids)."""
    base, _, (k_offsets, k_edges) = build_kernel_relation_base(
        coords, active_rows, kernel_size, stride, padding, dilation, want_kernel_lists=True
    )
    in_rows, out_rows, kernel_ids, row_offsets, out_coords, counts = base
    in_offsets, in_edges = build_relation_grouped_view(in_rows, counts, int(coords.shape[0]))
    return (*base, in_offsets, in_edges, k_offsets, k_edges)


def build_submanifold_kernel_relation(coords, active_rows, kernel_size, dilation):
    """``_ext.build_submanifold_kernel_relation`` (``coords.cpp:480-508``)."""
    return build_kernel_relation(coords, active_rows, kernel_size, 1, 0, dilation)


def build_target_kernel_relation_base(
    coords, active_rows, target_coords, target_active_rows, kernel_size, stride, padding,
    dilation, *, want_masks=False, want_kernel_lists=False,
):
    coords = _coords_arg(coords)
    target = _coords_arg(target_coords, 'target_coords')
    active_rows = _active_arg(active_rows)
    target_active = _active_arg(target_active_rows)
    ks = _triple(kernel_size)
    if min(ks.x, ks.y, ks.z) <= 0:
        raise ValueError('kernel_size values must be positive.')
    rows, target_rows = int(coords.shape[0]), int(target.shape[0])
    volume = ks.x * ks.y * ks.z
    device = coords.device
    in_rows, out_rows, kernel_ids, row_offsets, _, counts = _relation_buffers(
        target_rows * volume, target_rows, device, with_out_coords=False
    )
    words = (volume + 31) // 32
    masks = torch.empty((target_rows, words), dtype=torch.int32, device=device) if want_masks else None
    k_offsets = torch.empty(volume + 1, dtype=torch.int32, device=device) if want_kernel_lists else None
    k_edges = torch.empty(target_rows * volume, dtype=torch.int32, device=device) if want_kernel_lists else None
    lib = _lib()
    ws = _workspace(lib.lat_relation_workspace_bytes(rows, target_rows, volume), device)
    with torch.cuda.device(device):
        check(lib.lat_build_target_kernel_relation(
            _ptr(coords), rows, _ptr(active_rows), _ptr(target), target_rows,
            _ptr(target_active), ks, _triple(stride), _triple(padding), _triple(dilation),
            _ptr(in_rows), _ptr(out_rows), _ptr(kernel_ids), _ptr(row_offsets), _ptr(counts),
            _ptr(masks), _ptr(k_offsets), _ptr(k_edges), _ptr(ws), ws.numel(),
            _ptr(status_word(device)), _stream(),
        ))
    return (in_rows, out_rows, kernel_ids, row_offsets, target, counts), masks, (k_offsets, k_edges)


def build_target_kernel_relation(
    coords, active_rows, target_coords, target_active_rows, kernel_size, stride, padding, dilation
):
    """``_ext.build_target_kernel_relation`` (``coords.cpp:546-589``); the fifth
    entry is the caller's target coordinates (``relations.cpp:53-70``)."""
    base, _, (k_offsets, k_edges) = build_target_kernel_relation_base(
        coords, active_rows, target_coords, target_active_rows, kernel_size, stride, padding,
        dilation, want_kernel_lists=True,
    )
    in_offsets, in_edges = build_relation_grouped_view(base[0], base[5], int(coords.shape[0]))
    return (*base, in_offsets, in_edges, k_offsets, k_edges)


def build_transposed_kernel_relation_base(
    coords, active_rows, kernel_size, stride, padding, dilation
):
    coords = _coords_arg(coords)
    active_rows = _active_arg(active_rows)
    ks = _triple(kernel_size)
    if min(ks.x, ks.y, ks.z) <= 0:
        raise ValueError('kernel_size values must be positive.')
    rows = int(coords.shape[0])
    volume = ks.x * ks.y * ks.z
    device = coords.device
    cap = rows * volume
    bufs = _relation_buffers(cap, cap, device)
    lib = _lib()
    ws = _workspace(lib.lat_relation_workspace_bytes(rows, cap, volume), device)
    with torch.cuda.device(device):
        check(lib.lat_build_transposed_kernel_relation(
            _ptr(coords), rows, _ptr(active_rows), ks, _triple(stride), _triple(padding),
            _triple(dilation), *(_ptr(b) for b in bufs), _ptr(ws), ws.numel(),
            _ptr(status_word(device)), _stream(),
        ))
    return bufs


def build_transposed_kernel_relation(coords, active_rows, kernel_size, stride, padding, dilation):
    """``_ext.build_transposed_kernel_relation`` (``coords.cpp:509-545``)."""
    bufs = build_transposed_kernel_relation_base(
        coords, active_rows, kernel_size, stride, padding, dilation
    )
    ks = _triple(kernel_size)
    return (*bufs, *_views(bufs[0], bufs[2], bufs[5], int(coords.shape[0]), ks.x * ks.y * ks.z))


def build_generative_relation_base(coords, active_rows, kernel_size, stride):
    coords = _coords_arg(coords)
    active_rows = _active_arg(active_rows)
    ks = _triple(kernel_size)
    if min(ks.x, ks.y, ks.z) <= 0:
        raise ValueError('kernel_size values must be positive.')
    rows = int(coords.shape[0])
    volume = ks.x * ks.y * ks.z
    device = coords.device
    cap = rows * volume
    bufs = _relation_buffers(cap, cap, device)
    lib = _lib()
    ws = _workspace(256, device)
    with torch.cuda.device(device):
        check(lib.lat_build_generative_relation(
            _ptr(coords), rows, _ptr(active_rows), ks, _triple(stride),
            *(_ptr(b) for b in bufs), _ptr(ws), ws.numel(), _ptr(status_word(device)), _stream(),
        ))
    return bufs


def build_generative_relation(coords, active_rows, kernel_size, stride):
    """``_ext.build_generative_relation`` (``native/bindings/coords.cpp``)."""
    bufs = build_generative_relation_base(coords, active_rows, kernel_size, stride)
    ks = _triple(kernel_size)
    return (*bufs, *_views(bufs[0], bufs[2], bufs[5], int(coords.shape[0]), ks.x * ks.y * ks.z))


def build_target_transposed_relation_base(
    coords, active_rows, target_coords, target_active_rows, stride, *, want_masks=False,
    source_table=None,
):
    """Transposed map of a ``kernel_size == stride`` conv restricted to a given
    fine support (one edge per target row at most); see ``include/lattice_b200.h``."""
    coords = _coords_arg(coords)
    target = _coords_arg(target_coords, 'target_coords')
    active_rows = _active_arg(active_rows)
    target_active = _active_arg(target_active_rows)
    rows, target_rows = int(coords.shape[0]), int(target.shape[0])
    device = coords.device
    in_rows, out_rows, kernel_ids, row_offsets, _, counts = _relation_buffers(
        target_rows, target_rows, device, with_out_coords=False
    )
    step = _triple(stride)
    masks = None
    if want_masks and step.x * step.y * step.z <= 32:
        masks = torch.empty((target_rows, 1), dtype=torch.int32, device=device)
    lib = _lib()
    ws = _workspace(lib.lat_relation_workspace_bytes(rows, target_rows, 1), device)
    with torch.cuda.device(device):
        check(lib.lat_build_target_transposed_relation(
            _ptr(coords), rows, _ptr(active_rows), _ptr(target), target_rows,
            _ptr(target_active), step, _ptr(in_rows), _ptr(out_rows),
            _ptr(kernel_ids), _ptr(row_offsets), _ptr(counts), _ptr(masks), _ptr(source_table),
            _ptr(ws), ws.numel(), _ptr(status_word(device)), _stream(),
        ))
    if want_masks:
        return (in_rows, out_rows, kernel_ids, row_offsets, target, counts), masks
    return (in_rows, out_rows, kernel_ids, row_offsets, target, counts)


def build_relation_grouped_view(group_ids, counts, group_count: int):
    """Edge ids grouped by ``group_ids`` (``make_relation_grouped_view``,
    ``native/features/coordinates/relations.cpp:438-459``)."""
    group_ids = _i32(group_ids, 'group_ids')
    counts = _i32(counts, 'counts')
    device = group_ids.device
    cap = int(group_ids.shape[0])
    row_offsets = torch.empty(group_count + 1, dtype=torch.int32, device=device)
    edge_ids = torch.empty(cap, dtype=torch.int32, device=device)
    lib = _lib()
    ws = _workspace(lib.lat_grouped_view_workspace_bytes(cap, group_count), device)
    with torch.cuda.device(device):
        check(lib.lat_build_relation_grouped_view(
            _ptr(group_ids), cap, _ptr(counts), group_count, _ptr(row_offsets), _ptr(edge_ids),
            _ptr(ws), ws.numel(), _ptr(status_word(device)), _stream(),
        ))
    return row_offsets, edge_ids


def build_relation_implicit_gemm_view(
    source_coords, source_active_rows, output_coords, output_active_rows, offsets, stride, padding
):
    """``_ext.build_relation_implicit_gemm_view`` (``coords.cpp:590-627``):
    returns (out_in_map [N_out, K], row_masks [N_out, ceil(K/32)])."""
    src = _coords_arg(source_coords, 'source_coords')
    out = _coords_arg(output_coords, 'output_coords')
    offsets = _i32(offsets, 'offsets')
    if offsets.ndim != 2 or offsets.shape[1] != 3:
        raise ValueError('offsets must have shape (K, 3).')
    k = int(offsets.shape[0])
    device = src.device
    out_in_map = torch.empty((out.shape[0], k), dtype=torch.int32, device=device)
    row_masks = torch.empty((out.shape[0], (k + 31) // 32), dtype=torch.int32, device=device)
    lib = _lib()
    ws = _workspace(lib.lat_implicit_gemm_view_workspace_bytes(int(src.shape[0])), device)
    with torch.cuda.device(device):
        check(lib.lat_build_relation_implicit_gemm_view(
            _ptr(src), int(src.shape[0]), _ptr(_active_arg(source_active_rows)),
            _ptr(out), int(out.shape[0]), _ptr(_active_arg(output_active_rows)),
            _ptr(offsets), k, _triple(stride), _triple(padding), _ptr(out_in_map),
            _ptr(row_masks), _ptr(ws), ws.numel(), _ptr(status_word(device)), _stream(),
        ))
    return out_in_map, row_masks


# --------------------------------------------------------------------------- #
# coordinate sets (native/bindings/coords.cpp:132-222)
# --------------------------------------------------------------------------- #


def downsample_coords(coords, stride):
    """Returns (coords [N, 4] with a valid prefix, count [1])."""
    coords = _coords_arg(coords)
    device = coords.device
    rows = int(coords.shape[0])
    out = torch.empty_like(coords)
    count = torch.empty(1, dtype=torch.int32, device=device)
    lib = _lib()
    ws = _workspace(lib.lat_coord_set_workspace_bytes(rows), device)
    with torch.cuda.device(device):
        check(lib.lat_downsample_coords(
            _ptr(coords), rows, _triple(stride), _ptr(out), _ptr(count), _ptr(ws), ws.numel(),
            _ptr(status_word(device)), _stream(),
        ))
    return out, count


def lookup_coords(coords, queries):
    coords = _coords_arg(coords)
    queries = _coords_arg(queries, 'queries')
    device = coords.device
    out = torch.empty(queries.shape[0], dtype=torch.int32, device=device)
    lib = _lib()
    ws = _workspace(lib.lat_coord_set_workspace_bytes(int(coords.shape[0])), device)
    with torch.cuda.device(device):
        check(lib.lat_lookup_coords(
            _ptr(coords), int(coords.shape[0]), _ptr(queries), int(queries.shape[0]), _ptr(out),
            _ptr(ws), ws.numel(), _ptr(status_word(device)), _stream(),
        ))
    return out


def lookup_coords_static(coords, queries, out: torch.Tensor | None = None):
    """``lookup_coords`` without any scratch allocation: the hash table is a fixed
    array inside the library (at most ``lookup_coords_static_max_rows()`` source rows).
    For callers that may not allocate; pass ``out`` (int32, one entry per query) to
    avoid even the result allocation. Calls share the table, so do not overlap them."""
    coords = _coords_arg(coords)
    queries = _coords_arg(queries, 'queries')
    device = coords.device
    if out is None:
        out = torch.empty(queries.shape[0], dtype=torch.int32, device=device)
    elif (not isinstance(out, torch.Tensor) or not out.is_cuda or out.device != device
          or out.dtype != torch.int32 or out.numel() != queries.shape[0] or not out.is_contiguous()):
        raise ValueError('out must be a contiguous int32 CUDA tensor on the device of coords with one '
                         'entry per query.')
    if queries.device != device:
        raise ValueError('queries must be on the same device as coords.')
    with torch.cuda.device(device):
        check(_lib().lat_lookup_coords_static(
            _ptr(coords), int(coords.shape[0]), _ptr(queries), int(queries.shape[0]), _ptr(out),
            _ptr(status_word(device)), _stream(),
        ))
    return out


def lookup_coords_static_max_rows() -> int:
    return int(_lib().lat_lookup_coords_static_max_rows())


def build_sparse_alignment(lhs_coords, lhs_active_rows, rhs_coords, rhs_active_rows, join):
    """Returns (coords, active_rows [1], lhs_rows, rhs_rows)
    (``coords.cpp:191-222``)."""
    if join not in _JOIN:
        raise ValueError("join must be 'inner', 'left', 'right', or 'outer'.")
    lhs = _coords_arg(lhs_coords, 'lhs_coords')
    rhs = _coords_arg(rhs_coords, 'rhs_coords')
    device = lhs.device
    l, r = int(lhs.shape[0]), int(rhs.shape[0])
    capacity = r if join == 'right' else (l + r if join == 'outer' else l)
    coords = torch.empty((capacity, 4), dtype=torch.int32, device=device)
    count = torch.empty(1, dtype=torch.int32, device=device)
    lhs_rows = torch.empty(capacity, dtype=torch.int32, device=device)
    rhs_rows = torch.empty(capacity, dtype=torch.int32, device=device)
    lib = _lib()
    ws = _workspace(lib.lat_sparse_alignment_workspace_bytes(l, r), device)
    with torch.cuda.device(device):
        check(lib.lat_build_sparse_alignment(
            _ptr(lhs), l, _ptr(_active_arg(lhs_active_rows)), _ptr(rhs), r,
            _ptr(_active_arg(rhs_active_rows)), _JOIN[join], _ptr(coords), _ptr(count),
            _ptr(lhs_rows), _ptr(rhs_rows), _ptr(ws), ws.numel(), _ptr(status_word(device)),
            _stream(),
        ))
    return coords, count, lhs_rows, rhs_rows


# --------------------------------------------------------------------------- #
# point -> voxel front end (native/bindings/coords.cpp:294-352)
# --------------------------------------------------------------------------- #


def _float_triple(values, name: str) -> FloatTriple:
    values = tuple(float(v) for v in values)
    if len(values) != 3:
        raise ValueError(f'{name} must contain exactly 3 values.')
    return FloatTriple(*values)


def sparse_quantize(points, batch_indices, active_rows, voxel_size, origin):
    """``_ext.sparse_quantize`` (``coords.cpp:294-325``): ``(coords, active_rows,
    inverse_rows, counts)`` with the reference's capacities (all N rows)."""
    _require_cuda(points, 'points')
    if points.ndim != 2 or points.shape[1] != 3:
        raise ValueError('points must have shape (N, 3).')
    if points.dtype != torch.float32:
        raise ValueError('points must be float32.')
    points = points.contiguous()
    rows = int(points.shape[0])
    batch = _i32(batch_indices, 'batch_indices')
    if tuple(batch.shape) != (rows,):
        raise ValueError('batch_indices must have shape (N,) and int32 dtype.')
    active_rows = _active_arg(active_rows)
    size = _float_triple(voxel_size, 'voxel_size')
    if min(size.x, size.y, size.z) <= 0.0:
        raise ValueError('voxel_size values must be positive.')
    device = points.device
    coords = torch.empty((rows, 4), dtype=torch.int32, device=device)
    count = torch.empty(1, dtype=torch.int32, device=device)
    inverse = torch.empty(rows, dtype=torch.int32, device=device)
    counts = torch.empty(rows, dtype=torch.int32, device=device)
    lib = _lib()
    ws = _workspace(lib.lat_sparse_quantize_workspace_bytes(rows), device)
    with torch.cuda.device(device):
        check(lib.lat_sparse_quantize(
            _ptr(points), _ptr(batch), rows, _ptr(active_rows), size,
            _float_triple(origin, 'origin'), _ptr(coords), _ptr(count), _ptr(inverse),
            _ptr(counts), _ptr(ws), ws.numel(), _ptr(status_word(device)), _stream(),
        ))
    return coords, count, inverse, counts


def voxelize_features(feats, inverse_rows, voxel_counts, active_rows, reduction):
    """``_ext.voxelize_features`` (``coords.cpp:326-352``): (voxel rows, C) float32."""
    _require_cuda(feats, 'feats')
    if feats.ndim != 2:
        raise ValueError('feats must have shape (N, C).')
    if feats.dtype != torch.float32:
        raise ValueError('voxelize currently supports float32 features.')
    if reduction not in ('sum', 'mean'):
        raise ValueError("reduction must be 'sum' or 'mean'.")
    feats = feats.contiguous()
    inverse = _i32(inverse_rows, 'inverse_rows')
    counts = _i32(voxel_counts, 'voxel_counts')
    if inverse.shape[0] != feats.shape[0]:
        raise ValueError('feats and quantization metadata must share rows.')
    active_rows = _active_arg(active_rows)
    points, voxels, channels = int(feats.shape[0]), int(counts.shape[0]), int(feats.shape[1])
    device = feats.device
    out = torch.empty((voxels, channels), dtype=torch.float32, device=device)
    lib = _lib()
    ws = _workspace(lib.lat_voxelize_features_workspace_bytes(points, voxels), device)
    with torch.cuda.device(device):
        check(lib.lat_voxelize_features(
            _ptr(feats), _ptr(inverse), _ptr(counts), _ptr(active_rows), points, voxels, channels,
            1 if reduction == 'mean' else 0, _ptr(out), _ptr(ws), ws.numel(),
            _ptr(status_word(device)), _stream(),
        ))
    return out


def build_point_voxel_map(points, batch_indices, point_active_rows, voxel_coords,
                          voxel_active_rows, voxel_size, origin, interpolation):
    """``_ext.build_point_voxel_map`` (``coords.cpp:353-395``): ``(rows, weights)``, both
    ``(N, 8)``."""
    _require_cuda(points, 'points')
    if points.ndim != 2 or points.shape[1] != 3:
        raise ValueError('points must have shape (N, 3).')
    if points.dtype != torch.float32:
        raise ValueError('points must be float32.')
    if interpolation not in ('nearest', 'linear'):
        raise ValueError("interpolation must be 'nearest' or 'linear'.")
    points = points.contiguous()
    rows = int(points.shape[0])
    batch = _i32(batch_indices, 'batch_indices')
    if tuple(batch.shape) != (rows,):
        raise ValueError('batch_indices must have shape (N,) and int32 dtype.')
    voxel_coords = _coords_arg(voxel_coords, 'voxel_coords')
    point_active = _active_arg(point_active_rows)
    _require_cuda(voxel_active_rows, 'voxel_active_rows')
    if tuple(voxel_active_rows.shape) != (1,) or voxel_active_rows.dtype != torch.int32:
        raise ValueError('voxel_active_rows must have shape (1,) and int32 dtype.')
    size = _float_triple(voxel_size, 'voxel_size')
    if min(size.x, size.y, size.z) <= 0.0:
        raise ValueError('voxel_size values must be positive.')
    device = points.device
    voxels = int(voxel_coords.shape[0])
    out_rows = torch.empty((rows, 8), dtype=torch.int32, device=device)
    weights = torch.empty((rows, 8), dtype=torch.float32, device=device)
    lib = _lib()
    ws = _workspace(lib.lat_point_voxel_map_workspace_bytes(voxels), device)
    with torch.cuda.device(device):
        check(lib.lat_build_point_voxel_map(
            _ptr(points), _ptr(batch), rows, _ptr(point_active), _ptr(voxel_coords), voxels,
            _ptr(voxel_active_rows), size, _float_triple(origin, 'origin'),
            1 if interpolation == 'linear' else 0, _ptr(out_rows), _ptr(weights), _ptr(ws),
            ws.numel(), _ptr(status_word(device)), _stream(),
        ))
    return out_rows, weights


def interpolate_point_features(voxel_feats, rows, weights):
    """``_ext.interpolate_point_features``: (points, C) float32."""
    _require_cuda(voxel_feats, 'voxel_feats')
    if voxel_feats.ndim != 2:
        raise ValueError('voxel_feats must have shape (N, C).')
    if voxel_feats.dtype != torch.float32:
        raise ValueError('point interpolation currently supports float32.')
    rows = _i32(rows, 'rows')
    _require_cuda(weights, 'weights')
    if rows.ndim != 2 or rows.shape[1] != 8:
        raise ValueError('rows must have shape (N, 8) and int32 dtype.')
    if weights.shape != rows.shape or weights.dtype != torch.float32:
        raise ValueError('weights must be float32.')
    voxel_feats, weights = voxel_feats.contiguous(), weights.contiguous()
    points, voxels, channels = int(rows.shape[0]), int(voxel_feats.shape[0]), int(voxel_feats.shape[1])
    device = voxel_feats.device
    out = torch.empty((points, channels), dtype=torch.float32, device=device)
    with torch.cuda.device(device):
        check(_lib().lat_interpolate_point_features(
            _ptr(voxel_feats), _ptr(rows), _ptr(weights), points, voxels, channels, _ptr(out), _stream(),
        ))
    return out


# --------------------------------------------------------------------------- #
# convolution (native/bindings/convolution.cpp:12-146)
# --------------------------------------------------------------------------- #


def _weight_geometry(weights: torch.Tensor, n_kernels: int, in_channels: int, out_major: bool = False):
    if out_major:
        if weights.ndim != 3 or weights.shape[0] != n_kernels or weights.shape[2] != in_channels:
            raise ValueError('dequantised convolution weights must have shape (K, C_out, C_in).')
        return 2, Triple(n_kernels, 1, 1), int(weights.shape[1])
    if weights.ndim == 3:
        if weights.shape[0] != n_kernels:
            raise ValueError('weight kernel rows must match the convolution kernel.')
        if weights.shape[1] != in_channels:
            raise ValueError('weight input channels must match x.channels.')
        return 0, Triple(n_kernels, 1, 1), int(weights.shape[2])
    if weights.ndim == 5:
        if weights.shape[4] != in_channels:
            raise ValueError('weight input channels must match x.channels.')
        kx, ky, kz = (int(v) for v in weights.shape[1:4])
        if kx * ky * kz != n_kernels:
            raise ValueError('weight kernel rows must match the convolution kernel.')
        return 1, Triple(kx, ky, kz), int(weights.shape[0])
    raise ValueError(
        'mapped convolution weight must have shape (K, C_in, C_out) '
        'or (C_out, Kx, Ky, Kz, C_in).'
    )


def sparse_conv_features(
    feats, weights, in_rows, out_rows, kernel_ids, counts, row_offsets,
    in_row_offsets=None, in_edge_ids=None, kernel_row_offsets=None, kernel_edge_ids=None,
    out_capacity=None, n_kernels=None, *, bias=None, row_order=None, plan=None, feats2=None,
    out_major=False,
):
    """``_ext.sparse_conv_features`` (``convolution.cpp:90-146``). The four grouped
    view arguments are accepted for signature compatibility; the forward pass does
    not read them. ``feats2`` (optional, same rows) supplies the trailing input channels:
    the convolution reads the channel concatenation ``[feats | feats2]`` in place.
    ``out_major`` marks ``weights`` as the ``(K, C_out, C_in)`` array of
    ``dequantize_conv_weights`` (tensor-core route only)."""
    feats, stride = _feats_arg(feats)
    feats2, stride2, c2 = _second_source(feats, feats2)
    _require_cuda(weights, 'weights')
    if weights.dtype != feats.dtype:
        raise ValueError('convolution weights must match feature dtype.')
    dtype = _dtype_code(feats.dtype)
    weights = weights.contiguous()
    in_rows, out_rows, kernel_ids = (_i32(t, n) for t, n in (
        (in_rows, 'in_rows'), (out_rows, 'out_rows'), (kernel_ids, 'kernel_ids')))
    if not (in_rows.shape == out_rows.shape == kernel_ids.shape):
        raise ValueError('in_rows, out_rows and kernel_ids must have the same length.')
    counts, row_offsets = _i32(counts, 'counts'), _i32(row_offsets, 'row_offsets')
    out_capacity, n_kernels = int(out_capacity), int(n_kernels)
    if row_offsets.shape[0] != out_capacity + 1:
        raise ValueError('row_offsets must have length out_capacity + 1.')
    c_in = int(feats.shape[1]) + c2
    layout, shape, c_out = _weight_geometry(weights, n_kernels, c_in, out_major)
    device = feats.device
    bias = _vec_arg(bias, 'bias', c_out, feats)
    row_order, plan = _order_and_plan(row_order, plan, out_capacity, n_kernels, device)
    out = torch.empty((out_capacity, c_out), dtype=feats.dtype, device=device)
    lib = _lib()
    ws = _workspace(lib.lat_sparse_conv_workspace_bytes(n_kernels, c_in, c_out), device)
    info = {'c_in': c_in, 'c_out': c_out, 'n_kernels': n_kernels, 'bits': 0, 'counts': counts,
            'in_rows': int(feats.shape[0]), 'out_rows': out_capacity,
            'tensor_cores': conv_uses_tensor_cores(feats.dtype, n_kernels, c_in, c_out)}
    with torch.cuda.device(device):
        _profiled('conv', info, lambda: check(lib.lat_sparse_conv_features(
            dtype, _ptr(feats), int(feats.shape[0]), c_in, stride, _ptr(feats2), c2, stride2,
            _ptr(weights), layout, shape,
            c_out, _ptr(in_rows), _ptr(out_rows), _ptr(kernel_ids), int(in_rows.shape[0]),
            _ptr(counts), _ptr(row_offsets), out_capacity, n_kernels, _ptr(bias),
            _ptr(row_order), _ptr(plan), _ptr(out), _ptr(ws), ws.numel(),
            _ptr(status_word(device)), _stream(),
        )))
    return out


def sparse_quantized_conv_features(
    feats, weights, scales, biases, in_rows, out_rows, kernel_ids, counts, row_offsets,
    sorted_kv_out_in_map=None, reorder_rows=None, tile_masks=None,
    out_capacity=None, n_kernels=None, in_channels=None, out_channels=None,
    storage_in_channels=None, group_size=None, bits=None, *, bias=None, row_order=None,
    plan=None, feats2=None,
):
    """``_ext.sparse_quantized_conv_features`` (``convolution.cpp:12-89``). The
    three sorted-plan arrays may be empty in the reference call; here a non-empty
    ``reorder_rows`` is used as the row permutation of the tensor-core tiles."""
    feats, stride = _feats_arg(feats)
    feats2, stride2, c2 = _second_source(feats, feats2)
    dtype = _dtype_code(feats.dtype)
    for tensor, name in ((weights, 'weights'), (scales, 'scales'), (biases, 'biases')):
        _require_cuda(tensor, name)
    if weights.dtype != torch.uint32 and weights.dtype != torch.int32:
        raise ValueError('packed weight must be a three-dimensional uint32 array.')
    if scales.dtype != feats.dtype or biases.dtype != feats.dtype:
        raise ValueError('features must match quantized scale dtype.')
    n_kernels, out_capacity = int(n_kernels), int(out_capacity)
    in_channels, out_channels = int(in_channels), int(out_channels)
    storage, group_size, bits = int(storage_in_channels), int(group_size), int(bits)
    if feats.shape[1] + c2 != in_channels:
        raise ValueError('quantized weight input channels must match x.channels.')
    if bits not in (4, 8):
        raise ValueError('quantized convolution supports only 4 or 8 bits.')
    if group_size not in (32, 64, 128):
        raise ValueError('quantized convolution group_size must be 32, 64, or 128.')
    if storage % group_size != 0 or storage < in_channels:
        raise ValueError('packed storage channels must be divisible by group_size.')
    words, groups = storage * bits // 32, storage // group_size
    if tuple(weights.shape) != (n_kernels, words, out_channels):
        raise ValueError('packed weight must have shape (K, S * bits / 32, C_out).')
    if tuple(scales.shape) != (n_kernels, groups, out_channels) or scales.shape != biases.shape:
        raise ValueError('scales and biases must have shape (K, C_out, G).')
    weights, scales, biases = weights.contiguous(), scales.contiguous(), biases.contiguous()
    in_rows, out_rows, kernel_ids = (_i32(t, n) for t, n in (
        (in_rows, 'in_rows'), (out_rows, 'out_rows'), (kernel_ids, 'kernel_ids')))
    counts, row_offsets = _i32(counts, 'counts'), _i32(row_offsets, 'row_offsets')
    if row_offsets.shape[0] != out_capacity + 1:
        raise ValueError('row_offsets must have length out_capacity + 1.')
    if row_order is None and reorder_rows is not None and reorder_rows.numel() == out_capacity:
        row_order = _i32(reorder_rows, 'reorder_rows')
    device = feats.device
    bias = _vec_arg(bias, 'bias', out_channels, feats)
    row_order, plan = _order_and_plan(row_order, plan, out_capacity, n_kernels, device)
    out = torch.empty((out_capacity, out_channels), dtype=feats.dtype, device=device)
    lib = _lib()
    ws = _workspace(lib.lat_sparse_conv_workspace_bytes(n_kernels, in_channels, out_channels), device)
    info = {'c_in': in_channels, 'c_out': out_channels, 'n_kernels': n_kernels, 'bits': bits,
            'counts': counts, 'in_rows': int(feats.shape[0]), 'out_rows': out_capacity,
            'tensor_cores': conv_uses_tensor_cores(
                feats.dtype, n_kernels, in_channels, out_channels, bits, group_size)}
    with torch.cuda.device(device):
        _profiled('conv', info, lambda: check(lib.lat_sparse_quantized_conv_features(
            dtype, _ptr(feats), int(feats.shape[0]), stride, _ptr(feats2), c2, stride2,
            _ptr(weights), _ptr(scales), _ptr(biases), _ptr(in_rows), _ptr(out_rows), _ptr(kernel_ids),
            int(in_rows.shape[0]), _ptr(counts), _ptr(row_offsets), out_capacity, n_kernels,
            in_channels, out_channels, storage, group_size, bits, _ptr(bias), _ptr(row_order),
            _ptr(plan), _ptr(out), _ptr(ws), ws.numel(), _ptr(status_word(device)), _stream(),
        )))
    return out


def dequantize_conv_weights(weights, scales, biases, in_channels: int, out_channels: int,
                            storage_in_channels: int, group_size: int, bits: int) -> torch.Tensor:
    """The fp16 ``(K, C_out, C_in)`` weights a packed convolution weight stands for
    (``lat_dequantize_conv_weights``): what the tensor-core route of the quantized
    convolution would make in its workspace on every call."""
    for tensor, name in ((weights, 'weights'), (scales, 'scales'), (biases, 'biases')):
        _require_cuda(tensor, name)
    if scales.dtype != torch.float16 or biases.dtype != torch.float16:
        raise ValueError('dequantised convolution weights need float16 scales and biases.')
    n_kernels = int(weights.shape[0])
    words, groups = storage_in_channels * bits // 32, storage_in_channels // group_size
    if tuple(weights.shape) != (n_kernels, words, out_channels):
        raise ValueError('packed weight must have shape (K, S * bits / 32, C_out).')
    if tuple(scales.shape) != (n_kernels, groups, out_channels) or scales.shape != biases.shape:
        raise ValueError('scales and biases must have shape (K, C_out, G).')
    weights, scales, biases = weights.contiguous(), scales.contiguous(), biases.contiguous()
    out = torch.empty((n_kernels, out_channels, in_channels), dtype=torch.float16, device=weights.device)
    with torch.cuda.device(weights.device):
        check(_lib().lat_dequantize_conv_weights(
            _ptr(weights), _ptr(scales), _ptr(biases), n_kernels, int(in_channels), int(out_channels),
            int(storage_in_channels), int(group_size), int(bits), _ptr(out), _stream()))
    return out


def _order_and_plan(row_order, plan, out_capacity: int, n_kernels: int, device):
    """Validated optional row permutation and gather plan of a convolution call."""
    if row_order is not None:
        row_order = _i32(row_order, 'row_order')
        if row_order.device != device or row_order.numel() != out_capacity:
            raise ValueError('row_order must hold one int32 entry per output row, on the feature device.')
    if plan is not None:
        _require_cuda(plan, 'plan')
        need = int(_lib().lat_conv_plan_bytes(out_capacity, n_kernels)) if n_kernels <= 32 else 0
        if (plan.device != device or plan.dtype != torch.uint8 or not plan.is_contiguous()
                or plan.numel() < need):
            raise ValueError('plan must be the uint8 buffer build_conv_plan returned for this relation.')
    return row_order, plan


def conv_uses_tensor_cores(dtype, n_kernels, in_channels, out_channels, bits=0, group_size=0) -> bool:
    return bool(_lib().lat_conv_uses_tensor_cores(
        _dtype_code(dtype), n_kernels, in_channels, out_channels, bits, group_size))


def build_conv_plan(in_rows, kernel_ids, counts, row_offsets, in_capacity: int,
                    out_capacity: int, kernel_count: int, row_order=None, row_masks=None) -> torch.Tensor:
    """Gather plan of the tensor-core convolution over one relation
    (``lat_build_conv_plan``): per 256-row tile of ``row_order`` the mask of kernel
    offsets in use and, per used offset, the input row of every tile row. ``row_masks``
    (optional, ``(out_capacity, 1)`` int32, the relation's own) saves a walk over the edges."""
    in_rows, kernel_ids = _i32(in_rows, 'in_rows'), _i32(kernel_ids, 'kernel_ids')
    counts, row_offsets = _i32(counts, 'counts'), _i32(row_offsets, 'row_offsets')
    device = in_rows.device
    out_capacity = int(out_capacity)
    if kernel_ids.shape != in_rows.shape or any(t.device != device for t in (kernel_ids, counts, row_offsets)):
        raise ValueError('in_rows and kernel_ids must have the same length, on one device.')
    if row_offsets.numel() != out_capacity + 1 or counts.numel() != 2:
        raise ValueError('row_offsets must have length out_capacity + 1 and counts two entries.')
    if row_order is not None:
        row_order = _i32(row_order, 'row_order')
        if row_order.device != device or row_order.numel() != out_capacity:
            raise ValueError('row_order must hold one int32 entry per output row, on the relation device.')
    if row_masks is not None:
        row_masks = _i32(row_masks, 'row_masks')
        if row_masks.device != device or row_masks.numel() != out_capacity:
            raise ValueError('row_masks must hold one int32 word per output row, on the relation device.')
    lib = _lib()
    plan = torch.empty(max(int(lib.lat_conv_plan_bytes(out_capacity, kernel_count)), 256),
                       dtype=torch.uint8, device=device)
    with torch.cuda.device(device):
        check(lib.lat_build_conv_plan(
            _ptr(in_rows), _ptr(kernel_ids), int(in_rows.shape[0]), _ptr(counts),
            _ptr(row_offsets), int(in_capacity), out_capacity, int(kernel_count),
            _ptr(row_order), _ptr(row_masks), _ptr(plan), plan.numel(), _ptr(status_word(device)),
            _stream(),
        ))
    return plan


def build_mask_row_order(row_masks, counts, kernel_count: int = 32):
    """Row permutation grouping output rows by equal offset mask (K <= 32)."""
    row_masks = _i32(row_masks, 'row_masks')
    if row_masks.ndim != 2 or row_masks.shape[1] != 1:
        raise ValueError('sorted implicit GEMM view currently supports K <= 32.')
    rows = int(row_masks.shape[0])
    device = row_masks.device
    order = torch.empty(rows, dtype=torch.int32, device=device)
    lib = _lib()
    ws = _workspace(lib.lat_mask_order_workspace_bytes(rows), device)
    with torch.cuda.device(device):
        check(lib.lat_build_mask_row_order(
            _ptr(row_masks), rows, int(kernel_count), _ptr(_i32(counts, 'counts')), _ptr(order), _ptr(ws),
            ws.numel(), _ptr(status_word(device)), _stream(),
        ))
    return order


# --------------------------------------------------------------------------- #
# pooling and pointwise feature ops
# --------------------------------------------------------------------------- #


def sparse_pool_features(
    feats, in_rows, out_rows, kernel_ids, row_offsets, counts, input_exclusive, reduce,
    out_capacity, n_kernels,
):
    """``_ext.sparse_pool_features`` (``native/bindings/pooling.cpp:17-72``)."""
    feats, stride = _feats_arg(feats)
    if feats.dtype != torch.float32:
        raise ValueError('pooling currently supports float32 tensors.')
    if reduce not in _REDUCE:
        raise ValueError("reduce must be 'sum', 'max', or 'avg'.")
    in_rows, out_rows, kernel_ids = (_i32(t, n) for t, n in (
        (in_rows, 'in_rows'), (out_rows, 'out_rows'), (kernel_ids, 'kernel_ids')))
    row_offsets, counts = _i32(row_offsets, 'row_offsets'), _i32(counts, 'counts')
    out_capacity = int(out_capacity)
    if row_offsets.shape[0] != out_capacity + 1:
        raise ValueError('row_offsets must have length out_capacity + 1.')
    device = feats.device
    out = torch.empty((out_capacity, feats.shape[1]), dtype=torch.float32, device=device)
    with torch.cuda.device(device):
        check(_lib().lat_sparse_pool_features(
            _ptr(feats), int(feats.shape[0]), int(feats.shape[1]), stride, _ptr(in_rows),
            _ptr(out_rows), _ptr(kernel_ids), int(in_rows.shape[0]), _ptr(row_offsets),
            _ptr(counts), int(bool(input_exclusive)), _REDUCE[reduce], out_capacity,
            int(n_kernels), _ptr(out), _ptr(status_word(device)), _stream(),
        ))
    return out


def global_pool(feats, batch_offsets, reduce: str):
    feats, _ = _feats_arg(feats)
    feats = feats.contiguous()
    if feats.dtype != torch.float32:
        raise ValueError('pooling currently supports float32 tensors.')
    batch_offsets = _i32(batch_offsets, 'batch_offsets')
    batches = int(batch_offsets.shape[0]) - 1
    out = torch.empty((batches, feats.shape[1]), dtype=torch.float32, device=feats.device)
    with torch.cuda.device(feats.device):
        check(_lib().lat_global_pool(
            _ptr(feats), int(feats.shape[0]), int(feats.shape[1]), _ptr(batch_offsets), batches,
            _REDUCE[reduce], _ptr(out), _stream(),
        ))
    return out


# identity gather plans of the tensor-core linear, by (device index, rows): they depend on the
# row count only, so the few most recent ones are kept
_identity_plans: dict = {}
_TC_LINEAR_MIN_ROWS = 4096


def _identity_plan(rows: int, device: torch.device) -> torch.Tensor:
    key = (device.index, rows)
    plan = _identity_plans.get(key)
    if plan is None:
        lib = _lib()
        plan = torch.empty(max(int(lib.lat_conv_plan_bytes(rows, 1)), 256), dtype=torch.uint8, device=device)
        with torch.cuda.device(device):
            check(lib.lat_build_identity_conv_plan(rows, _ptr(plan), plan.numel(), _stream()))
        while len(_identity_plans) >= 8:
            _identity_plans.pop(next(iter(_identity_plans)))
        _identity_plans[key] = plan
    return plan


def linear(feats, weight, bias=None):
    """``feats @ weight.T + bias`` (``mlx_lattice/ops/feature.py:33-51``). float16 matrices
    whose shapes the tcgen05 tiles cover run on the tensor cores (the convolution kernel
    over the identity relation); everything else on the CUDA-core kernel."""
    feats, stride = _feats_arg(feats)
    _require_cuda(weight, 'weight')
    if (feats.dtype == torch.float16 and weight.dtype == torch.float16 and weight.ndim == 2
            and weight.shape[1] == feats.shape[1] and weight.device == feats.device
            and feats.shape[0] >= _TC_LINEAR_MIN_ROWS and stride % 8 == 0 and feats.data_ptr() % 16 == 0
            and _lib().lat_linear_uses_tensor_cores(1, int(feats.shape[1]), int(weight.shape[0]))):
        weight = weight.contiguous()
        bias = _vec_arg(bias, 'bias', weight.shape[0], feats)
        rows = int(feats.shape[0])
        out = torch.empty((rows, weight.shape[0]), dtype=feats.dtype, device=feats.device)
        plan = _identity_plan(rows, feats.device)
        with torch.cuda.device(feats.device):
            check(_lib().lat_linear_tensor_cores(
                _ptr(feats), rows, int(feats.shape[1]), stride, _ptr(weight), int(weight.shape[0]),
                _ptr(bias), _ptr(plan), _ptr(out), _ptr(status_word(feats.device)), _stream()))
        return out
    feats = feats.contiguous()
    if weight.dtype != feats.dtype:
        raise ValueError('convolution weights must match feature dtype.')
    if weight.ndim != 2 or weight.shape[1] != feats.shape[1] or weight.device != feats.device:
        raise ValueError('linear weight must have shape (C_out, C_in) on the feature device.')
    weight = weight.contiguous()
    bias = _vec_arg(bias, 'bias', weight.shape[0], feats)
    out = torch.empty((feats.shape[0], weight.shape[0]), dtype=feats.dtype, device=feats.device)
    with torch.cuda.device(feats.device):
        check(_lib().lat_linear(
            _dtype_code(feats.dtype), _ptr(feats), int(feats.shape[0]), int(feats.shape[1]),
            _ptr(weight), int(weight.shape[0]), _ptr(bias), _ptr(out), _stream(),
        ))
    return out


def quantized_linear(
    feats, packed, scales, biases, out_channels, storage_in_channels, group_size, bits, bias=None
):
    feats, _ = _feats_arg(feats)
    feats = feats.contiguous()
    out_channels, storage, group_size, bits = (int(out_channels), int(storage_in_channels),
                                               int(group_size), int(bits))
    if bits not in (4, 8) or group_size not in (32, 64, 128):
        raise ValueError('quantized linear supports 4 or 8 bits and group_size 32, 64, or 128.')
    if storage % group_size != 0 or storage < feats.shape[1]:
        raise ValueError('packed storage channels must be divisible by group_size.')
    for tensor, name in ((packed, 'packed'), (scales, 'scales'), (biases, 'biases')):
        _require_cuda(tensor, name)
        if tensor.device != feats.device:
            raise ValueError(f'{name} must be on the same device as the features.')
    if packed.dtype not in (torch.uint32, torch.int32) or tuple(packed.shape) != (out_channels, storage * bits // 32):
        raise ValueError('packed weight must have shape (C_out, S * bits / 32) and uint32 dtype.')
    if scales.dtype != feats.dtype or biases.dtype != feats.dtype:
        raise ValueError('features must match quantized scale dtype.')
    if tuple(scales.shape) != (out_channels, storage // group_size) or scales.shape != biases.shape:
        raise ValueError('scales and biases must have shape (C_out, S / group_size).')
    bias = _vec_arg(bias, 'bias', out_channels, feats)
    out = torch.empty((feats.shape[0], out_channels), dtype=feats.dtype, device=feats.device)
    with torch.cuda.device(feats.device):
        check(_lib().lat_quantized_linear(
            _dtype_code(feats.dtype), _ptr(feats), int(feats.shape[0]), int(feats.shape[1]),
            _ptr(packed.contiguous()), _ptr(scales.contiguous()), _ptr(biases.contiguous()),
            int(out_channels), int(storage_in_channels), int(group_size), int(bits), _ptr(bias),
            _ptr(out), _stream(),
        ))
    return out


def batch_norm_relu(feats, weight, bias, mean, var, eps: float, apply_relu: bool):
    feats, _ = _feats_arg(feats)
    feats = feats.contiguous()
    channels = int(feats.shape[1])
    weight, bias = _vec_arg(weight, 'weight', channels, feats), _vec_arg(bias, 'bias', channels, feats)
    mean, var = _vec_arg(mean, 'mean', channels, feats), _vec_arg(var, 'var', channels, feats)
    if mean is None or var is None:
        raise ValueError('batch_norm needs mean and var.')
    out = torch.empty_like(feats)
    with torch.cuda.device(feats.device):
        check(_lib().lat_batch_norm_relu(
            _dtype_code(feats.dtype), _ptr(feats), int(feats.shape[0]), int(feats.shape[1]),
            _ptr(weight), _ptr(bias), _ptr(mean), _ptr(var), float(eps), int(apply_relu),
            _ptr(out), _stream(),
        ))
    return out


_ACTIVATIONS = {
    'sigmoid': 0, 'silu': 1, 'tanh': 2, 'gelu_erf': 3, 'gelu_tanh': 4, 'gelu_fast': 5,
    'leaky_relu': 6, 'softplus': 7,
}


def activation(feats, name: str, p0: float = 0.0, p1: float = 0.0):
    """Pointwise activation of a feature matrix (``mlx_lattice/ops/feature.py:59-129``)."""
    feats, _ = _feats_arg(feats)
    feats = feats.contiguous()
    out = torch.empty_like(feats)
    with torch.cuda.device(feats.device):
        check(_lib().lat_activation(
            _dtype_code(feats.dtype), _ACTIVATIONS[name], _ptr(feats), feats.numel(), float(p0),
            float(p1), _ptr(out), _stream(),
        ))
    return out


def row_norm(feats, weight, bias, eps: float, rms: bool):
    """``layer_norm`` (``rms`` false) or ``rms_norm`` over the channels of every row."""
    feats, _ = _feats_arg(feats)
    feats = feats.contiguous()
    channels = int(feats.shape[1])
    for vector, name in ((weight, 'weight'), (bias, 'bias')):
        if vector is not None:
            _require_cuda(vector, name)
            if tuple(vector.shape) != (channels,):
                raise ValueError(f'{name} must have shape ({channels},).')
            if vector.dtype != feats.dtype:
                raise ValueError(f'{name} must match the feature dtype.')
    out = torch.empty_like(feats)
    with torch.cuda.device(feats.device):
        check(_lib().lat_row_norm(
            _dtype_code(feats.dtype), int(bool(rms)), _ptr(feats), int(feats.shape[0]), channels,
            _ptr(None if weight is None else weight.contiguous()),
            _ptr(None if bias is None else bias.contiguous()), float(eps), _ptr(out), _stream(),
        ))
    return out


def relu(feats):
    feats, _ = _feats_arg(feats)
    feats = feats.contiguous()
    out = torch.empty_like(feats)
    with torch.cuda.device(feats.device):
        check(_lib().lat_relu(
            _dtype_code(feats.dtype), _ptr(feats), feats.numel(), _ptr(out), _stream()
        ))
    return out


# --------------------------------------------------------------------------- #
# features through an alignment (mlx_lattice/ops/tensor.py:89-147, :228-249)
# --------------------------------------------------------------------------- #

_BINARY_OPS = {'add': 0, 'sub': 1, 'mul': 2, 'maximum': 3, 'minimum': 4}


def _aligned_pair(lhs, lhs_rows, rhs, rhs_rows):
    lhs, _ = _feats_arg(lhs)
    rhs, _ = _feats_arg(rhs)
    lhs, rhs = lhs.contiguous(), rhs.contiguous()
    if lhs.dtype != rhs.dtype:
        raise ValueError('sparse tensors must have matching feature dtype.')
    if (lhs_rows is None) != (rhs_rows is None):
        raise ValueError('row maps must be given for both sides or for neither.')
    if lhs_rows is None:
        if lhs.shape[0] != rhs.shape[0]:
            raise ValueError('tensors that share coordinates must have the same number of rows.')
        rows_out = int(lhs.shape[0])
    else:
        lhs_rows, rhs_rows = _i32(lhs_rows, 'lhs_rows'), _i32(rhs_rows, 'rhs_rows')
        if lhs_rows.ndim != 1 or lhs_rows.shape != rhs_rows.shape:
            raise ValueError('rows must have shape (N,) and int32 dtype.')
        rows_out = int(lhs_rows.shape[0])
    return lhs, lhs_rows, rhs, rhs_rows, rows_out


def concat_aligned_features(lhs, lhs_rows, rhs, rhs_rows):
    """``[lhs[lhs_rows] | rhs[rhs_rows]]`` along the channels, zero rows where a map holds
    -1; ``None`` maps mean the two matrices already share their rows."""
    lhs, lhs_rows, rhs, rhs_rows, rows_out = _aligned_pair(lhs, lhs_rows, rhs, rhs_rows)
    channels = int(lhs.shape[1]) + int(rhs.shape[1])
    out = torch.empty((rows_out, channels), dtype=lhs.dtype, device=lhs.device)
    with torch.cuda.device(lhs.device):
        check(_lib().lat_concat_aligned_features(
            lhs.element_size(), _ptr(lhs), _ptr(lhs_rows), int(lhs.shape[0]), int(lhs.shape[1]),
            _ptr(rhs), _ptr(rhs_rows), int(rhs.shape[0]), int(rhs.shape[1]), rows_out, _ptr(out),
            _ptr(status_word(lhs.device)), _stream(),
        ))
    return out


def binary_aligned_features(lhs, lhs_rows, rhs, rhs_rows, op: str, lhs_fill=0.0, rhs_fill=0.0):
    """``op(lhs[lhs_rows] or lhs_fill, rhs[rhs_rows] or rhs_fill)`` row by row."""
    if op not in _BINARY_OPS:
        raise ValueError(f'unknown sparse binary op: {op}.')
    lhs, lhs_rows, rhs, rhs_rows, rows_out = _aligned_pair(lhs, lhs_rows, rhs, rhs_rows)
    if lhs.shape[1] != rhs.shape[1]:
        raise ValueError('sparse binary operands must have matching channels.')
    out = torch.empty((rows_out, int(lhs.shape[1])), dtype=lhs.dtype, device=lhs.device)
    with torch.cuda.device(lhs.device):
        check(_lib().lat_binary_aligned_features(
            _dtype_code(lhs.dtype), _BINARY_OPS[op], _ptr(lhs), _ptr(lhs_rows), int(lhs.shape[0]),
            float(lhs_fill), _ptr(rhs), _ptr(rhs_rows), int(rhs.shape[0]), float(rhs_fill),
            rows_out, int(lhs.shape[1]), _ptr(out), _ptr(status_word(lhs.device)), _stream(),
        ))
    return out
