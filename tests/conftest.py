import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (sm_100)')


def _oracle():
    """The checker: the compiled reference CPU code when its library travelled with
    the checkout, else the numpy restatement."""
    from oracle import reference, restatement

    return reference if reference.available() else restatement


@pytest.fixture(scope='session')
def oracle():
    return _oracle()


@pytest.fixture(scope='session')
def restatement():
    from oracle import restatement as module

    return module


@pytest.fixture(scope='session')
def cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.skip('no CUDA device')
    from mlx_lattice_b200 import _native

    _native.load()  # fails loudly when the extension is not built
    return torch.device('cuda', 0)


RELATION_KEYS = ('in_rows', 'out_rows', 'kernel_ids', 'row_offsets', 'counts')


def relation_to_numpy(tuple10):
    names = ('in_rows', 'out_rows', 'kernel_ids', 'row_offsets', 'out_coords', 'counts',
             'in_row_offsets', 'in_edge_ids', 'kernel_row_offsets', 'kernel_edge_ids')
    return {name: value.cpu().numpy() for name, value in zip(names, tuple10)}


def canonical_edges(rel):
    """Edges sorted by (out_row, kernel_id, in_row)."""
    e = int(rel['counts'][0])
    triples = np.stack([rel['out_rows'][:e], rel['kernel_ids'][:e], rel['in_rows'][:e]], axis=1)
    order = np.lexsort((triples[:, 2], triples[:, 1], triples[:, 0]))
    return triples[order]


def canonical_pair_lists(rel, n_kernels):
    """Per-offset (in, out) pair lists sorted by (in, out) within each offset."""
    lists = []
    offs = rel['kernel_row_offsets']
    for k in range(n_kernels):
        ids = rel['kernel_edge_ids'][offs[k]:offs[k + 1]]
        pairs = np.stack([rel['in_rows'][ids], rel['out_rows'][ids]], axis=1)
        lists.append(pairs[np.lexsort((pairs[:, 1], pairs[:, 0]))])
    return lists


def run_ranks(target, world: int, args: tuple, timeout: float):
    """Start `world` spawned processes running target(rank, world, *args, results) and wait for
    them; a rank that is still alive after `timeout` seconds (stuck in a collective) is
    terminated, then killed, so that no worker outlives the test holding a device. Returns
    (exit codes, results queue)."""
    import torch.multiprocessing as mp

    ctx = mp.get_context('spawn')
    results = ctx.Queue()
    procs = [ctx.Process(target=target, args=(rank, world, *args, results), daemon=True)
             for rank in range(world)]
    try:
        for proc in procs:
            proc.start()
        for proc in procs:
            proc.join(timeout=timeout)
    finally:
        for proc in procs:
            if proc.is_alive():
                proc.terminate()
                proc.join(timeout=10)
            if proc.is_alive():
                proc.kill()
                proc.join()
    return [proc.exitcode for proc in procs], results
