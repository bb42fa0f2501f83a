"""Shared plumbing of the parity tests: fixtures, graphs and batch iteration."""
import functools
import os

import numpy as np

from orca_b200 import params, synthetic

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@functools.lru_cache(maxsize=None)
def golden(case):
    return dict(np.load(os.path.join(GOLDEN, f"{case}.npz"), allow_pickle=False))


@functools.lru_cache(maxsize=None)
def graph(spec_name):
    return synthetic.make_graph(spec_name)


def unpack(flat, off):
    return [flat[off[i]:off[i + 1]] for i in range(len(off) - 1)]


def batches(g, n_batches=None):
    """Yields (b, src, dst, ts, eidx) for the leading batches of the stream."""
    bs = g.spec.bs
    nb = g.n_batches if n_batches is None else min(n_batches, g.n_batches)
    for b in range(nb):
        s, e = b * bs, min(g.n_edges, (b + 1) * bs)
        yield b, g.sources[s:e], g.destinations[s:e], g.timestamps[s:e], g.edge_idxs[s:e]


def state_dict(n_layers):
    return params.random_state_dict(n_layers, seed=0)


def max_rel(a, b, floor=1e-3):
    """max |a-b| / max(|b|, floor)"""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.max(np.abs(a - b) / np.maximum(np.abs(b), floor))) if a.size else 0.0
