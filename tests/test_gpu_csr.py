"""The adjacency built on the device (orca_csr_build) against the oracle's restatement of
get_neighbor_finder (utils/util.py:91-105): same lists, same order inside every list, for streams in
time order, streams out of order with many equal timestamps and self loops, and signed timestamps."""
import types

import numpy as np
import pytest
import torch

from helpers import graph

pytestmark = pytest.mark.gpu


def _check(src, dst, eidx, ts, n):
    from oracle import tgn_oracle
    from orca_b200.neighbor_finder import NeighborFinder
    nf = NeighborFinder.build_on_device(src, dst, eidx, ts, n)
    adj = tgn_oracle.Adjacency(src, dst, eidx, ts, n)
    E = len(src)
    assert np.array_equal(nf.indptr.cpu().numpy(), adj.indptr)
    assert np.array_equal(nf.adj_nbr.cpu().numpy()[:2 * E], adj.nbr)
    assert np.array_equal(nf.adj_eid.cpu().numpy()[:2 * E], adj.eid)
    assert np.array_equal(nf.adj_ts.cpu().numpy()[:2 * E], adj.ts)
    return nf


@pytest.mark.parametrize("spec", ["t_nb2", "t_bip2", "c1", "c2"])
def test_device_build_matches_oracle(spec):
    g = graph(spec)
    _check(g.sources, g.destinations, g.edge_idxs, g.timestamps, g.n_nodes)


@pytest.mark.parametrize("E,n,span", [(5000, 60, 50), (70000, 300, 7), (40000, 70000, 1000)])
def test_unsorted_stream_ties_and_self_loops(E, n, span):
    rs = np.random.RandomState(E)
    src = rs.randint(1, n, E).astype(np.int64)
    dst = rs.randint(1, n, E).astype(np.int64)
    ts = rs.randint(0, span, E).astype(np.float64)
    _check(src, dst, np.arange(1, E + 1, dtype=np.int64), ts, n)


def test_signed_and_fractional_timestamps():
    rs = np.random.RandomState(3)
    E, n = 20000, 500
    src = rs.randint(0, n, E).astype(np.int64)
    dst = rs.randint(0, n, E).astype(np.int64)
    ts = np.round(rs.randn(E) * 1e3, 1)
    ts[::97] = 0.0
    ts[1::97] = -0.0          # equal to +0.0: the stream order decides
    ts[5::211] = 1e300
    ts[7::211] = -1e-300
    _check(src, dst, np.arange(E, dtype=np.int64), ts, n)


def test_find_before_and_sampling_on_a_device_built_finder():
    from oracle import tgn_oracle
    from orca_b200.neighbor_finder import get_neighbor_finder
    g = graph("t_nb2")
    nf = get_neighbor_finder(g, g.n_nodes - 1)
    adj = tgn_oracle.Adjacency(g.sources, g.destinations, g.edge_idxs, g.timestamps, g.n_nodes)
    v, t = int(g.sources[500]), float(g.timestamps[500])
    a, b, c = nf.find_before(v, t)
    lo = adj.indptr[v]
    i = int(np.searchsorted(adj.ts[lo:adj.indptr[v + 1]], t))
    assert np.array_equal(a, adj.nbr[lo:lo + i]) and np.array_equal(b, adj.eid[lo:lo + i])
    assert np.array_equal(c, adj.ts[lo:lo + i])
    q, qt = g.sources[:300], g.timestamps[:300]
    want = tgn_oracle.sample_neighbors(adj, q, qt, 10)
    got = nf.get_temporal_neighbor(q, qt, 10)
    for x, y in zip(got, want):
        assert np.array_equal(x, y)


def test_ids_out_of_range_are_reported_and_empty_graph_builds():
    from orca_b200 import _lib
    from orca_b200.neighbor_finder import NeighborFinder
    src = np.array([1, 2, 9], dtype=np.int64)
    with pytest.raises(_lib.OrcaError):
        NeighborFinder.build_on_device(src, src, src, np.zeros(3), 5)
    z = np.zeros(0, dtype=np.int64)
    nf = NeighborFinder.build_on_device(z, z, z, np.zeros(0), 4)
    assert np.array_equal(nf.indptr.cpu().numpy(), np.zeros(5, dtype=np.int64))
