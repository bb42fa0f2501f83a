"""CPU-side checks of the C-ABI library: it loads, exports every function the header declares,
rejects bad arguments with an error code and message, and the host-side adjacency build matches
the oracle.  No GPU is needed (no kernel is launched)."""
import ctypes
import os
import re

import numpy as np
import pytest

from helpers import graph
from orca_b200 import _lib, build
from oracle import tgn_oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    build.build()
    return _lib.lib()


def _declared():
    text = open(os.path.join(ROOT, "include", "orca_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(orca_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(L):
    names = _declared()
    assert len(names) >= 20
    for n in names:
        assert hasattr(L, n), f"{n} is declared in include/orca_b200.h but not exported"
        assert n in _lib.SYMBOLS, f"{n} has no ctypes signature in orca_b200/_lib.py"
    assert sorted(_lib.SYMBOLS) == names


def test_bad_arguments_return_codes(L):
    assert L.orca_version() >= 1
    rc = L.orca_sample_topk(None, None, None, None, 10, None, None, 4, None, 10, None, None, None, None, None, None)
    assert rc == 1
    assert b"orca_sample_topk" in L.orca_last_error()
    assert L.orca_eval_workspace_bytes(0, 0, 10, 100) == -1
    assert L.orca_eval_workspace_bytes(200, 600, 10, 1501) > 0


@pytest.mark.parametrize("spec", ["t_nb2", "t_bip2", "c1"])
def test_csr_build_host_matches_oracle(L, spec):
    g = graph(spec)
    E, n = g.n_edges, g.n_nodes
    indptr = np.empty(n + 1, dtype=np.int64)
    nbr = np.empty(2 * E, dtype=np.int32)
    eid = np.empty(2 * E, dtype=np.int32)
    ts = np.empty(2 * E, dtype=np.float64)
    src, dst, eidx = (np.ascontiguousarray(a, dtype=np.int64) for a in (g.sources, g.destinations, g.edge_idxs))
    rc = L.orca_csr_build_host(src.ctypes.data, dst.ctypes.data, eidx.ctypes.data, g.timestamps.ctypes.data, E, n,
                               indptr.ctypes.data, nbr.ctypes.data, eid.ctypes.data, ts.ctypes.data)
    assert rc == 0
    adj = tgn_oracle.Adjacency(g.sources, g.destinations, g.edge_idxs, g.timestamps, n)
    assert np.array_equal(indptr, adj.indptr)
    assert np.array_equal(nbr, adj.nbr) and np.array_equal(eid, adj.eid) and np.array_equal(ts, adj.ts)


def test_csr_build_host_unsorted_stream_and_ties(L):
    rs = np.random.RandomState(0)
    E, n = 5000, 60
    src = rs.randint(1, n, E).astype(np.int64)
    dst = rs.randint(1, n, E).astype(np.int64)
    ts = rs.randint(0, 50, E).astype(np.float64)   # unsorted, many equal times, self loops allowed
    eidx = np.arange(1, E + 1, dtype=np.int64)
    indptr = np.empty(n + 1, dtype=np.int64)
    nbr = np.empty(2 * E, dtype=np.int32)
    eid = np.empty(2 * E, dtype=np.int32)
    ats = np.empty(2 * E, dtype=np.float64)
    rc = L.orca_csr_build_host(src.ctypes.data, dst.ctypes.data, eidx.ctypes.data, ts.ctypes.data, E, n,
                               indptr.ctypes.data, nbr.ctypes.data, eid.ctypes.data, ats.ctypes.data)
    assert rc == 0
    adj = tgn_oracle.Adjacency(src, dst, eidx, ts, n)
    assert np.array_equal(indptr, adj.indptr)
    assert np.array_equal(nbr, adj.nbr) and np.array_equal(eid, adj.eid) and np.array_equal(ats, adj.ts)
    bad = src.copy()
    bad[3] = n + 5
    rc = L.orca_csr_build_host(bad.ctypes.data, dst.ctypes.data, eidx.ctypes.data, ts.ctypes.data, E, n,
                               indptr.ctypes.data, nbr.ctypes.data, eid.ctypes.data, ats.ctypes.data)
    assert rc == 5


def test_no_fallback_without_cuda():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from orca_b200.history import History
    with pytest.raises(RuntimeError):
        History(10, 172, device="cuda")
    with pytest.raises(RuntimeError):
        History(10, 172, device="cpu")
