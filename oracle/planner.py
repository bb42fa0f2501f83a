"""TEST INFRASTRUCTURE ONLY -- CPU restatement of the reference's offline cache planning.

`read_batches` restates utils/cache.py:19-89 in numpy; the three solvers are the C functions of
planner_oracle.c (loaded with ctypes from oracle/_build, built by oracle/Makefile).  Nothing that
ships may import this module.
"""
from __future__ import annotations

import ctypes
import math
import os
import subprocess

import numpy as np

from .tgn_oracle import Adjacency, sample_neighbors

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build():
    subprocess.check_call(["make", "-s", "-C", _HERE])


def _lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "_build", "liborca_oracle.so")
        if not os.path.exists(path):
            build()
        _LIB = ctypes.CDLL(path)
    return _LIB


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def read_batches(sources, destinations, timestamps, bs, k, adj: Adjacency, n_nodes):
    """utils/cache.py:19-89.  Per batch: sample the neighbours of [sources | destinations], drop
    padding, split the neighbour occurrences into in-batch (also a target of the batch) and
    out-of-batch; targets are the sorted unique query nodes.  Returns flattened lists
    (tgt_off, tgt, ngh_off, ngh) and the per-node occurrence records (occ_off, occ_batch,
    occ_kind): record 0 of a node is the dummy (0, 0), then one record per batch in which it is a
    target (kind 0) or an out-of-batch neighbour (kind 1), then the terminator (num_batch, 2)."""
    E = len(sources)
    nb = math.ceil(E / bs)
    tgt_l, ngh_l = [], []
    occ_node, occ_b, occ_k = [], [], []
    for b in range(nb):
        s, e = b * bs, min(E, (b + 1) * bs)
        q = np.concatenate([sources[s:e], destinations[s:e]])
        t = np.concatenate([timestamps[s:e], timestamps[s:e]])
        nbr, _, _ = sample_neighbors(adj, q, t, k)
        flat = nbr.reshape(-1)
        flat = flat[flat != 0]
        tgt = np.unique(q)
        out = flat[~np.isin(flat, tgt)]
        uo = np.unique(out)
        tgt_l.append(tgt.astype(np.int64))
        ngh_l.append(out.astype(np.int32))
        occ_node += [tgt, uo]
        occ_b += [np.full(len(tgt), b), np.full(len(uo), b)]
        occ_k += [np.zeros(len(tgt), np.uint8), np.ones(len(uo), np.uint8)]
    node = np.concatenate(occ_node + [np.arange(n_nodes), np.arange(n_nodes)]).astype(np.int64)
    bat = np.concatenate(occ_b + [np.full(n_nodes, -1), np.full(n_nodes, nb)]).astype(np.int64)
    kind = np.concatenate(occ_k + [np.zeros(n_nodes, np.uint8), np.full(n_nodes, 2, np.uint8)])
    order = np.lexsort((bat, node))
    occ_off = np.zeros(n_nodes + 1, dtype=np.int64)
    np.cumsum(np.bincount(node, minlength=n_nodes), out=occ_off[1:])
    occ_batch = bat[order].astype(np.int32)
    occ_batch[occ_off[:-1]] = 0  # the dummy record is (0, 0)
    occ_kind = kind[order]

    def flat_off(lst, dt):
        off = np.zeros(len(lst) + 1, dtype=np.int64)
        np.cumsum([len(a) for a in lst], out=off[1:])
        return off, (np.concatenate(lst).astype(dt) if lst else np.zeros(0, dt))

    tgt_off, tgt = flat_off(tgt_l, np.int64)
    ngh_off, ngh = flat_off(ngh_l, np.int32)
    return dict(num_batch=nb, tgt_off=tgt_off, tgt=tgt, ngh_off=ngh_off, ngh=ngh,
                occ_off=occ_off, occ_batch=occ_batch, occ_kind=np.ascontiguousarray(occ_kind))


def solve(strategy, rb, n_nodes, budget, seed=0):
    """Runs one solver over the lists of `read_batches`; returns (list of int64 arrays, stats)
    where stats = (n_reuse, n_recompute, average reuse distance) as printed by
    utils/cache.py:427."""
    lib = _lib()
    nb = rb["num_batch"]
    plan_flat = np.zeros(nb * (budget + 2) + 8, dtype=np.int64)
    plan_off = np.zeros(nb + 1, dtype=np.int64)
    stats = np.zeros(3, dtype=np.float64)
    i64 = ctypes.c_int64
    if strategy == "MRD":
        rc = lib.mrd_plan(i64(n_nodes), i64(nb), i64(budget), _p(rb["tgt_off"]), _p(rb["tgt"]),
                          _p(rb["ngh_off"]), _p(rb["ngh"]), _p(rb["occ_off"]), _p(rb["occ_batch"]),
                          _p(rb["occ_kind"]), _p(plan_flat), _p(plan_off), _p(stats))
    elif strategy == "LRU":
        rc = lib.lru_plan(i64(n_nodes), i64(nb), i64(budget), _p(rb["ngh_off"]), _p(rb["ngh"]),
                          ctypes.c_uint32(seed), _p(plan_flat), _p(plan_off), _p(stats))
    elif strategy == "2Q":
        rc = lib.twoq_plan(i64(n_nodes), i64(nb), i64(budget), _p(rb["ngh_off"]), _p(rb["ngh"]),
                           ctypes.c_uint32(seed), _p(plan_flat), _p(plan_off), _p(stats))
    else:
        raise ValueError(f"unsupported cache strategy {strategy}")
    assert rc == 0
    plan = [plan_flat[plan_off[b]:plan_off[b + 1]].copy() for b in range(nb)]
    avg = stats[2] / stats[0] if stats[0] else float("nan")
    return plan, (int(stats[0]), int(stats[1]), avg)


def get_cache_plan(sources, destinations, timestamps, bs, k, budget, adj, n_nodes, strategy, seed=0):
    """utils/cache.py:407-428."""
    rb = read_batches(np.asarray(sources), np.asarray(destinations), np.asarray(timestamps), bs, k, adj, n_nodes)
    return solve(strategy, rb, n_nodes, budget, seed)[0]
