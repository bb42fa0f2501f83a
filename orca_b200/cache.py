"""Offline cache planning with the interface of utils/cache.py:407-428.

``get_cache_plan(args, train_data, neighbor_finder, num_embeddings, strategy)`` returns one int64
array per batch, as the reference does.  The neighbour tables of every batch are sampled in one
launch of the GPU sampling kernel (the reference's ``read_batches`` spends its time there, batch by
batch in Python); the batch-sequential replacement policy runs in the library's host code.
"""
from __future__ import annotations

import math
import sys
import time

import numpy as np

from . import _lib

STRATEGIES = {"MRD": 0, "LRU": 1, "2Q": 2}


def batch_query_order(sources, destinations, timestamps, bs):
    """Query list in which batch b contributes its sources, then its destinations."""
    E = len(sources)
    nb = math.ceil(E / bs)
    nodes = np.empty(2 * E, dtype=np.int32)
    ts = np.empty(2 * E, dtype=np.float64)
    for b in range(nb):
        s, e = b * bs, min(E, (b + 1) * bs)
        m = e - s
        nodes[2 * s:2 * s + m] = sources[s:e]
        nodes[2 * s + m:2 * e] = destinations[s:e]
        ts[2 * s:2 * s + m] = timestamps[s:e]
        ts[2 * s + m:2 * e] = timestamps[s:e]
    return nodes, ts


def plan_from_tables(strategy, sources, destinations, bs, k, nbr_table, n_nodes, budget, seed=0):
    """Runs the policy over already-sampled neighbour tables ([2E, k] int32, host)."""
    if strategy not in STRATEGIES:
        print(f'unsupported cache strategy {strategy}')
        sys.exit(1)
    src = np.ascontiguousarray(sources, dtype=np.int64)
    dst = np.ascontiguousarray(destinations, dtype=np.int64)
    nbr = np.ascontiguousarray(nbr_table, dtype=np.int32)
    E = len(src)
    nb = math.ceil(E / bs)
    cap = nb * (budget + 2) + 8
    flat = np.empty(cap, dtype=np.int32)
    off = np.zeros(nb + 1, dtype=np.int64)
    stats = np.zeros(3, dtype=np.float64)
    _lib.check(_lib.lib().orca_plan_host(STRATEGIES[strategy], src.ctypes.data, dst.ctypes.data, E, bs, k,
                                         nbr.ctypes.data, n_nodes, budget, seed, flat.ctypes.data, cap,
                                         off.ctypes.data, stats.ctypes.data))
    plan = [flat[off[b]:off[b + 1]].astype(np.int64) for b in range(nb)]
    return plan, stats


def get_cache_plan(args, train_data, neighbor_finder, num_embeddings, strategy, seed=0):
    budget = args.budget
    t0 = time.time()
    nodes, ts = batch_query_order(train_data.sources, train_data.destinations, train_data.timestamps, args.bs)
    nbr, _, _, _ = neighbor_finder.sample_device(nodes, ts, args.n_degree)
    nbr = nbr.cpu().numpy()
    t_prepare = time.time() - t0
    t0 = time.time()
    plan, stats = plan_from_tables(strategy, train_data.sources, train_data.destinations, args.bs, args.n_degree,
                                   nbr, num_embeddings, budget, seed)
    t_cache = time.time() - t0
    n_reuse, n_recompute = int(stats[0]), int(stats[1])
    avg = stats[2] / stats[0] if stats[0] else float("nan")
    print(f'prepare {t_prepare}, cache {t_cache}, n_reuse {n_reuse}, n_recompute {n_recompute}, '
          f'average_reuse_distance {avg}')
    return plan
