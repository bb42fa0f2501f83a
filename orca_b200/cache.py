"""Offline cache planning with the interface of utils/cache.py:407-428.

``get_cache_plan(args, train_data, neighbor_finder, num_embeddings, strategy)`` returns one int64
array per batch, as the reference does.  The neighbour tables of every batch are sampled in one
launch of the GPU sampling kernel (the reference's ``read_batches`` spends its time there, batch by
batch in Python) and the policies run on the device as well (``orca_plan_device``): MRD on a thread-block
cluster, LRU and 2Q -- whose random evictions are one serial Mersenne-Twister shuffle per batch -- on one
block.  ``plan_from_tables`` runs the same policies in the library's host code over tables that are
already on the host.
"""
from __future__ import annotations

import math
import sys
import time

import numpy as np
import torch

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


def plan_device(strategy, nodes, nbr_table, n_edges, bs, k, n_nodes, budget, seed=0):
    """The policy over a sampled neighbour table that is still on the device.  nodes: [2E] int32 query list
    (``batch_query_order``), nbr_table: [2E, k] int32, both CUDA tensors.  Returns the plan (one int64
    array per batch) and (n_reuse, n_recompute, sum of reuse distances)."""
    if strategy not in STRATEGIES:
        print(f'unsupported cache strategy {strategy}')
        sys.exit(1)
    dev = nbr_table.device
    if dev.type != "cuda":
        raise ValueError("plan_device needs CUDA tensors")
    nodes = nodes.to(dev, torch.int32).contiguous()
    nbr_table = nbr_table.to(torch.int32).contiguous()
    nb = math.ceil(n_edges / bs)
    code = STRATEGIES[strategy]
    L = _lib.lib()
    with torch.cuda.device(dev):
        ws_bytes = L.orca_plan_device_workspace_bytes(code, n_edges, bs, k, n_nodes, budget)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        cap = max(nb * budget, 1)
        flat = torch.empty(cap, dtype=torch.int32, device=dev)
        off = torch.zeros(nb + 1, dtype=torch.int64, device=dev)
        stats = torch.zeros(3, dtype=torch.int64, device=dev)
        status = torch.zeros(4, dtype=torch.int32, device=dev)
        _lib.check(L.orca_plan_device(code, nodes.data_ptr(), n_edges, bs, k, nbr_table.data_ptr(), n_nodes, budget,
                                      seed, flat.data_ptr(), cap, off.data_ptr(), stats.data_ptr(),
                                      status.data_ptr(), ws.data_ptr(), ws_bytes, _lib.stream_ptr(dev)))
        _lib.check(L.orca_read_status(None, status.data_ptr(), None, _lib.stream_ptr(dev)))
    off_h = off.cpu().numpy()
    flat_h = flat[:int(off_h[-1])].cpu().numpy().astype(np.int64)
    plan = [flat_h[off_h[b]:off_h[b + 1]] for b in range(nb)]
    return plan, stats.cpu().numpy().astype(np.float64)


def plan_mrd_device(nodes, nbr_table, n_edges, bs, k, n_nodes, budget):
    return plan_device("MRD", nodes, nbr_table, n_edges, bs, k, n_nodes, budget)


def _plan_local(args, train_data, neighbor_finder, num_embeddings, strategy, seed):
    budget = args.budget
    t0 = time.time()
    nodes, ts = batch_query_order(train_data.sources, train_data.destinations, train_data.timestamps, args.bs)
    nodes_dev = torch.as_tensor(nodes).to(neighbor_finder.device)
    nbr, _, _, _ = neighbor_finder.sample_device(nodes_dev, ts, args.n_degree)
    torch.cuda.synchronize(neighbor_finder.device)
    t_prepare = time.time() - t0
    t0 = time.time()
    plan, stats = plan_device(strategy, nodes_dev, nbr, len(train_data.sources), args.bs, args.n_degree,
                              num_embeddings, budget, seed)
    t_cache = time.time() - t0
    n_reuse, n_recompute = int(stats[0]), int(stats[1])
    avg = stats[2] / stats[0] if stats[0] else float("nan")
    print(f'prepare {t_prepare}, cache {t_cache}, n_reuse {n_reuse}, n_recompute {n_recompute}, '
          f'average_reuse_distance {avg}')
    return plan


def get_cache_plan(args, train_data, neighbor_finder, num_embeddings, strategy, seed=0, broadcast_from=None):
    """utils/cache.py:407-428.  With ``broadcast_from`` = a rank of the default process group, only that
    rank plans (and prints the statistics line); the others receive the plan in one broadcast of the
    flattened lists (no counterpart in the reference, which runs on one GPU)."""
    if strategy not in STRATEGIES:
        print(f'unsupported cache strategy {strategy}')
        sys.exit(1)
    import torch.distributed as dist
    if broadcast_from is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return _plan_local(args, train_data, neighbor_finder, num_embeddings, strategy, seed)
    dev = neighbor_finder.device
    nb = math.ceil(len(train_data.sources) / args.bs)
    off = torch.zeros(nb + 1, dtype=torch.int64, device=dev)
    flat = None
    if dist.get_rank() == broadcast_from:
        plan = _plan_local(args, train_data, neighbor_finder, num_embeddings, strategy, seed)
        off[1:] = torch.as_tensor(np.cumsum([len(p) for p in plan], dtype=np.int64), device=dev)
        flat = torch.as_tensor(np.concatenate(plan) if plan else np.zeros(0, np.int64)).to(dev)
    dist.broadcast(off, src=broadcast_from)
    off_h = off.cpu().numpy()
    if flat is None:
        flat = torch.empty(int(off_h[-1]), dtype=torch.int64, device=dev)
    dist.broadcast(flat, src=broadcast_from)
    flat_h = flat.cpu().numpy()
    return [flat_h[off_h[b]:off_h[b + 1]] for b in range(nb)]
