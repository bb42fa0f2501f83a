"""Temporal neighbour finder on the GPU, with the interface of the reference's jitclass
(utils/util.py:91-151): ``get_neighbor_finder(data)``, ``NeighborFinder.find_before`` and
``NeighborFinder.get_temporal_neighbor`` keep their names, argument meaning and return dtypes.

The per-node Python lists of the reference become one time-sorted CSR (indptr int64, neighbour
int32, edge id int32, timestamp float64) resident in HBM; a host copy is kept for ``find_before``,
which returns array slices.
"""
from __future__ import annotations

import numpy as np
import torch

from . import _lib


class NeighborFinder:
    def __init__(self, node_to_neighbors, node_to_edge_idxs, node_to_edge_timestamps, device="cuda"):
        """Same arguments as utils/util.py:123-126: per-node arrays, each already sorted by time."""
        lens = np.fromiter((len(a) for a in node_to_neighbors), dtype=np.int64, count=len(node_to_neighbors))
        indptr = np.zeros(len(lens) + 1, dtype=np.int64)
        np.cumsum(lens, out=indptr[1:])
        cat = lambda lst, dt: (np.concatenate([np.asarray(a, dtype=dt) for a in lst]) if len(lst) and indptr[-1]
                               else np.zeros(0, dtype=dt))
        self._init_csr(indptr, cat(node_to_neighbors, np.int32), cat(node_to_edge_idxs, np.int32),
                       cat(node_to_edge_timestamps, np.float64), device)

    @classmethod
    def from_csr(cls, indptr, nbr, eid, ts, device="cuda"):
        self = cls.__new__(cls)
        self._init_csr(indptr, nbr, eid, ts, device)
        return self

    def _init_csr(self, indptr, nbr, eid, ts, device):
        self.device = _lib.require_cuda(device)
        self.n_nodes = len(indptr) - 1
        self.h_indptr = np.ascontiguousarray(indptr, dtype=np.int64)
        self.h_nbr = np.ascontiguousarray(nbr, dtype=np.int32)
        self.h_eid = np.ascontiguousarray(eid, dtype=np.int32)
        self.h_ts = np.ascontiguousarray(ts, dtype=np.float64)
        self.indptr = torch.from_numpy(self.h_indptr).to(self.device)
        # one spare element keeps the pointers valid for an empty graph
        pad = lambda a: a if len(a) else np.zeros(1, dtype=a.dtype)
        self.adj_nbr = torch.from_numpy(pad(self.h_nbr)).to(self.device)
        self.adj_eid = torch.from_numpy(pad(self.h_eid)).to(self.device)
        self.adj_ts = torch.from_numpy(pad(self.h_ts)).to(self.device)

    # --- utils/util.py:129-131
    def find_before(self, src_idx, cut_time):
        L = _lib.lib()
        node = torch.tensor([int(src_idx)], dtype=torch.int32, device=self.device)
        t = torch.tensor([float(cut_time)], dtype=torch.float64, device=self.device)
        cnt = torch.empty(1, dtype=torch.int32, device=self.device)
        _lib.check(L.orca_find_before(self.indptr.data_ptr(), self.adj_ts.data_ptr(), self.n_nodes,
                                      node.data_ptr(), t.data_ptr(), 1, cnt.data_ptr(),
                                      _lib.stream_ptr(self.device)))
        i = int(cnt.item())
        b = int(self.h_indptr[int(src_idx)])
        return self.h_nbr[b:b + i], self.h_eid[b:b + i], self.h_ts[b:b + i]

    # --- utils/util.py:134-151
    def get_temporal_neighbor(self, source_nodes, timestamps, n_neighbors):
        """Returns (neighbors int32 [Q,K], edge_idxs int32 [Q,K], edge_times float32 [Q,K]) as NumPy
        arrays: the K most recent interactions strictly before each query time, right-aligned,
        zero-padded on the left."""
        nbr, eid, et, _ = self.sample_device(source_nodes, timestamps, n_neighbors)
        return nbr.cpu().numpy(), eid.cpu().numpy(), et.cpu().numpy()

    def sample_device(self, source_nodes, timestamps, n_neighbors, want_delta=False):
        """Same as get_temporal_neighbor but the tables stay on the device (torch tensors);
        also returns the fused time differences when asked."""
        k = n_neighbors if n_neighbors > 0 else 1
        nodes = torch.as_tensor(np.asarray(source_nodes), dtype=torch.int32).to(self.device) \
            if not isinstance(source_nodes, torch.Tensor) else source_nodes.to(self.device, torch.int32)
        ts = torch.as_tensor(np.asarray(timestamps), dtype=torch.float64).to(self.device) \
            if not isinstance(timestamps, torch.Tensor) else timestamps.to(self.device, torch.float64)
        q = nodes.numel()
        nbr = torch.zeros((q, k), dtype=torch.int32, device=self.device)
        eid = torch.zeros((q, k), dtype=torch.int32, device=self.device)
        et = torch.zeros((q, k), dtype=torch.float32, device=self.device)
        dt = torch.zeros((q, k), dtype=torch.float32, device=self.device) if want_delta else None
        if q and n_neighbors > 0:
            status = torch.zeros(4, dtype=torch.int32, device=self.device)
            L = _lib.lib()
            _lib.check(L.orca_sample_topk(self.indptr.data_ptr(), self.adj_nbr.data_ptr(),
                                          self.adj_eid.data_ptr(), self.adj_ts.data_ptr(), self.n_nodes,
                                          nodes.data_ptr(), ts.data_ptr(), q, None, k, nbr.data_ptr(),
                                          eid.data_ptr(), et.data_ptr(), _lib.ptr(dt), status.data_ptr(),
                                          _lib.stream_ptr(self.device)))
            _lib.check(L.orca_read_status(None, status.data_ptr(), None, _lib.stream_ptr(self.device)))
        return nbr, eid, et, dt


def get_neighbor_finder(data, max_node_idx=None, device="cuda"):
    """utils/util.py:91-105: every interaction is listed under both endpoints, each node's list
    stably sorted by time.  `data` needs .sources, .destinations, .edge_idxs, .timestamps."""
    src = np.ascontiguousarray(data.sources, dtype=np.int64)
    dst = np.ascontiguousarray(data.destinations, dtype=np.int64)
    eidx = np.ascontiguousarray(data.edge_idxs, dtype=np.int64)
    ts = np.ascontiguousarray(data.timestamps, dtype=np.float64)
    if max_node_idx is None:
        max_node_idx = int(max(src.max(), dst.max())) if len(src) else 0
    n = int(max_node_idx) + 1
    E = len(src)
    indptr = np.empty(n + 1, dtype=np.int64)
    nbr = np.empty(max(2 * E, 1), dtype=np.int32)
    eid = np.empty(max(2 * E, 1), dtype=np.int32)
    ats = np.empty(max(2 * E, 1), dtype=np.float64)
    _lib.check(_lib.lib().orca_csr_build_host(src.ctypes.data, dst.ctypes.data, eidx.ctypes.data, ts.ctypes.data,
                                              E, n, indptr.ctypes.data, nbr.ctypes.data, eid.ctypes.data,
                                              ats.ctypes.data))
    return NeighborFinder.from_csr(indptr, nbr[:2 * E], eid[:2 * E], ats[:2 * E], device=device)
