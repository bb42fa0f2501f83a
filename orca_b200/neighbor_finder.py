"""Temporal neighbour finder on the GPU, with the interface of the reference's jitclass
(utils/util.py:91-151): ``get_neighbor_finder(data)``, ``NeighborFinder.find_before`` and
``NeighborFinder.get_temporal_neighbor`` keep their names, argument meaning and return dtypes.

The per-node Python lists of the reference become one time-sorted CSR (indptr int64, neighbour
int32, edge id int32, timestamp float64) resident in HBM, built there by ``orca_csr_build``;
``find_before`` copies the slice it returns to the host.
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
        self.indptr = torch.from_numpy(np.ascontiguousarray(indptr, dtype=np.int64)).to(self.device)
        # one spare element keeps the pointers valid for an empty graph
        pad = lambda a, dt: np.ascontiguousarray(a, dtype=dt) if len(a) else np.zeros(1, dtype=dt)
        self.adj_nbr = torch.from_numpy(pad(nbr, np.int32)).to(self.device)
        self.adj_eid = torch.from_numpy(pad(eid, np.int32)).to(self.device)
        self.adj_ts = torch.from_numpy(pad(ts, np.float64)).to(self.device)

    @classmethod
    def build_on_device(cls, sources, destinations, edge_idxs, timestamps, n_nodes, device="cuda"):
        """The adjacency of an edge stream, sorted on the GPU (utils/util.py:91-105)."""
        self = cls.__new__(cls)
        self.device = dev = _lib.require_cuda(device)
        self.n_nodes = int(n_nodes)
        E = len(sources)
        up = lambda a, dt: torch.as_tensor(np.array(a, dtype=dt, order="C")).to(dev)     # (a copy: the input may be read-only)
        src, dst, eidx = (up(a, np.int64) for a in (sources, destinations, edge_idxs))
        ts = up(timestamps, np.float64)
        L = _lib.lib()
        with torch.cuda.device(dev):
            self.indptr = torch.empty(self.n_nodes + 1, dtype=torch.int64, device=dev)
            self.adj_nbr = torch.zeros(max(2 * E, 1), dtype=torch.int32, device=dev)
            self.adj_eid = torch.zeros(max(2 * E, 1), dtype=torch.int32, device=dev)
            self.adj_ts = torch.zeros(max(2 * E, 1), dtype=torch.float64, device=dev)
            ws_bytes = L.orca_csr_build_workspace_bytes(E, self.n_nodes)
            ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
            status = torch.zeros(4, dtype=torch.int32, device=dev)
            _lib.check(L.orca_csr_build(src.data_ptr(), dst.data_ptr(), eidx.data_ptr(), ts.data_ptr(), E,
                                        self.n_nodes, self.indptr.data_ptr(), self.adj_nbr.data_ptr(),
                                        self.adj_eid.data_ptr(), self.adj_ts.data_ptr(), status.data_ptr(),
                                        ws.data_ptr(), ws.numel(), _lib.stream_ptr(dev)))
            _lib.check(L.orca_read_status(None, status.data_ptr(), None, _lib.stream_ptr(dev)))
        return self

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
        b = int(self.indptr[int(src_idx)].item())
        return (self.adj_nbr[b:b + i].cpu().numpy(), self.adj_eid[b:b + i].cpu().numpy(),
                self.adj_ts[b:b + i].cpu().numpy())

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
    src, dst = np.asarray(data.sources), np.asarray(data.destinations)
    if max_node_idx is None:
        max_node_idx = int(max(src.max(), dst.max())) if len(src) else 0
    return NeighborFinder.build_on_device(src, dst, data.edge_idxs, data.timestamps, int(max_node_idx) + 1,
                                          device=device)
