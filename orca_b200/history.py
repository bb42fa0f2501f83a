"""Historical-embedding cache with the interface of modules/history.py:4-46.

``emb`` ([n, D] float32) lives in HBM.  The reference keeps ``cache_flag`` as a float64 NumPy array
on the host; here the flags are a uint8 device tensor (``cache_flag_dev``) and ``cache_flag`` is a
property that converts to and from the reference's host representation.
"""
from __future__ import annotations

import numpy as np
import torch

from . import _lib


class History(torch.nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, device=None, history_budget=0):
        super().__init__()
        if embedding_dim != _lib.DIM:
            raise ValueError("orca_b200 is built for 172-wide embeddings")
        self._device = _lib.require_cuda(device if device is not None else "cuda")
        self.num_embeddings = num_embeddings
        self.embedding_dim = embedding_dim
        self.emb = torch.empty(num_embeddings, embedding_dim, device=self._device)
        # write-only bookkeeping in the reference (modules/embedding_module.py:190); kept as an
        # attribute, not maintained by the fused batch path
        self.update_times = torch.zeros(num_embeddings)
        self.reset_parameters()
        self.cache_flag_dev = torch.zeros(num_embeddings, dtype=torch.uint8, device=self._device)
        self.budget = history_budget if history_budget != 0 else num_embeddings
        # device copy of the plan whose flags are currently set, so that the next plan only clears
        # those entries; n_prev < 0 means "unknown, clear everything"
        self.prev_plan = torch.zeros(max(int(self.budget) + 2, 1), dtype=torch.int32, device=self._device)
        self.n_prev = np.zeros(1, dtype=np.int32)
        self.last_pos = torch.zeros(num_embeddings, dtype=torch.int64, device=self._device)
        self.epoch = np.ones(1, dtype=np.int64)

    # ---- reference-compatible view of the flags
    @property
    def cache_flag(self):
        return self.cache_flag_dev.cpu().numpy().astype(np.float64)

    @cache_flag.setter
    def cache_flag(self, value):
        self.cache_flag_dev = torch.as_tensor(np.asarray(value) != 0).to(self._device, torch.uint8)
        self.n_prev[0] = -1

    def reset_parameters(self):
        self.emb.fill_(0)

    def detach_history(self):
        self.emb.detach_()

    def _ids(self, inds):
        if isinstance(inds, torch.Tensor):
            return inds.to(self._device, torch.int32).contiguous()
        return torch.as_tensor(np.asarray(inds), dtype=torch.int32).to(self._device)

    # ---- modules/history.py:25-30
    def update_flag(self, cache_plan, source_node):
        L = _lib.lib()
        s = _lib.stream_ptr(self._device)
        if cache_plan is not None:
            plan = self._ids(cache_plan)
            if plan.numel() > self.prev_plan.numel():
                self.prev_plan = torch.zeros(plan.numel(), dtype=torch.int32, device=self._device)
                self.n_prev[0] = -1
            known = self.n_prev[0] >= 0
            _lib.check(L.orca_history_set_flags(self.cache_flag_dev.data_ptr(), self.num_embeddings,
                                                self.prev_plan.data_ptr() if known else None,
                                                int(self.n_prev[0]) if known else 0, plan.data_ptr(),
                                                plan.numel(), s))
            self.prev_plan[:plan.numel()].copy_(plan)
            self.n_prev[0] = plan.numel()
        else:
            ids = self._ids(source_node)
            _lib.check(L.orca_history_set_flags(self.cache_flag_dev.data_ptr(), self.num_embeddings,
                                                self.prev_plan.data_ptr(), 0, ids.data_ptr(), ids.numel(), s))
            self.n_prev[0] = -1

    # ---- modules/history.py:32-36
    @torch.no_grad()
    def pull(self, inds):
        ids = self._ids(inds).reshape(-1)
        out = torch.empty(ids.numel(), self.embedding_dim, device=self._device)
        _lib.check(_lib.lib().orca_history_pull(self.emb.data_ptr(), ids.data_ptr(), ids.numel(),
                                                out.data_ptr(), _lib.stream_ptr(self._device)))
        return out

    # ---- modules/history.py:38-40; among duplicate ids the last occurrence provides the row
    @torch.no_grad()
    def push(self, x, inds):
        ids = self._ids(inds).reshape(-1)
        x = x.to(self._device, torch.float32).contiguous()
        n = ids.numel()
        if n == 0:
            return
        L = _lib.lib()
        s = _lib.stream_ptr(self._device)
        win = torch.empty(n, dtype=torch.uint8, device=self._device)
        _lib.check(L.orca_last_occurrence(ids.data_ptr(), n, None, self.num_embeddings,
                                          self.last_pos.data_ptr(), int(self.epoch[0]), win.data_ptr(),
                                          None, None, s))
        self.epoch[0] += n
        _lib.check(L.orca_history_push(self.emb.data_ptr(), x.data_ptr(), ids.data_ptr(), win.data_ptr(),
                                       n, None, s))

    # ---- modules/history.py:42-46
    def push_and_pull(self, x, push_inds, pull_inds):
        self.push(x, push_inds)
        out = self.pull(pull_inds)
        self.emb = self.emb.clone()
        return out
