"""Node memory with the interface of modules/memory.py:5-50 and its GRU updater
(modules/memory_updater.py:25-53, 83-86).

All tables live in HBM.  The reference keeps the "has a pending message" flags as a host bool array
(``Memory.nodes``); here they are a uint8 device tensor (``nodes_dev``) and ``nodes`` is a property
that converts to and from the host representation.
"""
from __future__ import annotations

import numpy as np
import torch
from torch import nn

from . import _lib, weights


class Memory(nn.Module):
    def __init__(self, n_nodes, memory_dimension, input_dimension, message_dimension=None, device="cuda",
                 combination_method="sum"):
        super().__init__()
        if memory_dimension != _lib.DIM or (message_dimension or input_dimension) != _lib.MSG_DIM:
            raise ValueError("orca_b200 is built for a 172-wide memory and 688-wide raw messages")
        self.n_nodes = n_nodes
        self.memory_dimension = memory_dimension
        self.input_dimension = input_dimension
        self.message_dimension = message_dimension
        self.device = _lib.require_cuda(device)
        self.combination_method = combination_method
        self.__init_memory__()

    def __init_memory__(self):
        d = self.device
        self.memory = torch.zeros((self.n_nodes, self.memory_dimension), device=d)
        self.last_update = torch.zeros(self.n_nodes, device=d)
        self.nodes_dev = torch.zeros(self.n_nodes, dtype=torch.uint8, device=d)
        self.messages = torch.zeros((self.n_nodes, self.message_dimension), device=d)
        self.timestamps = torch.zeros(self.n_nodes, device=d)

    @property
    def nodes(self):
        return self.nodes_dev.cpu().numpy().astype(bool)

    @nodes.setter
    def nodes(self, value):
        self.nodes_dev = torch.as_tensor(np.asarray(value) != 0).to(self.device, torch.uint8)

    def _ix(self, idx):
        if isinstance(idx, torch.Tensor):
            return idx.to(self.device, torch.long)
        return torch.as_tensor(np.asarray(idx), dtype=torch.long).to(self.device)

    def store_raw_messages(self, nodes, messages, timestamps):
        ix = self._ix(nodes)
        self.nodes_dev[ix] = 1
        self.messages[ix] = messages
        self.timestamps[ix] = timestamps

    def get_memory(self, node_idxs):
        return self.memory[self._ix(node_idxs), :]

    def set_memory(self, node_idxs, values):
        self.memory[self._ix(node_idxs), :] = values

    def get_last_update(self, node_idxs):
        return self.last_update[self._ix(node_idxs)]

    def backup_memory(self):
        return (self.memory.clone(), self.last_update.clone(), self.messages.clone(), self.nodes_dev.clone(),
                self.timestamps.clone())

    def restore_memory(self, memory_backup):
        self.memory, self.last_update, self.messages = (memory_backup[0].clone(), memory_backup[1].clone(),
                                                        memory_backup[2].clone())
        flags = memory_backup[3]
        self.nodes_dev = flags.clone() if isinstance(flags, torch.Tensor) else \
            torch.as_tensor(np.asarray(flags) != 0).to(self.device, torch.uint8)
        self.timestamps = memory_backup[4].clone()

    def detach_memory(self):
        self.memory.detach_()
        self.messages.detach_()

    def clear_messages(self, positives):
        self.nodes_dev[self._ix(positives)] = 0

    def c_struct(self):
        return _lib.MemoryT(self.memory.data_ptr(), self.last_update.data_ptr(), self.messages.data_ptr(),
                            self.timestamps.data_ptr(), self.nodes_dev.data_ptr(), self.n_nodes)


class GRUMemoryUpdater(nn.Module):
    """modules/memory_updater.py:83-86.  ``memory_updater`` (an nn.GRUCell) and ``layer_norm`` only
    hold the parameters under the reference's names; the update runs in the fused CUDA kernel."""

    def __init__(self, message_dimension, memory_dimension, device):
        super().__init__()
        self.layer_norm = nn.LayerNorm(memory_dimension)
        self.message_dimension = message_dimension
        self.device = device
        self.memory_updater = nn.GRUCell(input_size=message_dimension, hidden_size=memory_dimension)
        self._prepared = None

    def invalidate(self):
        self._prepared = None

    def prepared(self):
        if self._prepared is None:
            sd = {"memory_updater.memory_updater." + k: v.detach().cpu().numpy()
                  for k, v in self.memory_updater.state_dict().items()}
            w = weights.prepare_gru(sd)
            dev = self.memory_updater.weight_ih.device
            self._prepared = {k: torch.from_numpy(v).to(dev) for k, v in w.items()}
        return self._prepared

    def c_struct(self):
        p = self.prepared()
        return _lib.GruWeights(p["Wg"].data_ptr(), p["bg"].data_ptr(), p["Wg_tc"].data_ptr())

    def _run(self, memory: Memory, ids: torch.Tensor, clear: bool):
        n = ids.numel()
        if n == 0:
            return
        L = _lib.lib()
        scratch = torch.empty(n, _lib.DIM, device=memory.device)
        gw, ms = self.c_struct(), memory.c_struct()
        _lib.check(L.orca_gru_update(gw, ms, ids.data_ptr(), n, None, 1 if clear else 0, scratch.data_ptr(),
                                     _lib.stream_ptr(memory.device)))

    @torch.no_grad()
    def update_memory(self, memory: Memory, positives):
        """modules/memory_updater.py:25-39: listed nodes with a pending message get
        last_update = message time and memory = GRU(message, memory).  Flags stay set."""
        ids = torch.as_tensor(np.asarray(positives), dtype=torch.int32).to(memory.device)
        self._run(memory, ids, clear=False)

    @torch.no_grad()
    def update_memory_in_test(self, memory: Memory):
        """modules/memory_updater.py:42-53: flush every pending message, then clear the flags."""
        ids = torch.nonzero(memory.nodes_dev, as_tuple=False).reshape(-1).to(torch.int32)
        self._run(memory, ids, clear=True)


def get_memory_updater(module_type, message_dimension, memory_dimension, device):
    if module_type == "gru":
        return GRUMemoryUpdater(message_dimension, memory_dimension, device)
    raise ValueError("Memory updater {} not supported (only 'gru' has a kernel)".format(module_type))
