"""The allocation-free GRU update (orca_gru_update_static) against orca_gru_update.

A host that may not call cudaMalloc (a serving process with a frozen memory budget, a plugin whose
owner bans allocator calls after start-up) uses the variant whose scratch is a fixed array inside the
library.  It must give what the ordinary entry point gives, on a first call and on a second call that
finds the previous call's data still in the shared scratch.  Runs last so that a failure here cannot
hide the other tests in a run that stops at the first failure."""
import numpy as np
import pytest
import torch

from helpers import state_dict

pytestmark = pytest.mark.gpu

D = 172


def _fill(mem, rs, n_flag):
    n = mem.n_nodes
    mem.memory.copy_(torch.from_numpy(rs.randn(n, D).astype(np.float32)))
    mem.messages.copy_(torch.from_numpy(rs.randn(n, 4 * D).astype(np.float32)))
    mem.timestamps.copy_(torch.from_numpy(rs.uniform(0, 1e6, n).astype(np.float32)))
    mem.last_update.zero_()
    flags = np.zeros(n, dtype=np.uint8)
    flags[rs.choice(np.arange(1, n), size=n_flag, replace=False)] = 1
    mem.nodes = flags
    return flags


def _clone_into(dst, src):
    for name in ("memory", "messages", "timestamps", "last_update", "nodes_dev"):
        getattr(dst, name).copy_(getattr(src, name))


def test_static_scratch_matches_caller_scratch():
    from orca_b200 import _lib
    from orca_b200.memory import GRUMemoryUpdater, Memory
    L = _lib.lib()
    dev = torch.device("cuda:0")
    sd = state_dict(1)
    upd = GRUMemoryUpdater(4 * D, D, dev).to(dev)
    upd.memory_updater.load_state_dict({k.split(".")[-1]: torch.as_tensor(v) for k, v in sd.items()
                                        if k.startswith("memory_updater.memory_updater.")})
    n_nodes = 3000
    a, b = Memory(n_nodes, D, 4 * D, 4 * D, device=dev), Memory(n_nodes, D, 4 * D, 4 * D, device=dev)
    rs = np.random.RandomState(17)
    s = _lib.stream_ptr(dev)
    # two calls in a row, different sizes: the second one finds the first one's rows in the scratch
    for n_list, n_flag in ((700, 1500), (333, 900)):
        _fill(a, rs, n_flag)
        _clone_into(b, a)
        nodes = torch.as_tensor(rs.choice(np.arange(1, n_nodes), size=n_list, replace=False).astype(np.int32)).to(dev)
        scratch = torch.empty(n_list, D, device=dev)
        _lib.check(L.orca_gru_update(upd.c_struct(), a.c_struct(), nodes.data_ptr(), n_list, None, 1,
                                     scratch.data_ptr(), s))
        _lib.check(L.orca_gru_update_static(upd.c_struct(), b.c_struct(), nodes.data_ptr(), n_list, None, 1, s))
        torch.cuda.synchronize()
        # same kernels, same inputs: the tables must agree exactly (tolerance of the GRU tests: 1e-3)
        assert torch.equal(a.memory, b.memory)
        assert torch.equal(a.last_update, b.last_update)
        assert torch.equal(a.nodes_dev, b.nodes_dev)
        assert not torch.equal(a.memory[nodes.long()], torch.zeros_like(a.memory[nodes.long()]))


def test_static_scratch_rejects_oversize():
    from orca_b200 import _lib
    from orca_b200.memory import GRUMemoryUpdater, Memory
    L = _lib.lib()
    dev = torch.device("cuda:0")
    upd = GRUMemoryUpdater(4 * D, D, dev).to(dev)
    mem = Memory(10, D, 4 * D, 4 * D, device=dev)
    nodes = torch.zeros(8, dtype=torch.int32, device=dev)
    rc = L.orca_gru_update_static(upd.c_struct(), mem.c_struct(), nodes.data_ptr(), 4097, None, 0, _lib.stream_ptr(dev))
    assert rc == 4
    assert b"4096" in L.orca_last_error()
