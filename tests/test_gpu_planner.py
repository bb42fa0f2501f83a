"""The device planners (orca_plan_device: MRD, LRU, 2Q) against the reference's plans (golden fixtures) and
against the oracle's planner on inputs that put many equal keys at the budget line, where the order numba's
argsort leaves among equal keys -- and, for LRU and 2Q, the stream of its Mersenne Twister -- decide which
nodes stay cached.  Plans are compared entry by entry, in order; the statistics are compared as integers."""
import dataclasses

import numpy as np
import pytest
import torch

from helpers import golden, graph, unpack

pytestmark = pytest.mark.gpu


def _device_plan(g, bs, k, budget, tables_from_oracle=True, strategy="MRD", seed=0):
    """Plan of the device planner; the neighbour table comes from the oracle's sampler (so that the test
    isolates the planner) or from the product sampler."""
    from oracle import tgn_oracle
    from orca_b200 import cache
    nodes, ts = cache.batch_query_order(g.sources, g.destinations, g.timestamps, bs)
    adj = tgn_oracle.Adjacency(g.sources, g.destinations, g.edge_idxs, g.timestamps, g.n_nodes)
    if tables_from_oracle:
        nbr = torch.as_tensor(tgn_oracle.sample_neighbors(adj, nodes, ts, k)[0].astype(np.int32)).cuda()
    else:
        from orca_b200.neighbor_finder import get_neighbor_finder
        nbr = get_neighbor_finder(g, g.n_nodes - 1, device="cuda").sample_device(nodes, ts, k)[0]
    plan, stats = cache.plan_device(strategy, torch.as_tensor(nodes).cuda(), nbr, g.n_edges, bs, k, g.n_nodes, budget,
                                    seed)
    return adj, plan, stats


@pytest.mark.parametrize("case", ["c1", "t_bip2", "t_nb2", "t_lru", "t_2q"])
@pytest.mark.parametrize("strategy", ["MRD", "LRU", "2Q"])
def test_plans_match_reference(case, strategy):
    gold = golden(case)
    g = graph(str(gold["spec"]))
    _, got, _ = _device_plan(g, g.spec.bs, g.spec.n_degree, g.spec.budget, tables_from_oracle=False,
                             strategy=strategy)
    want = unpack(gold[f"plan_{strategy}_flat"], gold[f"plan_{strategy}_off"])
    assert len(got) == len(want)
    for b, (a, w) in enumerate(zip(got, want)):
        assert a.dtype == np.int64 and np.array_equal(a, w), f"batch {b}"


@pytest.mark.parametrize("budget,bs,seed", [(7, 50, 1), (40, 120, 2), (300, 200, 3), (2, 64, 4), (1000, 400, 5),
                                            (100000, 200, 6), (200000, 200, 7)])
@pytest.mark.parametrize("strategy", ["MRD", "LRU", "2Q"])
def test_plans_match_oracle_on_tight_budgets(strategy, budget, bs, seed):
    """Budgets from far below to far above the number of candidates; statistics included.  (The last budget
    makes the candidate capacity larger than a thread-block cluster takes, so the one-CTA kernels run.)"""
    from oracle import planner
    from orca_b200 import synthetic
    spec = dataclasses.replace(synthetic.SPECS["t_nb2"], n_src=400, n_edges=3000, bs=bs, budget=budget)
    g = synthetic.make_graph(spec, seed=seed)
    adj, got, stats = _device_plan(g, bs, 10, budget, strategy=strategy, seed=seed)
    rb = planner.read_batches(g.sources, g.destinations, g.timestamps, bs, 10, adj, g.n_nodes)
    want, wstats = planner.solve(strategy, rb, g.n_nodes, budget, seed=seed)
    assert len(got) == len(want)
    for b, (a, w) in enumerate(zip(got, want)):
        assert np.array_equal(a, w), f"batch {b}"
    assert (int(stats[0]), int(stats[1])) == wstats[:2]
    if wstats[0]:
        assert stats[2] / stats[0] == wstats[2]


def test_mrd_long_ranges_of_equal_keys():
    """A wide graph with large batches: tens of thousands of candidates per batch, nearly all with the key
    of "not needed again as a neighbour", cut by a budget in the middle of them -- every level of the
    partition emulation is exercised, over many ranges at once."""
    from oracle import planner
    from orca_b200 import synthetic
    spec = dataclasses.replace(synthetic.SPECS["t_nb2"], n_src=60000, n_edges=60000, bs=2000,
                               budget=9000)
    g = synthetic.make_graph(spec, seed=11)
    adj, got, stats = _device_plan(g, spec.bs, 10, spec.budget)
    rb = planner.read_batches(g.sources, g.destinations, g.timestamps, spec.bs, 10, adj, g.n_nodes)
    want, wstats = planner.solve("MRD", rb, g.n_nodes, spec.budget)
    assert max(len(w) for w in want) == spec.budget
    for b, (a, w) in enumerate(zip(got, want)):
        assert np.array_equal(a, w), f"batch {b}"
    assert (int(stats[0]), int(stats[1])) == wstats[:2]


def test_plan_buffer_too_small_is_reported():
    from orca_b200 import _lib, cache
    g = graph("t_nb2")
    bs, k, budget = g.spec.bs, g.spec.n_degree, 50
    nodes, ts = cache.batch_query_order(g.sources, g.destinations, g.timestamps, bs)
    from orca_b200.neighbor_finder import get_neighbor_finder
    nbr = get_neighbor_finder(g, g.n_nodes - 1, device="cuda").sample_device(nodes, ts, k)[0]
    L = _lib.lib()
    ws_bytes = L.orca_plan_mrd_workspace_bytes(g.n_edges, bs, k, g.n_nodes, budget)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    nd = torch.as_tensor(nodes).cuda()
    flat = torch.empty(60, dtype=torch.int32, device="cuda")
    off = torch.zeros(g.n_batches + 1, dtype=torch.int64, device="cuda")
    stats = torch.zeros(3, dtype=torch.int64, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    _lib.check(L.orca_plan_mrd(nd.data_ptr(), g.n_edges, bs, k, nbr.data_ptr(), g.n_nodes, budget, flat.data_ptr(), 60,
                               off.data_ptr(), stats.data_ptr(), status.data_ptr(), ws.data_ptr(), ws_bytes,
                               _lib.stream_ptr(torch.device("cuda"))))
    torch.cuda.synchronize()
    assert int(status[0]) == 4        # ORCA_E_CAPACITY
    with pytest.raises(_lib.OrcaError):
        # the same call with too small a workspace is refused on the host
        _lib.check(L.orca_plan_mrd(nd.data_ptr(), g.n_edges, bs, k, nbr.data_ptr(), g.n_nodes, budget,
                                   flat.data_ptr(), 60, off.data_ptr(), stats.data_ptr(), status.data_ptr(),
                                   ws.data_ptr(), ws_bytes - 1, _lib.stream_ptr(torch.device("cuda"))))
