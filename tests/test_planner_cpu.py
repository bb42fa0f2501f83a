"""The library's host-side planners against the reference's plans (golden fixtures) and against the
oracle on tie-heavy random inputs.  The neighbour tables the policies consume come from the oracle's
sampler here, so no GPU is needed."""
import numpy as np
import pytest

from helpers import golden, graph, unpack
from orca_b200 import build, cache
from oracle import planner, tgn_oracle


@pytest.fixture(scope="module", autouse=True)
def _built():
    build.build()


def _tables(g, bs, k):
    adj = tgn_oracle.Adjacency(g.sources, g.destinations, g.edge_idxs, g.timestamps, g.n_nodes)
    nodes, ts = cache.batch_query_order(g.sources, g.destinations, g.timestamps, bs)
    return adj, tgn_oracle.sample_neighbors(adj, nodes, ts, k)[0]


@pytest.mark.parametrize("case", ["c1", "t_bip2", "t_nb2", "t_lru", "t_2q"])
@pytest.mark.parametrize("strategy", ["MRD", "LRU", "2Q"])
def test_plans_match_reference(case, strategy):
    gold = golden(case)
    g = graph(str(gold["spec"]))
    _, nbr = _tables(g, g.spec.bs, g.spec.n_degree)
    got, _ = cache.plan_from_tables(strategy, g.sources, g.destinations, g.spec.bs, g.spec.n_degree, nbr,
                                    g.n_nodes, g.spec.budget, seed=0)
    want = unpack(gold[f"plan_{strategy}_flat"], gold[f"plan_{strategy}_off"])
    assert len(got) == len(want)
    for b, (a, w) in enumerate(zip(got, want)):
        assert a.dtype == np.int64 and np.array_equal(a, w), f"{strategy} batch {b}"


@pytest.mark.parametrize("strategy", ["MRD", "LRU", "2Q"])
@pytest.mark.parametrize("budget,bs,seed", [(7, 50, 1), (40, 120, 2), (300, 200, 3), (2, 64, 4)])
def test_plans_match_oracle_on_tight_budgets(strategy, budget, bs, seed):
    """Small budgets put the ties of the sort and the random evictions right at the cut-off."""
    import dataclasses
    from orca_b200 import synthetic
    spec = dataclasses.replace(synthetic.SPECS["t_nb2"], n_src=400, n_edges=3000, bs=bs, budget=budget)
    g = synthetic.make_graph(spec, seed=seed)
    adj, nbr = _tables(g, bs, 10)
    got, stats = cache.plan_from_tables(strategy, g.sources, g.destinations, bs, 10, nbr, g.n_nodes, budget, seed=seed)
    rb = planner.read_batches(g.sources, g.destinations, g.timestamps, bs, 10, adj, g.n_nodes)
    want, wstats = planner.solve(strategy, rb, g.n_nodes, budget, seed=seed)
    for b, (a, w) in enumerate(zip(got, want)):
        assert np.array_equal(a, w), f"batch {b}"
    assert (int(stats[0]), int(stats[1])) == wstats[:2]


def test_unknown_strategy_exits():
    g = graph("t_nb2")
    with pytest.raises(SystemExit):
        cache.plan_from_tables("FIFO", g.sources, g.destinations, 200, 10, np.zeros((2 * g.n_edges, 10), np.int32),
                               g.n_nodes, 10)
