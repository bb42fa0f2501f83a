"""Pins the CPU oracle against fixtures produced by the reference itself (CPU only)."""
import numpy as np
import pytest
from sklearn.metrics import average_precision_score

from helpers import batches, golden, graph, max_rel, state_dict, unpack
from oracle import planner, tgn_oracle

CASES = ["c1", "t_bip2", "t_nb2", "t_lru", "t_2q", "c2_prefix"]
SMALL = ["c1", "t_bip2", "t_nb2", "t_lru", "t_2q"]


def _adj(g):
    return tgn_oracle.Adjacency(g.sources, g.destinations, g.edge_idxs, g.timestamps, g.n_nodes)


@pytest.mark.parametrize("case", CASES)
def test_generator_is_pinned(case):
    gold = golden(case)
    assert graph(str(gold["spec"])).sha256() == str(gold["graph_sha"])


@pytest.mark.parametrize("case", CASES)
def test_sampler_tables(case):
    gold = golden(case)
    g = graph(str(gold["spec"]))
    adj = _adj(g)
    neg = gold["neg"]
    bs = g.spec.bs
    for b in gold["emb_batches"]:
        s, e = b * bs, min(g.n_edges, (b + 1) * bs)
        nodes = np.concatenate([g.sources[s:e], g.destinations[s:e], neg[s:e]])
        tt = np.tile(g.timestamps[s:e], 3)
        nbr, eid, et = tgn_oracle.sample_neighbors(adj, nodes, tt, g.spec.n_degree)
        assert np.array_equal(nbr, gold[f"samp_{b}_nbr"])
        assert np.array_equal(eid, gold[f"samp_{b}_eid"])
        assert et.tobytes() == gold[f"samp_{b}_et"].tobytes()


@pytest.mark.parametrize("case", SMALL)
@pytest.mark.parametrize("strategy", ["MRD", "LRU", "2Q"])
def test_plans_bit_exact(case, strategy):
    gold = golden(case)
    g = graph(str(gold["spec"]))
    want = unpack(gold[f"plan_{strategy}_flat"], gold[f"plan_{strategy}_off"])
    got = planner.get_cache_plan(g.sources, g.destinations, g.timestamps, g.spec.bs, g.spec.n_degree,
                                 g.spec.budget, _adj(g), g.n_nodes, strategy, seed=0)
    assert len(got) == len(want)
    for b, (a, w) in enumerate(zip(got, want)):
        assert np.array_equal(a, w), f"{strategy} batch {b}"


def test_plan_c2_prefix():
    gold = golden("c2_prefix")
    g = graph("c2")
    want = unpack(gold["plan_MRD_flat"], gold["plan_MRD_off"])
    got = planner.get_cache_plan(g.sources, g.destinations, g.timestamps, g.spec.bs, g.spec.n_degree,
                                 g.spec.budget, _adj(g), g.n_nodes, "MRD")
    import hashlib
    h = hashlib.sha256()
    for p in got:
        h.update(np.asarray(p, dtype=np.int64).tobytes())
        h.update(b"|")
    assert h.hexdigest() == str(gold["plan_MRD_sha"])
    for a, w in zip(got, want):
        assert np.array_equal(a, w)


@pytest.mark.parametrize("case", CASES)
def test_forward_matches_reference(case):
    gold = golden(case)
    g = graph(str(gold["spec"]))
    spec = g.spec
    plan = unpack(gold[f"plan_{spec.strategy}_flat"], gold[f"plan_{spec.strategy}_off"])
    scores = gold["scores"]
    nb = scores.shape[0]
    model = tgn_oracle.OracleTGN(_adj(g), g.edge_features, state_dict(spec.n_layers), g.n_nodes,
                                 n_layers=spec.n_layers, budget=spec.budget)
    neg = gold["neg"]
    u_rec = []
    aps = []
    worst = 0.0
    for b, src, dst, ts, eidx in batches(g, nb):
        n = len(src)
        ng = neg[b * spec.bs: b * spec.bs + n]
        p, q = model.compute_edge_probabilities(src, dst, ng, ts, eidx, spec.n_degree, plan[b], record=u_rec)
        p, q = p.numpy().ravel(), q.numpy().ravel()
        worst = max(worst, max_rel(p, scores[b, 0, :n]), max_rel(q, scores[b, 1, :n]))
        aps.append(average_precision_score(np.r_[np.ones(n), np.zeros(n)], np.r_[p, q]))
    assert worst < 2e-5, worst
    assert abs(np.mean(aps) - float(gold["ap"])) < 5e-4
    if spec.n_layers > 1:
        want_u = unpack(gold["u_flat"], gold["u_off"])
        assert len(u_rec) == len(want_u)
        for a, w in zip(u_rec, want_u):
            assert np.array_equal(a, w)
        pick = gold["state_nodes"].astype(np.int64)
        assert max_rel(model.hist[0][pick].numpy(), gold["state_history"], floor=0.05) < 2e-4
        assert np.array_equal(np.nonzero(model.cache_flag[0])[0], gold["cache_flag_nodes"])
    pick = gold["state_nodes"].astype(np.int64)
    assert max_rel(model.memory[pick].numpy(), gold["state_memory"], floor=0.05) < 2e-4
    assert np.array_equal(model.last_update[pick].numpy(), gold["state_last_update"])
    assert max_rel(model.messages[pick[:32]].numpy(), gold["state_messages"], floor=0.05) < 2e-4
    assert np.array_equal(model.msg_ts[pick].numpy(), gold["state_msg_ts"])
    assert np.array_equal(model.msg_flag[pick].astype(np.uint8), gold["state_flags"])


@pytest.mark.parametrize("case,reuse,budget", [("t_nb2_reuse0", True, 0), ("t_nb2_noreuse", False, 0)])
def test_other_recursions_match_reference(case, reuse, budget):
    """Unlimited reuse (modules/embedding_module.py:154-182) and no reuse (:116-147)."""
    gold = golden(case)
    g = graph(str(gold["spec"]))
    spec = g.spec
    scores = gold["scores"]
    model = tgn_oracle.OracleTGN(_adj(g), g.edge_features, state_dict(spec.n_layers), g.n_nodes,
                                 n_layers=spec.n_layers, budget=budget)
    neg = gold["neg"]
    worst = 0.0
    for b, src, dst, ts, eidx in batches(g, scores.shape[0]):
        n = len(src)
        p, q = model.compute_edge_probabilities(src, dst, neg[b * spec.bs: b * spec.bs + n], ts, eidx,
                                                spec.n_degree, None, reuse=reuse)
        worst = max(worst, max_rel(p.numpy().ravel(), scores[b, 0, :n]), max_rel(q.numpy().ravel(), scores[b, 1, :n]))
    assert worst < 2e-5, worst
    pick = gold["state_nodes"].astype(np.int64)
    assert max_rel(model.memory[pick].numpy(), gold["state_memory"], floor=0.05) < 2e-4
    if reuse:
        assert max_rel(model.hist[0][pick].numpy(), gold["state_history"], floor=0.05) < 2e-4
