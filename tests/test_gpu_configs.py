"""The three large workloads (c3: K=20, LRU; c4: 194 k nodes, 2Q; c5: 1.14 M nodes, MRD budget 10 000)
against the live CPU oracle, at the head of the stream and in its middle.

Plans come from the product planner (``orca_b200.cache.get_cache_plan``: GPU sampling of every batch +
the policy in the library) and are compared entry by entry with the oracle's planner over the same
half stream.  The head window starts both sides from zero state.  For the mid-stream window the GPU
path runs the stream up to the window by itself (the oracle needs 0.1 s per batch, the stream has
thousands); its state tables are then copied into the oracle, so the window compares one batch step
after another from a common state -- it does not prove the fast-forwarded state itself, which the
whole-stream fixtures of the smaller workloads cover.

Tolerances: link scores 1e-3 relative; state rows 1e-3 relative to a 0.05 floor; row counts,
uncached sets, unique-positive counts and cache flags identical."""
import argparse
import types

import numpy as np
import pytest
import torch

from helpers import graph, max_rel, state_dict

pytestmark = pytest.mark.gpu

HEAD_BATCHES = 8
MID_BATCHES = 6


def _batch(g, neg, b):
    bs = g.spec.bs
    s, e = b * bs, min(g.n_edges, (b + 1) * bs)
    return g.sources[s:e], g.destinations[s:e], neg[s:e], g.timestamps[s:e], g.edge_idxs[s:e]


def _uncached_rows(tgn, n, n1):
    """The appended layer-1 rows of the last batch: entries [3n, n1) of its row list."""
    return tgn.last_layer1_nodes(n1)[3 * n:]


def _copy_state_to_oracle(tgn, orc):
    m = tgn.memory
    orc.memory = m.memory.cpu().clone()
    orc.last_update = m.last_update.cpu().clone()
    orc.messages = m.messages.cpu().clone()
    orc.msg_ts = m.timestamps.cpu().clone()
    orc.msg_flag = m.nodes.astype(bool).copy()
    h = tgn.embedding_module.histories[0]
    orc.hist = [h.emb.cpu().clone()]
    orc.cache_flag = [np.asarray(h.cache_flag, dtype=np.float64).copy()]
    orc.first_eval = False


def _compare_window(g, neg, plan, tgn, orc, first, count, label):
    spec = g.spec
    worst = 0.0
    touched = []
    for b in range(first, first + count):
        src, dst, ng, ts, eidx = _batch(g, neg, b)
        n = len(src)
        rec = []
        wp, wq = orc.compute_edge_probabilities(src, dst, ng, ts, eidx, spec.n_degree, plan[b], record=rec)
        p, q = tgn.compute_edge_probabilities(src, dst, ng, ts, eidx, spec.n_degree, True, False, plan[b])
        n1, n_pos, _ = tgn.check_status()
        assert n1 == 3 * n + len(rec[0]), f"{label} batch {b}: layer-1 rows"
        assert np.array_equal(_uncached_rows(tgn, n, n1), rec[0]), f"{label} batch {b}: uncached set"
        assert n_pos == len(np.unique(np.r_[src, dst])), f"{label} batch {b}: unique positives"
        worst = max(worst, max_rel(p.cpu().numpy(), wp.numpy()), max_rel(q.cpu().numpy(), wq.numpy()))
        touched.append(np.r_[src, dst, ng, rec[0]])
    assert worst < 1e-3, f"{label}: scores differ by {worst}"
    # state tables on the rows the window touched (the whole tables are gigabytes at c5)
    rows = np.unique(np.concatenate(touched))[:20000]
    rt = torch.as_tensor(rows, dtype=torch.long)
    dev = rt.to(tgn.device)
    h = tgn.embedding_module.histories[0]
    assert max_rel(tgn.memory.memory[dev].cpu().numpy(), orc.memory[rt].numpy(), floor=0.05) < 1e-3, label
    assert np.array_equal(tgn.memory.last_update[dev].cpu().numpy(), orc.last_update[rt].numpy()), label
    assert max_rel(h.emb[dev].cpu().numpy(), orc.hist[0][rt].numpy(), floor=0.05) < 1e-3, label
    assert max_rel(tgn.memory.messages[dev[:2000]].cpu().numpy(), orc.messages[rt[:2000]].numpy(), floor=0.05) < 1e-3
    assert np.array_equal(np.asarray(h.cache_flag) != 0, orc.cache_flag[0] != 0), f"{label}: cache flags"


@pytest.mark.parametrize("case", ["c3", "c4", "c5"])
def test_head_and_midstream_match_live_oracle(case, capsys):
    from oracle import planner, tgn_oracle
    from orca_b200 import synthetic
    from orca_b200.cache import get_cache_plan
    from test_gpu_model import make_model

    g = graph(case)
    spec = g.spec
    neg = synthetic.negative_destinations(g, seed=0)
    mid = g.n_batches // 2
    m = (mid + MID_BATCHES) * spec.bs
    tgn = make_model(g)
    nf = tgn.embedding_module.neighbor_finder
    ns = argparse.Namespace(bs=spec.bs, n_degree=spec.n_degree, budget=spec.budget)
    half = types.SimpleNamespace(sources=g.sources[:m], destinations=g.destinations[:m], timestamps=g.timestamps[:m])

    # ---- plans: product planner against the oracle's, every batch of the half stream, entry by entry
    plan = get_cache_plan(ns, half, nf, g.n_nodes, spec.strategy)
    out = capsys.readouterr().out
    assert "n_reuse" in out and "n_recompute" in out        # the reference's statistics line
    adj = tgn_oracle.Adjacency(g.sources, g.destinations, g.edge_idxs, g.timestamps, g.n_nodes)
    rb = planner.read_batches(half.sources, half.destinations, half.timestamps, spec.bs, spec.n_degree, adj, g.n_nodes)
    want, stats = planner.solve(spec.strategy, rb, g.n_nodes, spec.budget)
    assert len(plan) == len(want) == mid + MID_BATCHES
    for b in range(len(want)):
        assert plan[b].dtype == np.int64
        assert np.array_equal(plan[b], want[b]), f"{case}: plan of batch {b}"
    assert f"n_reuse {stats[0]}, n_recompute {stats[1]}" in out

    # ---- head of the stream: both sides from zero state
    orc = tgn_oracle.OracleTGN(adj, g.edge_features, state_dict(spec.n_layers), g.n_nodes, n_layers=spec.n_layers,
                               budget=spec.budget)
    _compare_window(g, neg, plan, tgn, orc, 0, HEAD_BATCHES, f"{case} head")

    # ---- fast-forward on the GPU, hand the state to the oracle, compare the mid-stream window
    for b in range(HEAD_BATCHES, mid):
        src, dst, ng, ts, eidx = _batch(g, neg, b)
        tgn.compute_edge_probabilities(src, dst, ng, ts, eidx, spec.n_degree, True, False, plan[b])
        if b % 256 == 0:
            tgn.check_status()
    tgn.check_status()
    _copy_state_to_oracle(tgn, orc)
    _compare_window(g, neg, plan, tgn, orc, mid, MID_BATCHES, f"{case} mid-stream")
