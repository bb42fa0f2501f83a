"""End-to-end parity on the GPU: the drop-in ``TGN`` against (a) the golden fixtures produced by
the reference itself and (b) the CPU oracle on the same seeded inputs.

Tolerances: link scores within 1e-3 relative (the bound the path is specified to; the fp32 kernels
measure ~1e-5), state tables within 1e-3 relative to a 0.05 floor, average precision to 3 decimals,
uncached sets / cache flags / counters identical."""
import argparse

import numpy as np
import pytest
import torch
from sklearn.metrics import average_precision_score

from helpers import batches, golden, graph, max_rel, state_dict, unpack

pytestmark = pytest.mark.gpu

CASES = ["c1", "t_bip2", "t_nb2", "t_lru", "t_2q", "c2_prefix"]


def make_model(g, device="cuda:0", reuse=True, budget=None):
    from orca_b200.neighbor_finder import get_neighbor_finder
    from orca_b200.tgn import TGN
    spec = g.spec
    nf = get_neighbor_finder(g, device=device)
    budget = spec.budget if budget is None else budget
    args = argparse.Namespace(bs=spec.bs, n_degree=spec.n_degree, budget=budget, reuse=reuse, gradient=False,
                              n_nodes=g.n_nodes, n_edges=g.n_edges + 1)
    tgn = TGN(neighbor_finder=nf, node_features=None, edge_features=g.edge_features, device=torch.device(device),
              n_layers=spec.n_layers, n_heads=2, dropout=0.1, use_memory=True, node_dimension=172,
              time_dimension=172, memory_dimension=172, embedding_module_type="graph_attention",
              message_function="identity", aggregator_type="last", memory_updater_type="gru",
              n_neighbors=spec.n_degree, args=args)
    sd = {k: torch.from_numpy(v) for k, v in state_dict(spec.n_layers).items()}
    sd["embedding_module.time_encoder.w.weight"] = sd["time_encoder.w.weight"]
    sd["embedding_module.time_encoder.w.bias"] = sd["time_encoder.w.bias"]
    tgn.load_state_dict(sd, strict=True)
    tgn.eval()
    return tgn


@pytest.mark.parametrize("case", CASES)
def test_eval_matches_reference_fixture(case):
    gold = golden(case)
    g = graph(str(gold["spec"]))
    spec = g.spec
    plan = unpack(gold[f"plan_{spec.strategy}_flat"], gold[f"plan_{spec.strategy}_off"])
    scores = gold["scores"]
    nb = scores.shape[0]
    neg = gold["neg"]
    tgn = make_model(g)
    want_u = unpack(gold["u_flat"], gold["u_off"]) if spec.n_layers > 1 else None
    worst, aps = 0.0, []
    for b, src, dst, ts, eidx in batches(g, nb):
        n = len(src)
        ng = neg[b * spec.bs: b * spec.bs + n]
        if b in gold["emb_batches"]:
            # embeddings of this batch, taken from a throw-away copy of the state
            pass
        p, q = tgn.compute_edge_probabilities(src, dst, ng, ts, eidx, spec.n_degree, True, False, plan[b])
        n1, n_pos, launches = tgn.check_status()
        assert p.shape == (n, 1) and q.shape == (n, 1)
        p, q = p.cpu().numpy().ravel(), q.cpu().numpy().ravel()
        worst = max(worst, max_rel(p, scores[b, 0, :n]), max_rel(q, scores[b, 1, :n]))
        aps.append(average_precision_score(np.r_[np.ones(n), np.zeros(n)], np.r_[p, q]))
        assert n_pos == len(np.unique(np.r_[src, dst]))
        assert launches > 0
        if want_u is not None:
            assert n1 == 3 * n + len(want_u[b]), f"batch {b}"
    assert worst < 1e-3, worst
    assert round(float(np.mean(aps)), 3) == round(float(gold["ap"]), 3)
    pick = gold["state_nodes"].astype(np.int64)
    mem = tgn.memory
    assert max_rel(mem.memory[pick].cpu().numpy(), gold["state_memory"], floor=0.05) < 1e-3
    assert np.array_equal(mem.last_update[pick].cpu().numpy(), gold["state_last_update"])
    assert max_rel(mem.messages[pick[:32]].cpu().numpy(), gold["state_messages"], floor=0.05) < 1e-3
    assert np.array_equal(mem.timestamps[pick].cpu().numpy(), gold["state_msg_ts"])
    assert np.array_equal(mem.nodes[pick].astype(np.uint8), gold["state_flags"])
    if spec.n_layers > 1:
        h = tgn.embedding_module.histories[0]
        assert max_rel(h.emb[pick].cpu().numpy(), gold["state_history"], floor=0.05) < 1e-3
        assert np.array_equal(np.nonzero(h.cache_flag)[0], gold["cache_flag_nodes"])


@pytest.mark.parametrize("case", ["t_nb2", "c1"])
def test_embeddings_match_reference_fixture(case):
    gold = golden(case)
    g = graph(str(gold["spec"]))
    spec = g.spec
    plan = unpack(gold[f"plan_{spec.strategy}_flat"], gold[f"plan_{spec.strategy}_off"])
    neg = gold["neg"]
    tgn = make_model(g)
    for b, src, dst, ts, eidx in batches(g, gold["scores"].shape[0]):
        n = len(src)
        ng = neg[b * spec.bs: b * spec.bs + n]
        s, d, q = tgn.compute_temporal_embeddings(src, dst, ng, ts, eidx, spec.n_degree, True, False, plan[b])
        if b in gold["emb_batches"]:
            want = gold[f"emb_{b}"]
            for got, w in zip((s, d, q), want):
                assert max_rel(got[:32].cpu().numpy(), w, floor=0.05) < 1e-3
    tgn.check_status()


def test_eval_matches_oracle_on_fresh_inputs():
    """Not a fixture: a graph, weights and negatives the fixtures never saw, oracle run live."""
    import dataclasses
    from orca_b200 import params, synthetic
    from oracle import planner, tgn_oracle
    spec = dataclasses.replace(synthetic.SPECS["t_nb2"], name="fresh", n_src=900, n_edges=4000, budget=60, bs=250)
    g = synthetic.make_graph(spec, seed=11)
    adj = tgn_oracle.Adjacency(g.sources, g.destinations, g.edge_idxs, g.timestamps, g.n_nodes)
    plan = planner.get_cache_plan(g.sources, g.destinations, g.timestamps, spec.bs, spec.n_degree, spec.budget, adj,
                                  g.n_nodes, "MRD")
    sd = params.random_state_dict(2, seed=9)
    orc = tgn_oracle.OracleTGN(adj, g.edge_features, sd, g.n_nodes, n_layers=2, budget=spec.budget)
    tgn = make_model(g)
    t = {k: torch.from_numpy(v) for k, v in sd.items()}
    t["embedding_module.time_encoder.w.weight"] = t["time_encoder.w.weight"]
    t["embedding_module.time_encoder.w.bias"] = t["time_encoder.w.bias"]
    tgn.load_state_dict(t)
    neg = synthetic.negative_destinations(g, seed=5)
    worst = 0.0
    for b, src, dst, ts, eidx in batches(g):
        ng = neg[b * spec.bs: b * spec.bs + len(src)]
        # every third batch runs without a plan (the cumulative flag rule)
        pl = None if b % 3 == 2 else plan[b]
        wp, wq = orc.compute_edge_probabilities(src, dst, ng, ts, eidx, spec.n_degree, pl)
        p, q = tgn.compute_edge_probabilities(src, dst, ng, ts, eidx, spec.n_degree, True, False, pl)
        worst = max(worst, max_rel(p.cpu().numpy(), wp.numpy()), max_rel(q.cpu().numpy(), wq.numpy()))
        tgn.check_status()
    assert worst < 1e-3, worst
    assert max_rel(tgn.memory.memory.cpu().numpy(), orc.memory.numpy(), floor=0.05) < 1e-3
    assert max_rel(tgn.embedding_module.histories[0].emb.cpu().numpy(), orc.hist[0].numpy(), floor=0.05) < 1e-3
    assert np.array_equal(tgn.embedding_module.histories[0].cache_flag != 0, orc.cache_flag[0] != 0)


def test_large_uncached_sets_take_the_bitmap_path():
    """Batches whose uncached set exceeds the candidate list (ORCA_CAND_CAP) fall back to the bitmap
    scan; both finishes must give the oracle's rows (counts, scores, pushed history rows)."""
    import dataclasses
    from orca_b200 import _lib, params, synthetic
    from oracle import tgn_oracle
    spec = dataclasses.replace(synthetic.SPECS["t_nb2"], name="wide", n_src=30000, n_edges=24000, budget=40, bs=1500,
                               zipf_src=0.3, zipf_dst=0.3)
    g = synthetic.make_graph(spec, seed=3)
    adj = tgn_oracle.Adjacency(g.sources, g.destinations, g.edge_idxs, g.timestamps, g.n_nodes)
    sd = params.random_state_dict(2, seed=4)
    orc = tgn_oracle.OracleTGN(adj, g.edge_features, sd, g.n_nodes, n_layers=2, budget=spec.budget)
    tgn = make_model(g)
    t = {k: torch.from_numpy(v) for k, v in sd.items()}
    t["embedding_module.time_encoder.w.weight"] = t["time_encoder.w.weight"]
    t["embedding_module.time_encoder.w.bias"] = t["time_encoder.w.bias"]
    tgn.load_state_dict(t)
    neg = synthetic.negative_destinations(g, seed=6)
    worst, sizes = 0.0, []
    for b, src, dst, ts, eidx in batches(g, 8):
        ng = neg[b * spec.bs: b * spec.bs + len(src)]
        pl = np.zeros(0, dtype=np.int64)     # empty plan: nothing stays cached
        rec = []
        wp, wq = orc.compute_edge_probabilities(src, dst, ng, ts, eidx, spec.n_degree, pl, record=rec)
        p, q = tgn.compute_edge_probabilities(src, dst, ng, ts, eidx, spec.n_degree, True, False, pl)
        n1, _, _ = tgn.check_status()
        assert n1 == 3 * len(src) + len(rec[0]), f"batch {b}"
        sizes.append(len(rec[0]))
        worst = max(worst, max_rel(p.cpu().numpy(), wp.numpy()), max_rel(q.cpu().numpy(), wq.numpy()))
    assert min(sizes[1:]) < _lib.CAND_CAP < max(sizes), sizes     # both finishes were exercised
    assert worst < 1e-3, worst
    assert max_rel(tgn.embedding_module.histories[0].emb.cpu().numpy(), orc.hist[0].numpy(), floor=0.05) < 1e-3


@pytest.mark.parametrize("case,reuse", [("t_nb2_reuse0", True), ("t_nb2_noreuse", False)])
def test_other_recursions_match_reference_fixture(case, reuse):
    """compute_embedding_reuse (budget == 0) and compute_embedding (reuse=False) of the reference,
    modules/embedding_module.py:154-182 and :116-147."""
    gold = golden(case)
    g = graph(str(gold["spec"]))
    spec = g.spec
    scores, neg = gold["scores"], gold["neg"]
    tgn = make_model(g, reuse=reuse, budget=0)
    worst = 0.0
    for b, src, dst, ts, eidx in batches(g, scores.shape[0]):
        n = len(src)
        p, q = tgn.compute_edge_probabilities(src, dst, neg[b * spec.bs: b * spec.bs + n], ts, eidx,
                                              spec.n_degree, reuse, False, None)
        n1, n_pos, _ = tgn.check_status()
        assert n1 == (3 * n if reuse else 3 * n * (1 + spec.n_degree))
        assert n_pos == len(np.unique(np.r_[src, dst]))
        worst = max(worst, max_rel(p.cpu().numpy().ravel(), scores[b, 0, :n]),
                    max_rel(q.cpu().numpy().ravel(), scores[b, 1, :n]))
    assert worst < 1e-3, worst
    pick = gold["state_nodes"].astype(np.int64)
    assert max_rel(tgn.memory.memory[pick].cpu().numpy(), gold["state_memory"], floor=0.05) < 1e-3
    if reuse:
        h = tgn.embedding_module.histories[0]
        assert max_rel(h.emb[pick].cpu().numpy(), gold["state_history"], floor=0.05) < 1e-3


def test_recursions_share_one_model():
    """The call's `reuse` argument picks the recursion per batch (model/tgn_model.py:114-120): a model
    built with history tables also serves reuse=False, and gives the scores of a model without."""
    g = graph("t_nb2")
    a, b = make_model(g, reuse=True), make_model(g, reuse=False, budget=0)
    spec = g.spec
    for i, src, dst, ts, eidx in batches(g, 3):
        neg = np.roll(dst, 1)
        pa, qa = a.compute_edge_probabilities(src, dst, neg, ts, eidx, spec.n_degree, False, False, None)
        pb, qb = b.compute_edge_probabilities(src, dst, neg, ts, eidx, spec.n_degree, False, False, None)
        a.check_status(), b.check_status()
        assert torch.equal(pa, pb) and torch.equal(qa, qb)
    with pytest.raises(AttributeError):
        b.compute_edge_probabilities(src, dst, neg, ts, eidx, spec.n_degree, True, False, None)


@pytest.mark.parametrize("option", ["dependent_launch", "lookahead", "overlap"])
def test_scheduling_switches_change_nothing(option):
    """Programmatic dependent launch, the four-stream look-ahead of the batch pipeline and the side stream
    of the raw-message / GRU chain only change WHEN kernels run: scores and state tables must be bit-identical
    with each of them off."""
    from orca_b200 import _lib
    g = graph("t_nb2")
    spec = g.spec
    gold = golden("t_nb2")
    plan = unpack(gold[f"plan_{spec.strategy}_flat"], gold[f"plan_{spec.strategy}_off"])
    opt = {"dependent_launch": _lib.OPT_DEPENDENT_LAUNCH, "lookahead": _lib.OPT_LOOKAHEAD,
           "overlap": _lib.OPT_OVERLAP}[option]
    out = []
    for enable in (0, 1):
        tgn = make_model(g)
        tgn.set_option(opt, enable)
        scores = []
        for b, src, dst, ts, eidx in batches(g, 12):
            # no synchronisation between the batches: the lanes really run ahead of each other
            p, q = tgn.compute_edge_probabilities(src, dst, np.roll(dst, 1), ts, eidx, spec.n_degree, True, False,
                                                  plan[b])
            scores.append(torch.cat([p, q]))
        tgn.check_status()
        out.append((torch.cat(scores).clone(), tgn.memory.memory.clone(), tgn.memory.messages.clone(),
                    tgn.embedding_module.histories[0].emb.clone(),
                    tgn.embedding_module.histories[0].cache_flag_dev.clone()))
    for a, b in zip(out[0], out[1]):
        assert torch.equal(a, b)


def test_batches_of_changing_size_share_a_model():
    """A stream whose batches differ in size (the short last batch of every stream) lays the workspace out
    anew while the previous batch may still be in flight on the library's side streams."""
    g = graph("t_nb2")
    spec = g.spec
    sizes = [200, 37, 200, 5, 163, 200]
    ref, tgn = make_model(g), make_model(g)
    from orca_b200 import _lib
    ref.set_option(_lib.OPT_LOOKAHEAD, 0)
    lo = 0
    got, want = [], []
    for n in sizes:
        sl = slice(lo, lo + n)
        a = (g.sources[sl], g.destinations[sl], np.roll(g.destinations[sl], 1), g.timestamps[sl], g.edge_idxs[sl])
        plan = np.unique(np.r_[a[0], a[1]])[: spec.budget]
        want.append(torch.cat(ref.compute_edge_probabilities(*a, spec.n_degree, True, False, plan)))
        ref.check_status()        # the reference run is synchronised batch by batch, this one is not
        got.append(torch.cat(tgn.compute_edge_probabilities(*a, spec.n_degree, True, False, plan)))
        lo += n
    tgn.check_status()
    assert torch.equal(torch.cat(got), torch.cat(want))
    assert torch.equal(tgn.memory.memory, ref.memory.memory)
    assert torch.equal(tgn.embedding_module.histories[0].emb, ref.embedding_module.histories[0].emb)


@pytest.mark.parametrize("case", ["t_nb2", "t_lru"])
def test_eval_epoch_equals_per_batch_calls(case):
    """One library call for the whole stream (TGN.eval_epoch) gives the bits of one
    compute_edge_probabilities call per batch: scores and every state table; the stream's last batch is
    short, a few batches run without a plan."""
    gold = golden(case)
    g = graph(str(gold["spec"]))
    spec = g.spec
    plan = unpack(gold[f"plan_{spec.strategy}_flat"], gold[f"plan_{spec.strategy}_off"])
    neg = gold["neg"]
    E = (len(plan) - 1) * spec.bs - 37           # a short last batch
    nb = -(-E // spec.bs)
    a, b = make_model(g), make_model(g)
    pos, ngs = [], []
    for i in range(nb):
        sl = slice(i * spec.bs, min(E, (i + 1) * spec.bs))
        p, q = a.compute_edge_probabilities(g.sources[sl], g.destinations[sl], neg[sl], g.timestamps[sl],
                                            g.edge_idxs[sl], spec.n_degree, True, False, plan[i])
        pos.append(p.cpu().numpy().ravel()), ngs.append(q.cpu().numpy().ravel())
    a.check_status()
    p2, q2 = b.eval_epoch(g.sources[:E], g.destinations[:E], neg[:E], g.timestamps[:E], g.edge_idxs[:E],
                          spec.n_degree, spec.bs, plan[:nb])
    b.check_status()
    assert np.array_equal(np.concatenate(pos), p2) and np.array_equal(np.concatenate(ngs), q2)
    assert torch.equal(a.memory.memory, b.memory.memory) and torch.equal(a.memory.messages, b.memory.messages)
    assert torch.equal(a.embedding_module.histories[0].emb, b.embedding_module.histories[0].emb)
    assert torch.equal(a.embedding_module.histories[0].cache_flag_dev, b.embedding_module.histories[0].cache_flag_dev)
    # a second epoch on the same model (staging ring and pinned buffers reused), without plans
    p3, _ = b.eval_epoch(g.sources[:E], g.destinations[:E], neg[:E], g.timestamps[:E], g.edge_idxs[:E],
                         spec.n_degree, spec.bs, None)
    b.check_status()
    assert p3.shape == (E,) and np.all((p3 > 0) & (p3 < 1))


def test_eval_edge_prediction_reproduces_reference_ap():
    """The reference's evaluation entry point (evaluation/evaluation.py:6-47) on the whole c1 stream: the
    mean average precision of the fixture the reference produced, to 3 decimals."""
    import types
    from orca_b200.evaluation import RandEdgeSampler, eval_edge_prediction
    gold = golden("c1")
    g = graph(str(gold["spec"]))
    spec = g.spec
    plan = unpack(gold[f"plan_{spec.strategy}_flat"], gold[f"plan_{spec.strategy}_off"])
    nb = gold["scores"].shape[0]
    n = min(g.n_edges, nb * spec.bs)
    data = types.SimpleNamespace(sources=g.sources, destinations=g.destinations, timestamps=g.timestamps,
                                 edge_idxs=g.edge_idxs, n_interactions=n)
    sampler = RandEdgeSampler(g.sources, g.destinations, seed=0)
    tgn = make_model(g)
    ap, auc, acc = eval_edge_prediction(tgn, sampler, data, spec.n_degree, spec.bs, True, plan)
    tgn.check_status()
    assert round(float(ap), 3) == round(float(gold["ap"]), 3)
    assert 0.0 <= auc <= 1.0 and 0.0 <= acc <= 1.0


def test_unsupported_modes_fail_loudly():
    g = graph("t_nb2")
    tgn = make_model(g)
    src, dst, ts, eidx = g.sources[:10], g.destinations[:10], g.timestamps[:10], g.edge_idxs[:10]
    with pytest.raises(NotImplementedError):
        tgn.compute_edge_probabilities(src, dst, dst, ts, eidx, 10, True, True, None)


@pytest.mark.parametrize("world,direct", [(4, False), (8, False), (2, True), (8, True), (3, "split"), (2, "layers"),
                                          (5, "layers"), (8, "layers")])
def test_sharded_entry_points_with_emulated_ranks(world, direct):
    """The row/edge split of the multi-GPU path for more ranks than GPUs at hand: every rank is a model
    replica of its own on this GPU, the two phases are called rank after rank through the C ABI (all ranks'
    phase 1 before any phase 2, so no kernel ever waits for a later launch).  The exchange between the
    phases is a stack of the ranks' layer-1 rows, or -- direct -- the library's own peer stores into every
    replica's exchange buffer.  "split": the memory update is split by node too; "layers": the first half of
    the ranks computes layer 1 and the memory update, the second half the top layer and the scores.  Scores
    and state must equal the unsharded run."""
    from orca_b200 import _lib, shard
    L = _lib.lib()
    g = graph("t_nb2")
    spec = g.spec
    gold = golden("t_nb2")
    plan = unpack(gold[f"plan_{spec.strategy}_flat"], gold[f"plan_{spec.strategy}_off"])
    ref = make_model(g)
    ranks = [make_model(g) for _ in range(world)]
    for r, m in enumerate(ranks):
        m._rank, m._world = r, world
        # one stream for everything: the ranks share this GPU, and a rank's wait for its peers' rows must
        # never be scheduled ahead of the kernels that deliver them
        m.set_option(_lib.OPT_LOOKAHEAD, 0)
        m.set_option(_lib.OPT_OVERLAP, 0)
    dev = ref.device
    if direct:
        # the ranks' exchange buffers and flag words; on one GPU a "peer" address is a plain device address
        from orca_b200.tgn import TGN
        cap = TGN.exchange_floats(spec.bs, world, spec.n_degree, g.n_nodes)
        bufs = [torch.zeros(_lib.EXCHANGE_SLOTS * cap, device=dev) for _ in range(world)]
        flags = [torch.zeros(_lib.FLAG_WORDS, dtype=torch.int32, device=dev) for _ in range(world)]
        # "split": the memory update is split by node as well, its rows exchanged the same way
        gcap = 2 * spec.bs * 172
        grus = [torch.zeros(2 * gcap, device=dev) for _ in range(world)] if direct in ("split", "layers") else None
        for m in ranks:
            m.set_exchange([x.data_ptr() for x in bufs], [f.data_ptr() for f in flags], cap, bufs + flags,
                           [x.data_ptr() for x in grus] if grus else None, gcap)
            m._keep_gru = grus
            if direct == "layers":
                m._layer1_ranks = world // 2
    wa = world // 2 if direct == "layers" else 0        # ranks wa.. hold the scores
    wb = world - wa
    stream = _lib.stream_ptr(dev)
    k = spec.n_degree
    worst = 0.0
    for b, src, dst, ts, eidx in batches(g, 8):
        n = len(src)
        neg = np.roll(dst, 3)
        p_ref, q_ref = ref.compute_edge_probabilities(src, dst, neg, ts, eidx, k, True, False, plan[b])
        ref.check_status()
        pl = np.asarray(plan[b], dtype=np.int32)
        ints = torch.from_numpy(np.concatenate([src, dst, neg, eidx, pl]).astype(np.int32)).to(dev)
        tsd = torch.from_numpy(np.ascontiguousarray(ts, dtype=np.float64)).to(dev)
        d_plan = ints.data_ptr() + 16 * n
        locals_, ctx = [], []
        for m in ranks:
            desc = m._descriptor(k)
            ws, u_cap = m._workspace(n, k)
            rpr = shard.rows_per_rank(3 * n + u_cap, wa if wa else world)
            emb1 = torch.zeros(rpr, 172, device=dev)
            _lib.check(L.orca_tgn_eval_batch_sharded(desc, 1, ints.data_ptr(), tsd.data_ptr(), n, d_plan, len(pl),
                                                     u_cap, ws.data_ptr(), ws.numel(),
                                                     None if direct else emb1.data_ptr(), None, None,
                                                     None, m._status.data_ptr(), stream))
            locals_.append(emb1)
            ctx.append((desc, ws, u_cap))
        emb1_all = torch.stack(locals_).contiguous()
        p = torch.zeros(n, device=dev)
        q = torch.zeros(n, device=dev)
        for r, m in enumerate(ranks):
            desc, ws, u_cap = ctx[r]
            n_loc = shard.local_count(n, r - wa, wb) if r >= wa else 0
            prob = torch.zeros(2 * shard.rows_per_rank(n, wb), device=dev)
            _lib.check(L.orca_tgn_eval_batch_sharded(desc, 2, ints.data_ptr(), tsd.data_ptr(), n, d_plan, len(pl),
                                                     u_cap, ws.data_ptr(), ws.numel(), None,
                                                     None if direct else emb1_all.data_ptr(),
                                                     prob.data_ptr(), None, m._status.data_ptr(), stream))
            m.check_status()
            if r >= wa:
                e = torch.arange(r - wa, n, wb, device=dev)
                p[e] = prob[:n_loc]
                q[e] = prob[n_loc:2 * n_loc]
        worst = max(worst, float((p - p_ref.view(-1)).abs().max()), float((q - q_ref.view(-1)).abs().max()))
    assert worst < 1e-6, worst
    for m in ranks:
        assert torch.equal(m.memory.memory, ref.memory.memory)
        assert torch.equal(m.embedding_module.histories[0].emb, ref.embedding_module.histories[0].emb)
        assert np.array_equal(m.embedding_module.histories[0].cache_flag, ref.embedding_module.histories[0].cache_flag)


def test_wait_for_peers_gives_up_and_leaves_the_tables_alone():
    """A rank whose peer never delivers its rows: the bounded waits of phase 2 run out (the limit is set to
    about a millisecond), the status word reports ORCA_E_TIMEOUT, the kernels return, and neither the history
    replica nor the memory table receives rows from the incomplete exchange.  Nothing faults or hangs: the
    wait is a poll of a flag word that is never set."""
    from orca_b200 import _lib, shard
    from orca_b200.tgn import TGN
    L = _lib.lib()
    g = graph("t_nb2")
    spec = g.spec
    gold = golden("t_nb2")
    plan = unpack(gold[f"plan_{spec.strategy}_flat"], gold[f"plan_{spec.strategy}_off"])
    world = 2
    m = make_model(g)
    m._rank, m._world = 0, world
    m.set_option(_lib.OPT_LOOKAHEAD, 0)
    m.set_option(_lib.OPT_OVERLAP, 0)
    m.set_option(_lib.OPT_WAIT_LIMIT, 2_000_000)
    dev = m.device
    cap = TGN.exchange_floats(spec.bs, world, spec.n_degree, g.n_nodes)
    gcap = 2 * spec.bs * 172
    bufs = [torch.zeros(_lib.EXCHANGE_SLOTS * cap, device=dev) for _ in range(world)]
    flags = [torch.zeros(_lib.FLAG_WORDS, dtype=torch.int32, device=dev) for _ in range(world)]
    grus = [torch.zeros(2 * gcap, device=dev) for _ in range(world)]
    m.set_exchange([x.data_ptr() for x in bufs], [f.data_ptr() for f in flags], cap, bufs + flags + grus,
                   [x.data_ptr() for x in grus], gcap)
    _, src, dst, ts, eidx = next(iter(batches(g, 1)))
    n, k = len(src), spec.n_degree
    pl = np.asarray(plan[0], dtype=np.int32)
    ints = torch.from_numpy(np.concatenate([src, dst, np.roll(dst, 3), eidx, pl]).astype(np.int32)).to(dev)
    tsd = torch.from_numpy(np.ascontiguousarray(ts, dtype=np.float64)).to(dev)
    desc = m._descriptor(k)
    ws, u_cap = m._workspace(n, k)
    hist_before = m.embedding_module.histories[0].emb.clone()
    mem_before = m.memory.memory.clone()
    prob = torch.zeros(2 * shard.rows_per_rank(n, world), device=dev)
    stream = _lib.stream_ptr(dev)
    for phase in (1, 2):        # rank 1 never runs: its flag words stay zero
        _lib.check(L.orca_tgn_eval_batch_sharded(desc, phase, ints.data_ptr(), tsd.data_ptr(), n,
                                                 ints.data_ptr() + 16 * n, len(pl), u_cap, ws.data_ptr(), ws.numel(),
                                                 None, None, prob.data_ptr(), None, m._status.data_ptr(), stream))
    with pytest.raises(_lib.OrcaError) as err:
        m.check_status()
    assert err.value.code == 6          # ORCA_E_TIMEOUT
    assert torch.equal(m.embedding_module.histories[0].emb, hist_before)
    assert torch.equal(m.memory.memory, mem_before)
    # the context is still usable: an unsharded model on the same GPU runs a batch
    ok = make_model(g)
    p, q = ok.compute_edge_probabilities(src, dst, np.roll(dst, 3), ts, eidx, k, True, False, plan[0])
    ok.check_status()
    assert torch.isfinite(p).all() and torch.isfinite(q).all()


def test_device_side_errors_surface_through_the_reference_api():
    """The reference API has no status call.  What a kernel reports in the status word (here: the code a kernel
    writes when the uncached set exceeds its capacity, put there by the host so that no kernel has to fail)
    travels to pinned host memory behind each batch and is raised by the first later call that finds the copy
    complete."""
    from orca_b200 import _lib
    g = graph("t_nb2")
    spec = g.spec
    gold = golden("t_nb2")
    plan = unpack(gold[f"plan_{spec.strategy}_flat"], gold[f"plan_{spec.strategy}_off"])
    m = make_model(g)
    it = iter(batches(g, 3))
    _, src, dst, ts, eidx = next(it)
    m.compute_edge_probabilities(src, dst, np.roll(dst, 3), ts, eidx, spec.n_degree, True, False, plan[0])
    torch.cuda.synchronize()
    m._status[0] = 4                     # ORCA_E_CAPACITY, as report() would leave it
    _, src, dst, ts, eidx = next(it)
    m.compute_edge_probabilities(src, dst, np.roll(dst, 3), ts, eidx, spec.n_degree, True, False, plan[1])
    torch.cuda.synchronize()
    _, src, dst, ts, eidx = next(it)
    with pytest.raises(_lib.OrcaError) as err:
        m.compute_edge_probabilities(src, dst, np.roll(dst, 3), ts, eidx, spec.n_degree, True, False, plan[2])
    assert err.value.code == 4
