"""The eval flow of the reference's train.py on a dataset read from files: preprocess -> get_data ->
get_neighbor_finder(full_data) -> get_cache_plan(val_data) -> compute_edge_probabilities over the validation
batches, against the CPU oracle fed with the same arrays (plans identical, scores within 1e-3)."""
import argparse

import numpy as np
import pytest
import torch

from helpers import max_rel, state_dict

pytestmark = pytest.mark.gpu


def _write_raw(path, n=4000, n_u=300, n_i=80, n_feat=172, seed=9):
    rs = np.random.RandomState(seed)
    u, i = rs.randint(0, n_u, n), rs.randint(0, n_i, n)
    u[:n_u], i[:n_i] = np.arange(n_u), np.arange(n_i)
    ts = np.sort(rs.uniform(0, 3e5, n)).round(2)
    feat = rs.randn(n, n_feat).astype(np.float32)
    with open(path, "w") as f:
        f.write("user_id,item_id,timestamp,state_label,comma_separated_list_of_features\n")
        for r in range(n):
            f.write(f"{u[r]},{i[r]},{float(ts[r])!r},0.0," + ",".join(repr(float(x)) for x in feat[r]) + "\n")


def test_validation_batches_of_a_dataset_read_from_files(tmp_path, capsys):
    from oracle import planner, tgn_oracle
    from orca_b200 import data_processing as dp
    from orca_b200.cache import get_cache_plan
    from orca_b200.neighbor_finder import get_neighbor_finder
    from orca_b200.tgn import TGN

    (tmp_path / "toy").mkdir()
    _write_raw(tmp_path / "toy" / "toy.csv")
    dp.run("toy", bipartite=True, data_dir=str(tmp_path))
    full, train, val, test, nn_val, nn_test, n_unique, n_edges = dp.get_data("toy", str(tmp_path), verbose=False)
    _, edge_features = dp.load_feat("toy", str(tmp_path))
    edge_features = edge_features.astype(np.float32)
    n_nodes = int(max(full.sources.max(), full.destinations.max())) + 1
    bs, k, budget = 100, 10, 150
    args = argparse.Namespace(bs=bs, n_degree=k, budget=budget, reuse=True, gradient=False, n_nodes=n_nodes,
                              n_edges=n_edges + 1)
    nf = get_neighbor_finder(full)
    tgn = TGN(neighbor_finder=nf, node_features=None, edge_features=edge_features, device=torch.device("cuda:0"),
              n_layers=2, n_heads=2, dropout=0.1, use_memory=True, node_dimension=172, time_dimension=172,
              memory_dimension=172, embedding_module_type="graph_attention", message_function="identity",
              aggregator_type="last", memory_updater_type="gru", n_neighbors=k, args=args)
    sd = {kk: torch.from_numpy(v) for kk, v in state_dict(2).items()}
    sd["embedding_module.time_encoder.w.weight"] = sd["time_encoder.w.weight"]
    sd["embedding_module.time_encoder.w.bias"] = sd["time_encoder.w.bias"]
    tgn.load_state_dict(sd, strict=True)
    tgn.eval()
    plan = get_cache_plan(args, val, nf, n_nodes, "MRD")
    capsys.readouterr()

    adj = tgn_oracle.Adjacency(full.sources, full.destinations, full.edge_idxs, full.timestamps, n_nodes)
    want_plan = planner.get_cache_plan(val.sources, val.destinations, val.timestamps, bs, k, budget, adj, n_nodes, "MRD")
    assert len(plan) == len(want_plan) == -(-val.n_interactions // bs)
    for a, w in zip(plan, want_plan):
        assert np.array_equal(a, w)
    orc = tgn_oracle.OracleTGN(adj, edge_features, state_dict(2), n_nodes, n_layers=2, budget=budget)
    rs = np.random.RandomState(0)
    worst = 0.0
    for b in range(4):
        s = slice(b * bs, min(val.n_interactions, (b + 1) * bs))
        src, dst, ts, eidx = val.sources[s], val.destinations[s], val.timestamps[s], val.edge_idxs[s]
        neg = rs.choice(np.unique(full.destinations), len(src))
        wp, wq = orc.compute_edge_probabilities(src, dst, neg, ts, eidx, k, plan[b])
        p, q = tgn.compute_edge_probabilities(src, dst, neg, ts, eidx, k, True, False, plan[b])
        tgn.check_status()
        worst = max(worst, max_rel(p.cpu().numpy(), wp.numpy()), max_rel(q.cpu().numpy(), wq.numpy()))
    assert worst < 1e-3, worst
