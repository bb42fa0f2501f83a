"""Dataset ingestion (orca_b200.data_processing) against a row-by-row restatement of
utils/preprocess_data.py and utils/data_processing.py on a small synthetic interaction file."""
import os
import random

import numpy as np
import pandas as pd
import pytest

from orca_b200 import data_processing as dp


@pytest.fixture()
def raw_dataset(tmp_path):
    rs = np.random.RandomState(5)
    n, n_u, n_i, n_feat = 3000, 120, 40, 6
    u = rs.randint(0, n_u, n)
    i = rs.randint(0, n_i, n)
    u[:n_u] = np.arange(n_u)          # every id occurs (the reference asserts a dense id range)
    i[:n_i] = np.arange(n_i)
    ts = np.sort(rs.uniform(0, 1e5, n)).round(3)
    label = (rs.rand(n) < 0.05).astype(float)
    feat = rs.randn(n, n_feat).round(4)
    d = tmp_path / "toy"
    d.mkdir()
    with open(d / "toy.csv", "w") as f:
        f.write("user_id,item_id,timestamp,state_label,comma_separated_list_of_features\n")
        for r in range(n):
            f.write(",".join([str(u[r]), str(i[r]), repr(float(ts[r])), str(label[r])] + [repr(float(x)) for x in feat[r]]) + "\n")
    return str(tmp_path), u, i, ts, label, feat


def test_preprocess_and_reindex_write_the_ml_files(raw_dataset):
    data_dir, u, i, ts, label, feat = raw_dataset
    dp.run("toy", bipartite=True, data_dir=data_dir)
    df = pd.read_csv(os.path.join(data_dir, "toy", "ml_toy.csv"))
    assert list(df.columns[1:]) == ["u", "i", "ts", "label", "idx"]
    assert np.array_equal(df.u.values, u + 1)
    assert np.array_equal(df.i.values, i + u.max() + 1 + 1)        # items follow the users, ids start at 1
    assert np.array_equal(df.idx.values, np.arange(1, len(u) + 1))
    assert np.array_equal(df.ts.values, ts) and np.array_equal(df.label.values, label)
    ef = np.load(os.path.join(data_dir, "toy", "ml_toy.npy"))
    assert ef.shape == (len(u) + 1, feat.shape[1]) and not ef[0].any() and np.array_equal(ef[1:], feat)
    node_feats, edge_feats = dp.load_feat("toy", data_dir)
    assert node_feats is None and np.array_equal(edge_feats, ef)
    # a non-bipartite graph keeps one id space
    df2 = dp.reindex(pd.DataFrame({"u": u, "i": i, "ts": ts, "label": label, "idx": np.arange(len(u))}), bipartite=False)
    assert np.array_equal(df2.i.values, i + 1)


def _reference_split(df):
    """utils/data_processing.py:43-96, row by row (sets and list comprehensions)."""
    val_time, test_time = list(np.quantile(df.ts, [0.70, 0.85]))
    s, d, t = df.u.values, df.i.values, df.ts.values
    random.seed(2020)
    node_set = set(s) | set(d)
    test_nodes = set(s[t > val_time]).union(set(d[t > val_time]))
    new_test = set(random.sample(tuple(test_nodes), int(0.1 * len(node_set))))
    src_new = np.array([x in new_test for x in s])
    dst_new = np.array([x in new_test for x in d])
    train = np.logical_and(t <= val_time, np.logical_and(~src_new, ~dst_new))
    train_nodes = set(s[train]).union(d[train])
    new_nodes = node_set - train_nodes
    val = np.logical_and(t <= test_time, t > val_time)
    test = t > test_time
    has_new = np.array([(a in new_nodes or b in new_nodes) for a, b in zip(s, d)])
    return train, val, test, np.logical_and(val, has_new), np.logical_and(test, has_new), len(node_set), new_test


def test_get_data_matches_the_row_by_row_split(raw_dataset, capsys):
    data_dir = raw_dataset[0]
    dp.run("toy", bipartite=True, data_dir=data_dir)
    full, train, val, test, nn_val, nn_test, n_nodes, n_edges = dp.get_data("toy", data_dir)
    out = capsys.readouterr().out
    assert "nodes were used for the inductive testing" in out
    df = pd.read_csv(os.path.join(data_dir, "toy", "ml_toy.csv"))
    m_train, m_val, m_test, m_nnv, m_nnt, want_nodes, held = _reference_split(df)
    assert n_nodes == want_nodes and n_edges == len(df) == full.n_interactions
    for part, mask in ((train, m_train), (val, m_val), (test, m_test), (nn_val, m_nnv), (nn_test, m_nnt)):
        assert np.array_equal(part.sources, df.u.values[mask])
        assert np.array_equal(part.destinations, df.i.values[mask])
        assert np.array_equal(part.timestamps, df.ts.values[mask])
        assert np.array_equal(part.edge_idxs, df.idx.values[mask])
        assert np.array_equal(part.labels, df.label.values[mask])
        assert part.n_interactions == int(mask.sum())
    assert not (set(train.sources) | set(train.destinations)) & held
    assert train.timestamps.max() <= val.timestamps.min() <= val.timestamps.max() <= test.timestamps.min()
    sub = full.sample(0.25)
    assert sub.n_interactions == int(0.25 * full.n_interactions) and np.all(np.diff(sub.timestamps) >= 0)
