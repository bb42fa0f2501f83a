"""Dataset ingestion with the interface of utils/data_processing.py:6-112 and utils/preprocess_data.py:9-80:
``Data``, ``load_feat``, ``get_data`` (chronological 70 / 15 / 15 split with a tenth of the nodes held out
for inductive testing) and ``preprocess`` / ``reindex`` / ``run`` (raw ``<name>.csv`` -> ``ml_<name>.csv`` +
``ml_<name>.npy``).  Host-side file handling only; everything downstream (``get_neighbor_finder``,
``get_cache_plan``, ``TGN``) takes the arrays these functions return.

Differences a caller can observe:

* the data directory is an argument (the reference hard-codes ``../data`` and ``./data``);
* the masks are computed with NumPy set operations instead of per-row Python lambdas;
* ``random.sample`` no longer accepts a set (Python 3.11): the held-out nodes are drawn from
  ``tuple(test_node_set)``, which is what older interpreters did with the set internally, so the draw is
  the same for the same interpreter's set order.
"""
from __future__ import annotations

import os
import random

import numpy as np
import pandas as pd


class Data:
    """utils/data_processing.py:6-29."""

    def __init__(self, sources, destinations, timestamps, edge_idxs, labels):
        self.sources = sources
        self.destinations = destinations
        self.timestamps = timestamps
        self.edge_idxs = edge_idxs
        self.labels = labels
        self.n_interactions = len(sources)
        self.unique_nodes = set(sources) | set(destinations)
        self.n_unique_nodes = len(self.unique_nodes)
        self.tbatch = None
        self.n_batch = 0

    def sample(self, ratio):
        size = int(ratio * self.n_interactions)
        inds = np.sort(random.sample(range(self.n_interactions), size)).astype(np.int64)
        return Data(self.sources[inds], self.destinations[inds], self.timestamps[inds], self.edge_idxs[inds],
                    self.labels[inds])


def _paths(d, data_dir):
    base = os.path.join(data_dir, d)
    return (os.path.join(base, f"ml_{d}.csv"), os.path.join(base, f"ml_{d}.npy"),
            os.path.join(base, f"ml_{d}_node.npy"))


def load_feat(d, data_dir="../data"):
    """utils/data_processing.py:31-40: (node features, edge features), None where the file is absent."""
    _, edge_path, node_path = _paths(d, data_dir)
    node_feats = np.load(node_path) if os.path.exists(node_path) else None
    edge_feats = np.load(edge_path) if os.path.exists(edge_path) else None
    return node_feats, edge_feats


def get_data(dataset_name, data_dir="../data", verbose=True):
    """utils/data_processing.py:43-112.  Returns (full, train, val, test, new-node val, new-node test,
    number of nodes, number of edges)."""
    graph_df = pd.read_csv(_paths(dataset_name, data_dir)[0])
    val_time, test_time = list(np.quantile(graph_df.ts, [0.70, 0.85]))
    sources = graph_df.u.values
    destinations = graph_df.i.values
    edge_idxs = graph_df.idx.values
    labels = graph_df.label.values
    timestamps = graph_df.ts.values
    full_data = Data(sources, destinations, timestamps, edge_idxs, labels)

    random.seed(2020)
    node_set = set(sources) | set(destinations)
    n_total_unique_nodes = len(node_set)
    n_edges = len(sources)

    late = timestamps > val_time
    test_node_set = set(sources[late]).union(set(destinations[late]))
    new_test_node_set = set(random.sample(tuple(test_node_set), int(0.1 * n_total_unique_nodes)))
    held = np.fromiter(new_test_node_set, dtype=np.asarray(sources).dtype, count=len(new_test_node_set))
    observed = ~np.isin(sources, held) & ~np.isin(destinations, held)
    train_mask = (timestamps <= val_time) & observed

    def part(mask):
        return Data(sources[mask], destinations[mask], timestamps[mask], edge_idxs[mask], labels[mask])

    train_data = part(train_mask)
    train_node_set = set(train_data.sources).union(train_data.destinations)
    assert len(train_node_set & new_test_node_set) == 0
    new_node_set = node_set - train_node_set     # (the validation set may contain held-out nodes)
    new_nodes = np.fromiter(new_node_set, dtype=np.asarray(sources).dtype, count=len(new_node_set))
    val_mask = (timestamps <= test_time) & (timestamps > val_time)
    test_mask = timestamps > test_time
    has_new = np.isin(sources, new_nodes) | np.isin(destinations, new_nodes)
    val_data, test_data = part(val_mask), part(test_mask)
    new_node_val_data, new_node_test_data = part(val_mask & has_new), part(test_mask & has_new)

    if verbose:
        print("The dataset has {} interactions, involving {} different nodes".format(
            full_data.n_interactions, full_data.n_unique_nodes))
        for name, d in (("training", train_data), ("validation", val_data), ("test", test_data),
                        ("new node validation", new_node_val_data), ("new node test", new_node_test_data)):
            print("The {} dataset has {} interactions, involving {} different nodes".format(
                name, d.n_interactions, d.n_unique_nodes))
        print("{} nodes were used for the inductive testing, i.e. are never seen during training".format(
            len(new_test_node_set)))
    return (full_data, train_data, val_data, test_data, new_node_val_data, new_node_test_data,
            n_total_unique_nodes, n_edges)


def preprocess(data_name):
    """utils/preprocess_data.py:9-40: the raw file has a header line, then ``u, i, ts, label, f0, f1, ...``."""
    raw = np.loadtxt(data_name, delimiter=",", skiprows=1, ndmin=2, dtype=np.float64)
    n = raw.shape[0]
    df = pd.DataFrame({"u": raw[:, 0].astype(np.int64), "i": raw[:, 1].astype(np.int64), "ts": raw[:, 2],
                       "label": raw[:, 3], "idx": np.arange(n, dtype=np.int64)})
    return df, np.ascontiguousarray(raw[:, 4:])


def reindex(df, bipartite=True):
    """utils/preprocess_data.py:43-66: ids start at 1 (0 is the padding node); items follow the users."""
    new_df = df.copy()
    if bipartite:
        assert df.u.max() - df.u.min() + 1 == len(df.u.unique())
        assert df.i.max() - df.i.min() + 1 == len(df.i.unique())
        new_df.i = df.i + (df.u.max() + 1)
    new_df.u += 1
    new_df.i += 1
    new_df.idx += 1
    return new_df


def run(data_name, bipartite=True, data_dir="./data"):
    """utils/preprocess_data.py:69-86: writes ml_<name>.csv and ml_<name>.npy (row 0 = zeros for the
    padding edge) next to <name>.csv."""
    base = os.path.join(data_dir, data_name)
    df, feat = preprocess(os.path.join(base, f"{data_name}.csv"))
    reindex(df, bipartite).to_csv(os.path.join(base, f"ml_{data_name}.csv"))
    np.save(os.path.join(base, f"ml_{data_name}.npy"), np.vstack([np.zeros((1, feat.shape[1])), feat]))
