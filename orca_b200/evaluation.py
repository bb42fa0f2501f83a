"""``eval_edge_prediction`` with the signature and return value of the reference's evaluation loop
(evaluation/evaluation.py:6-47): mean average precision, AUC and accuracy over the batches of the
stream, one uniform negative destination per positive edge drawn batch by batch from the sampler.

The reference calls the model once per batch and brings the scores back per batch; here the
negatives of all batches are drawn first (same draws, same order: the sampler is consumed exactly as
the reference consumes it) and the whole stream goes through ``TGN.eval_epoch`` -- one library call.
The metrics are scikit-learn's, per batch, as in the reference.
"""
from __future__ import annotations

import math

import numpy as np
from sklearn.metrics import accuracy_score, average_precision_score, roc_auc_score


class RandEdgeSampler:
    """Uniform negative sampler with the interface of utils/util.py:68-87: sample(size) draws `size`
    source indices and then `size` destination indices from one seeded RandomState over the sorted
    unique id lists."""

    def __init__(self, src_list, dst_list, seed=None):
        self.seed = seed
        self.src_list = np.unique(src_list)
        self.dst_list = np.unique(dst_list)
        self.random_state = np.random.RandomState(seed) if seed is not None else np.random

    def sample(self, size):
        src_index = self.random_state.randint(0, len(self.src_list), size)
        dst_index = self.random_state.randint(0, len(self.dst_list), size)
        return self.src_list[src_index], self.dst_list[dst_index]

    def reset_random_state(self):
        self.random_state = np.random.RandomState(self.seed)


def eval_edge_prediction(model, negative_edge_sampler, data, n_neighbors, batch_size, reuse=True, cache_plan=None):
    assert negative_edge_sampler.seed is not None
    negative_edge_sampler.reset_random_state()
    model = model.eval()
    n = data.n_interactions
    nb = math.ceil(n / batch_size)
    negatives = np.empty(n, dtype=np.int64)
    for i in range(nb):
        lo, hi = i * batch_size, min(n, (i + 1) * batch_size)
        _, negatives[lo:hi] = negative_edge_sampler.sample(hi - lo)
    pos, neg = model.eval_epoch(data.sources[:n], data.destinations[:n], negatives, data.timestamps[:n],
                                data.edge_idxs[:n], n_neighbors, batch_size, cache_plan, reuse=reuse)
    val_ap, val_auc, val_acc = [], [], []
    for i in range(nb):
        lo, hi = i * batch_size, min(n, (i + 1) * batch_size)
        size = hi - lo
        pred_score = np.concatenate([pos[lo:hi], neg[lo:hi]])
        true_label = np.concatenate([np.ones(size), np.zeros(size)])
        val_ap.append(average_precision_score(true_label, pred_score))
        val_auc.append(roc_auc_score(true_label, pred_score))
        # evaluation/evaluation.py:39-40: the positive "wins" when its score is not below the negative's
        val_acc.append(accuracy_score(np.zeros(size), np.argmax(np.stack([pos[lo:hi], neg[lo:hi]], axis=1), axis=1)))
    return np.mean(val_ap), np.mean(val_auc), np.mean(val_acc)
