"""Seeded random weights under the reference's state-dict names.

Both sides of every parity check load the same dictionary: the reference's ``TGN`` through
``load_state_dict`` and this package's ``TGN`` through ``load_state_dict`` as well.  Names and
shapes are those of model/tgn_model.py:14-92 with ``message_function="identity"`` (the only value
that constructs; the message is the 4*D raw message, see model/tgn_model.py:49-58).
"""
from __future__ import annotations

import numpy as np

D = 172


def time_encoder_weights(dim: int = D):
    """Frozen frequencies of model/time_encoding.py:18-19: w_i = 10^(-9 i/(dim-1)) in fp32."""
    w = (1 / 10 ** np.linspace(0, 9, dim, dtype=np.float32)).astype(np.float32)
    return w.reshape(dim, 1), np.zeros(dim, dtype=np.float32)


def random_state_dict(n_layers: int = 2, seed: int = 0, dim: int = D, edge_dim: int = D,
                      time_dim: int = D):
    """Returns {name: float32 ndarray}.  Weights are uniform with Xavier bounds; biases and
    LayerNorm affine parameters are perturbed away from 0/1 so that every term is exercised."""
    rs = np.random.RandomState(seed)

    def W(out_f, in_f):
        a = np.sqrt(6.0 / (in_f + out_f))
        return rs.uniform(-a, a, size=(out_f, in_f)).astype(np.float32)

    def b(n, s=0.05):
        return rs.uniform(-s, s, size=n).astype(np.float32)

    sd = {}
    tw, tb = time_encoder_weights(time_dim)
    sd["time_encoder.w.weight"] = tw
    sd["time_encoder.w.bias"] = tb
    msg = 2 * dim + edge_dim + time_dim
    sd["memory_updater.memory_updater.weight_ih"] = W(3 * dim, msg)
    sd["memory_updater.memory_updater.weight_hh"] = W(3 * dim, dim)
    sd["memory_updater.memory_updater.bias_ih"] = b(3 * dim)
    sd["memory_updater.memory_updater.bias_hh"] = b(3 * dim)
    sd["memory_updater.layer_norm.weight"] = np.ones(dim, dtype=np.float32)
    sd["memory_updater.layer_norm.bias"] = np.zeros(dim, dtype=np.float32)
    qd = dim + time_dim
    kd = dim + edge_dim + time_dim
    for l in range(n_layers):
        p = f"embedding_module.attention_models.{l}."
        sd[p + "multi_head_target.q_proj_weight"] = W(qd, qd)
        sd[p + "multi_head_target.k_proj_weight"] = W(qd, kd)
        sd[p + "multi_head_target.v_proj_weight"] = W(qd, kd)
        sd[p + "multi_head_target.in_proj_bias"] = b(3 * qd)
        sd[p + "multi_head_target.out_proj.weight"] = W(qd, qd)
        sd[p + "multi_head_target.out_proj.bias"] = b(qd)
        sd[p + "merger.fc1.weight"] = W(dim, qd + dim)
        sd[p + "merger.fc1.bias"] = b(dim)
        sd[p + "merger.fc2.weight"] = W(dim, dim)
        sd[p + "merger.fc2.bias"] = b(dim)
        sd[p + "norm.weight"] = (1.0 + b(dim, 0.1)).astype(np.float32)
        sd[p + "norm.bias"] = b(dim)
    sd["affinity_score.fc1.weight"] = W(dim, 2 * dim)
    sd["affinity_score.fc1.bias"] = b(dim)
    sd["affinity_score.fc2.weight"] = W(1, dim)
    sd["affinity_score.fc2.bias"] = b(1)
    return sd
