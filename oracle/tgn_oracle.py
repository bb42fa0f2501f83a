"""TEST INFRASTRUCTURE ONLY -- CPU restatement of the reference's per-batch temporal-embedding path.

Only tests/, the smoke check and the CPU-baseline legs of the benchmark may import this module, and
only as the checker or the timed baseline.  Nothing here is reachable from the shipped package.

Integer work is numpy, floating-point work is plain fp32 torch on the CPU, written out as the
reference computes it (projections, softmax, GRU gates), without the algebraic re-association the
CUDA path uses.  Every function cites the reference lines it follows.

Parity status: pinned.  tests/test_oracle_golden.py checks this file against fixtures produced by
running the reference itself (tests/golden/make_golden.py) -- sampler tables, uncached sets, cache
plans, embeddings, link scores, state tables and AP.
"""
from __future__ import annotations

import math

import numpy as np
import torch


# --------------------------------------------------------------------------------------------
# adjacency and sampling
# --------------------------------------------------------------------------------------------
class Adjacency:
    """Time-sorted CSR of the undirected interaction graph (utils/util.py:91-105): every edge is
    listed under both endpoints, each node's list stably sorted by timestamp, insertion order being
    stream order with the source-side entry of an edge ahead of its destination-side entry."""

    def __init__(self, sources, destinations, edge_idxs, timestamps, n_nodes=None):
        sources = np.asarray(sources, dtype=np.int64)
        destinations = np.asarray(destinations, dtype=np.int64)
        if n_nodes is None:
            n_nodes = int(max(sources.max(), destinations.max())) + 1
        E = len(sources)
        owner = np.empty(2 * E, dtype=np.int64)
        other = np.empty(2 * E, dtype=np.int64)
        owner[0::2], owner[1::2] = sources, destinations
        other[0::2], other[1::2] = destinations, sources
        eid = np.repeat(np.asarray(edge_idxs, dtype=np.int64), 2)
        ts = np.repeat(np.asarray(timestamps, dtype=np.float64), 2)
        order = np.lexsort((ts, owner))  # stable: ties keep insertion order
        self.n_nodes = n_nodes
        self.indptr = np.zeros(n_nodes + 1, dtype=np.int64)
        np.cumsum(np.bincount(owner, minlength=n_nodes), out=self.indptr[1:])
        self.nbr = other[order].astype(np.int32)
        self.eid = eid[order].astype(np.int32)
        self.ts = ts[order]


def sample_neighbors(adj: Adjacency, nodes, timestamps, k: int):
    """utils/util.py:129-151: for each query the interactions strictly before its time
    (searchsorted, side left), the last k of them, right-aligned and zero-padded on the left.
    Returns (neighbors int32 [Q,k], edge_idxs int32 [Q,k], edge_times float32 [Q,k])."""
    nodes = np.asarray(nodes, dtype=np.int64)
    t = np.asarray(timestamps, dtype=np.float64)
    Q = len(nodes)
    kk = k if k > 0 else 1
    nbr = np.zeros((Q, kk), dtype=np.int32)
    eid = np.zeros((Q, kk), dtype=np.int32)
    et = np.zeros((Q, kk), dtype=np.float32)
    if Q == 0 or k <= 0:
        return nbr, eid, et
    beg = adj.indptr[nodes]
    lo, hi = beg.copy(), adj.indptr[nodes + 1].copy()
    while True:  # vectorised lower bound inside each node's segment
        act = lo < hi
        if not act.any():
            break
        mid = (lo + hi) >> 1
        less = np.zeros(Q, dtype=bool)
        less[act] = adj.ts[mid[act]] < t[act]
        lo = np.where(act & less, mid + 1, lo)
        hi = np.where(act & ~less, mid, hi)
    cnt = np.minimum(lo - beg, k)
    slot = np.arange(k)[None, :]
    src_pos = lo[:, None] - k + slot
    valid = slot >= (k - cnt)[:, None]
    pos = np.where(valid, src_pos, 0)
    nbr[valid] = adj.nbr[pos][valid]
    eid[valid] = adj.eid[pos][valid]
    et[valid] = adj.ts[pos][valid].astype(np.float32)
    return nbr, eid, et


def find_uncached(source_nodes, neighbors, cache_flag):
    """modules/embedding_module.py:200-212: sorted unique neighbour ids that are neither query
    nodes of the batch nor flagged as cached, and then -- unconditionally -- without the first
    entry (which is the padding node 0 whenever some slot of the table is padding)."""
    u = np.unique(neighbors)
    u = u[~np.isin(u, source_nodes)]
    u = u[np.asarray(cache_flag)[u] == 0]
    return u[1:]


def last_occurrence(nodes):
    """model/tgn_model.py:172-176: sorted unique ids and, for each, the LAST position at which
    it occurs in `nodes` (the position whose message is kept)."""
    nodes = np.asarray(nodes)
    uniq, ridx = np.unique(nodes[::-1], return_index=True)
    return uniq, len(nodes) - 1 - ridx


# --------------------------------------------------------------------------------------------
# floating-point blocks
# --------------------------------------------------------------------------------------------
def time_encode(p, t):
    """model/time_encoding.py:23-28: cos(t * w + b), fp32, t of any shape -> [..., dim]."""
    w = p["time_encoder.w.weight"].reshape(-1)
    b = p["time_encoder.w.bias"]
    return torch.cos(t.unsqueeze(-1) * w + b)


def attention_layer(p, layer, h_src, h_nbr, efeat, dt, nbr_ids, n_heads=2):
    """model/temporal_attention.py:24-56 with torch.nn.MultiheadAttention (kdim != embed_dim)
    written out.  h_src [N,D], h_nbr [N,K,D], efeat [N,K,De], dt [N,K] fp32, nbr_ids [N,K]."""
    pre = f"embedding_module.attention_models.{layer}."
    N, K, _ = h_nbr.shape
    src_t = time_encode(p, torch.zeros(N, dtype=torch.float32))
    nbr_t = time_encode(p, dt)
    q_in = torch.cat([h_src, src_t], dim=1)
    k_in = torch.cat([h_nbr, efeat, nbr_t], dim=2)
    mask = torch.as_tensor(nbr_ids == 0)
    invalid = mask.all(dim=1)
    mask = mask.clone()
    mask[invalid, 0] = False
    E = q_in.shape[1]
    bias = p[pre + "multi_head_target.in_proj_bias"]
    q = q_in @ p[pre + "multi_head_target.q_proj_weight"].T + bias[:E]
    k = k_in @ p[pre + "multi_head_target.k_proj_weight"].T + bias[E:2 * E]
    v = k_in @ p[pre + "multi_head_target.v_proj_weight"].T + bias[2 * E:]
    hd = E // n_heads
    q = (q * (1.0 / math.sqrt(hd))).view(N, n_heads, hd)
    k = k.view(N, K, n_heads, hd)
    v = v.view(N, K, n_heads, hd)
    logits = torch.einsum("nhd,nkhd->nhk", q, k)
    logits = logits.masked_fill(mask[:, None, :], float("-inf"))
    a = torch.softmax(logits, dim=2)
    ctx = torch.einsum("nhk,nkhd->nhd", a, v).reshape(N, E)
    attn = ctx @ p[pre + "multi_head_target.out_proj.weight"].T + p[pre + "multi_head_target.out_proj.bias"]
    attn = attn.masked_fill(invalid[:, None], 0.0)
    x = torch.cat([attn, h_src], dim=1)
    h = torch.relu(x @ p[pre + "merger.fc1.weight"].T + p[pre + "merger.fc1.bias"])
    y = h @ p[pre + "merger.fc2.weight"].T + p[pre + "merger.fc2.bias"]
    return torch.nn.functional.layer_norm(y, (y.shape[1],), p[pre + "norm.weight"], p[pre + "norm.bias"], 1e-5)


def gru_cell(p, x, h):
    """torch.nn.GRUCell as used by modules/memory_updater.py:38,86."""
    pre = "memory_updater.memory_updater."
    gi = x @ p[pre + "weight_ih"].T + p[pre + "bias_ih"]
    gh = h @ p[pre + "weight_hh"].T + p[pre + "bias_hh"]
    H = h.shape[1]
    r = torch.sigmoid(gi[:, :H] + gh[:, :H])
    z = torch.sigmoid(gi[:, H:2 * H] + gh[:, H:2 * H])
    n = torch.tanh(gi[:, 2 * H:] + r * gh[:, 2 * H:])
    return (1 - z) * n + z * h


def affinity(p, a, b):
    """utils/util.py:12-24 as the link scorer of model/tgn_model.py:154-157 (before sigmoid)."""
    x = torch.cat([a, b], dim=1)
    h = torch.relu(x @ p["affinity_score.fc1.weight"].T + p["affinity_score.fc1.bias"])
    return h @ p["affinity_score.fc2.weight"].T + p["affinity_score.fc2.bias"]


# --------------------------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------------------------
class OracleTGN:
    """Eval-mode forward of model/tgn_model.py:95-157 with `reuse=True` and the three embedding
    recursions of modules/embedding_module.py (no reuse :116-147, unlimited reuse :154-182,
    budgeted reuse :215-285)."""

    def __init__(self, adj: Adjacency, edge_features, state_dict, n_nodes, n_layers=2, n_heads=2,
                 budget=1000, dim=172):
        self.adj = adj
        self.p = {k: torch.as_tensor(np.asarray(v), dtype=torch.float32) for k, v in state_dict.items()}
        self.efeat = torch.as_tensor(np.asarray(edge_features), dtype=torch.float32)
        self.n_nodes, self.n_layers, self.n_heads, self.budget, self.dim = n_nodes, n_layers, n_heads, budget, dim
        self.msg_dim = 2 * dim + self.efeat.shape[1] + dim
        self.reset_state()

    def reset_state(self):
        n, d = self.n_nodes, self.dim
        # modules/memory.py:17-23
        self.memory = torch.zeros(n, d)
        self.last_update = torch.zeros(n)
        self.messages = torch.zeros(n, self.msg_dim)
        self.msg_ts = torch.zeros(n)
        self.msg_flag = np.zeros(n, dtype=bool)
        # modules/history.py:6-17, one table per layer below the top
        self.hist = [torch.zeros(n, d) for _ in range(self.n_layers - 1)]
        self.cache_flag = [np.zeros(n) for _ in range(self.n_layers - 1)]
        self.first_eval = True

    # ---- memory (modules/memory_updater.py:25-53)
    def _apply_gru(self, ids):
        if len(ids) == 0:
            return
        ids_t = torch.as_tensor(ids, dtype=torch.long)
        x = self.messages[ids_t]
        h = self.memory[ids_t]
        self.last_update[ids_t] = self.msg_ts[ids_t]
        self.memory[ids_t] = gru_cell(self.p, x, h)

    def update_memory(self, positives):
        positives = np.asarray(positives)
        self._apply_gru(positives[self.msg_flag[positives]])

    def flush_pending(self):
        ids = np.nonzero(self.msg_flag)[0]
        self._apply_gru(ids)
        self.msg_flag[ids] = False

    # ---- raw messages (model/tgn_model.py:172-191, modules/memory.py:25-28)
    def store_messages(self, cat_src, cat_dst, cat_ts, cat_eidx):
        uniq, pos = last_occurrence(cat_src)
        other = cat_dst[pos]
        t = torch.as_tensor(cat_ts[pos]).float()
        ef = self.efeat[torch.as_tensor(cat_eidx[pos], dtype=torch.long)]
        u_t = torch.as_tensor(uniq, dtype=torch.long)
        delta = t - self.last_update[u_t]
        enc = time_encode(self.p, delta)
        msg = torch.cat([self.memory[u_t], self.memory[torch.as_tensor(other, dtype=torch.long)], ef, enc], dim=1)
        self.msg_flag[uniq] = True
        self.messages[u_t] = msg
        self.msg_ts[u_t] = t
        return uniq

    # ---- per-level inputs shared by all three recursions
    def _level_inputs(self, nodes, ts, k):
        nbr, eid, et = sample_neighbors(self.adj, nodes, ts, k)
        # float64 query time minus float32 edge time, rounded to float32 last
        # (modules/embedding_module.py:266-267)
        dt = torch.as_tensor((np.asarray(ts, dtype=np.float64)[:, None] - et).astype(np.float32))
        ef = self.efeat[torch.as_tensor(eid, dtype=torch.long)]
        return nbr, dt, ef

    def embed_no_reuse(self, nodes, ts, n_layers, k):
        """modules/embedding_module.py:116-147."""
        if n_layers == 0:
            return self.memory[torch.as_tensor(nodes, dtype=torch.long)]
        nbr, dt, ef = self._level_inputs(nodes, ts, k)
        comb_nodes = np.concatenate([nodes, nbr.reshape(-1)])
        comb_ts = np.concatenate([ts, np.repeat(ts, k)])
        below = self.embed_no_reuse(comb_nodes, comb_ts, n_layers - 1, k)
        n = len(nodes)
        return attention_layer(self.p, n_layers - 1, below[:n], below[n:].view(n, k, -1), ef, dt, nbr, self.n_heads)

    def embed_reuse(self, nodes, ts, n_layers, k):
        """modules/embedding_module.py:154-182 (budget == 0: every pushed row stays usable)."""
        nbr, dt, ef = self._level_inputs(nodes, ts, k)
        n = len(nodes)
        flat = torch.as_tensor(nbr.reshape(-1), dtype=torch.long)
        h_nbr = self.memory[flat].view(n, k, -1)
        h = self.memory[torch.as_tensor(nodes, dtype=torch.long)]
        for layer in range(1, n_layers):
            h = attention_layer(self.p, layer - 1, h, h_nbr, ef, dt, nbr, self.n_heads)
            self._push(layer - 1, h, nodes)
            h_nbr = self.hist[layer - 1][flat].view(n, k, -1)
        return attention_layer(self.p, n_layers - 1, h, h_nbr, ef, dt, nbr, self.n_heads)

    def _push(self, hist_idx, x, ids):
        """modules/history.py:38-40 under deterministic execution: the last occurrence of an id
        in `ids` provides its row."""
        uniq, pos = last_occurrence(ids)
        self.hist[hist_idx][torch.as_tensor(uniq, dtype=torch.long)] = x[torch.as_tensor(pos, dtype=torch.long)]

    def embed_budget(self, nodes, ts, n_layers, k, plan, record=None):
        """modules/embedding_module.py:215-285."""
        if n_layers == 0:
            return self.memory[torch.as_tensor(nodes, dtype=torch.long)]
        nbr, dt, ef = self._level_inputs(nodes, ts, k)
        n = len(nodes)
        if n_layers == 1:
            comb_nodes = np.concatenate([nodes, nbr.reshape(-1)])
            comb_ts = np.concatenate([ts, np.repeat(ts, k)])
            below = self.embed_budget(comb_nodes, comb_ts, 0, k, plan)
            return attention_layer(self.p, 0, below[:n], below[n:].view(n, k, -1), ef, dt, nbr, self.n_heads)
        unc = find_uncached(nodes, nbr, self.cache_flag[0])
        if record is not None:
            record.append(unc.copy())
        if len(unc):
            comb_nodes = np.concatenate([nodes, unc])
            comb_ts = np.concatenate([ts, np.repeat(np.max(ts), len(unc))])
        else:
            comb_nodes, comb_ts = nodes, ts
        below = self.embed_budget(comb_nodes, comb_ts, n_layers - 1, k, plan, record)
        h_src = below[:n]
        hi = n_layers - 2
        self._push(hi, below, comb_nodes)
        h_nbr = self.hist[hi][torch.as_tensor(nbr.reshape(-1), dtype=torch.long)].view(n, k, -1)
        # modules/history.py:25-30
        if plan is not None:
            self.cache_flag[hi] = np.zeros(self.n_nodes)
            self.cache_flag[hi][np.asarray(plan, dtype=np.int64)] = 1
        else:
            self.cache_flag[hi][comb_nodes] = 1
        return attention_layer(self.p, n_layers - 1, h_src, h_nbr, ef, dt, nbr, self.n_heads)

    # ---- model/tgn_model.py:95-157, train=False
    def compute_temporal_embeddings(self, src, dst, neg, ts, eidx, k, plan=None, reuse=True, record=None):
        src, dst, neg = (np.asarray(a, dtype=np.int64) for a in (src, dst, neg))
        ts = np.asarray(ts, dtype=np.float64)
        eidx = np.asarray(eidx, dtype=np.int64)
        B = len(src)
        nodes = np.concatenate([src, dst, neg])
        tt = np.concatenate([ts, ts, ts])
        positives = np.unique(np.concatenate([src, dst]))
        if self.first_eval:
            self.flush_pending()
            self.first_eval = False
        with torch.no_grad():
            if reuse and self.budget != 0:
                emb = self.embed_budget(nodes, tt, self.n_layers, k, plan, record)
            elif reuse:
                emb = self.embed_reuse(nodes, tt, self.n_layers, k)
            else:
                emb = self.embed_no_reuse(nodes, tt, self.n_layers, k)
            self.store_messages(np.concatenate([src, dst]), np.concatenate([dst, src]),
                                np.concatenate([ts, ts]), np.concatenate([eidx, eidx]))
            self.update_memory(positives)
            self.msg_flag[positives] = False
        return emb[:B], emb[B:2 * B], emb[2 * B:]

    def compute_edge_probabilities(self, src, dst, neg, ts, eidx, k, plan=None, reuse=True, record=None):
        s, d, n = self.compute_temporal_embeddings(src, dst, neg, ts, eidx, k, plan, reuse, record)
        with torch.no_grad():
            score = affinity(self.p, torch.cat([s, s]), torch.cat([d, n]))
        B = len(src)
        return torch.sigmoid(score[:B]), torch.sigmoid(score[B:])
