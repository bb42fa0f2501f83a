"""Generates the golden fixtures in this folder by running the UNMODIFIED reference.

Run where a checkout of the reference is available; its location is given by the environment
variable ORCA_REFERENCE::

    ORCA_REFERENCE=<path of the checkout> python tests/golden/make_golden.py [case ...]

The reference is imported, never copied.  Settings needed for a repeatable run:

* ``torch.use_deterministic_algorithms(True)``: the reference's ``History.push`` writes duplicate
  ids with ``emb[ids] = x`` (modules/history.py:38-40); deterministic mode makes the last
  occurrence win, every time.
* numba keeps its own Mersenne Twister; LRU and 2Q planning call ``np.random.choice`` inside
  nopython code (utils/cache.py:251,266,315,394), so the generator is seeded by a jitted helper.
* ``tgn.test_mode`` is read before it is ever assigned (model/tgn_model.py:109); it is set False.

Each fixture stores the SHA-256 of the input graph (which pins the generator), the per-batch link
scores, the cache plans, the per-batch uncached-neighbour sets, sampler outputs for a few batches,
slices of the state tables after the last batch, and the versions of the libraries that ran.
"""
import argparse
import hashlib
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("ORCA_REFERENCE")
if not REF or not os.path.isdir(REF):
    raise SystemExit("set ORCA_REFERENCE to the path of a checkout of the reference")
sys.path.insert(0, ROOT)
sys.path.insert(0, REF)

import numba  # noqa: E402
import torch  # noqa: E402

from orca_b200 import params, synthetic  # noqa: E402

# reference modules
from evaluation.evaluation import eval_edge_prediction  # noqa: E402,F401
from model.tgn_model import TGN  # noqa: E402
from modules.embedding_module import GraphEmbedding  # noqa: E402
from utils.cache import get_cache_plan  # noqa: E402
from utils.data_processing import Data  # noqa: E402
from utils.util import get_neighbor_finder  # noqa: E402


@numba.njit
def _seed_numba(s):
    np.random.seed(s)


# case name -> (graph spec name, number of leading batches to run, strategies to plan)
CASES = {
    "c1": ("c1", None),
    "t_bip2": ("t_bip2", None),
    "t_nb2": ("t_nb2", None),
    "t_lru": ("t_lru", None),
    "t_2q": ("t_2q", None),
    "c2_prefix": ("c2", 40),
    # the two other recursions of modules/embedding_module.py: unlimited reuse (budget 0, :154-182)
    # and no reuse (:116-147); 12 batches each
    "t_nb2_reuse0": ("t_nb2", 12, "reuse0"),
    "t_nb2_noreuse": ("t_nb2", 12, "noreuse"),
}


def plan_digest(plan):
    h = hashlib.sha256()
    for p in plan:
        h.update(np.asarray(p, dtype=np.int64).tobytes())
        h.update(b"|")
    return h.hexdigest()


def pack(list_of_arrays, dtype=np.int32):
    off = np.zeros(len(list_of_arrays) + 1, dtype=np.int64)
    for i, a in enumerate(list_of_arrays):
        off[i + 1] = off[i] + len(a)
    flat = np.concatenate([np.asarray(a, dtype=dtype) for a in list_of_arrays]) if list_of_arrays \
        else np.zeros(0, dtype=dtype)
    return flat, off


def run_case(case):
    spec_name, n_run = CASES[case][:2]
    mode = CASES[case][2] if len(CASES[case]) > 2 else "budget"
    g = synthetic.make_graph(spec_name)
    spec = g.spec
    data = Data(g.sources, g.destinations, g.timestamps, g.edge_idxs, np.zeros(g.n_edges))
    nf = get_neighbor_finder(data)
    args = argparse.Namespace(bs=spec.bs, n_degree=spec.n_degree, budget=spec.budget, reuse=True,
                              gradient=False, n_nodes=g.n_nodes, n_edges=g.n_edges + 1)
    out = {"graph_sha": g.sha256(), "spec": spec_name, "mode": mode}
    if mode != "budget":
        return run_other_recursion(case, g, data, nf, args, mode, n_run, out)

    # ---- plans for every strategy on the small cases, the spec's own strategy otherwise
    strategies = ["MRD", "LRU", "2Q"] if g.n_edges <= 20000 else [spec.strategy]
    plans = {}
    for st in strategies:
        _seed_numba(0)
        t0 = time.time()
        plans[st] = get_cache_plan(args, data, nf, g.n_nodes, st)
        print(case, st, "plan %.1fs" % (time.time() - t0))
        n_keep = len(plans[st]) if n_run is None else n_run
        flat, off = pack(plans[st][:n_keep])
        out[f"plan_{st}_flat"], out[f"plan_{st}_off"] = flat, off
        out[f"plan_{st}_sha"] = plan_digest(plans[st])
    plan = plans[spec.strategy]

    # ---- model
    torch.use_deterministic_algorithms(True)
    torch.manual_seed(0)
    tgn = TGN(neighbor_finder=nf, node_features=None, edge_features=g.edge_features,
              device=torch.device("cpu"), n_layers=spec.n_layers, n_heads=2, dropout=0.1,
              use_memory=True, node_dimension=172, time_dimension=172, memory_dimension=172,
              embedding_module_type="graph_attention", message_function="identity",
              aggregator_type="last", memory_updater_type="gru", n_neighbors=spec.n_degree,
              args=args)
    sd = {k: torch.from_numpy(v) for k, v in params.random_state_dict(spec.n_layers, seed=0).items()}
    # the time encoder is registered twice (TGN and its embedding module share the object)
    sd["embedding_module.time_encoder.w.weight"] = sd["time_encoder.w.weight"]
    sd["embedding_module.time_encoder.w.bias"] = sd["time_encoder.w.bias"]
    missing = tgn.load_state_dict(sd, strict=True)
    print(case, "state dict loaded", missing)
    tgn.test_mode = False
    tgn.eval()

    # record the uncached sets the reference finds
    u_sets = []
    orig = GraphEmbedding.find_uncached_out_of_batch_neighbors

    def spy(self, source, neighbors, n_layers):
        r = orig(self, source, neighbors, n_layers)
        if n_layers > 1:
            u_sets.append(np.asarray(r, dtype=np.int64).copy())
        return r

    GraphEmbedding.find_uncached_out_of_batch_neighbors = spy

    # record the embeddings the scorer consumes (compute_edge_probabilities calls this method)
    last_emb = {}
    orig_cte = tgn.compute_temporal_embeddings

    def cte_spy(*a, **k):
        r = orig_cte(*a, **k)
        last_emb["v"] = r
        return r

    tgn.compute_temporal_embeddings = cte_spy

    neg_all = synthetic.negative_destinations(g, seed=0)
    nb = g.n_batches if n_run is None else min(n_run, g.n_batches)
    bs = spec.bs
    scores = np.full((nb, 2, bs), np.nan, dtype=np.float32)
    emb_batches = sorted(set([0, nb // 2, nb - 1]))
    emb_rec = {}
    samp_rec = {}
    t0 = time.time()
    with torch.no_grad():
        for b in range(nb):
            s, e = b * bs, min(g.n_edges, (b + 1) * bs)
            src, dst, neg = g.sources[s:e], g.destinations[s:e], neg_all[s:e]
            ts, eidx = g.timestamps[s:e], g.edge_idxs[s:e]
            if b in emb_batches:
                nodes = np.concatenate([src, dst, neg])
                tt = np.concatenate([ts, ts, ts])
                samp_rec[b] = nf.get_temporal_neighbor(nodes, tt, spec.n_degree)
            p, n = tgn.compute_edge_probabilities(src, dst, neg, ts, eidx, spec.n_degree, True,
                                                  False, plan[b])
            if b in emb_batches:
                se, de, ne = last_emb["v"]
                emb_rec[b] = np.stack([se[:32].numpy(), de[:32].numpy(), ne[:32].numpy()])
            scores[b, 0, :e - s] = p.numpy().ravel()
            scores[b, 1, :e - s] = n.numpy().ravel()
    print(case, "eval %.1fs (%d batches)" % (time.time() - t0, nb))
    GraphEmbedding.find_uncached_out_of_batch_neighbors = orig
    out["scores"] = scores
    out["neg"] = neg_all[: nb * bs].astype(np.int32)
    if spec.n_layers > 1:
        out["u_flat"], out["u_off"] = pack(u_sets)
    for b in emb_batches:
        out[f"emb_{b}"] = emb_rec[b]
        nbr, eid, et = samp_rec[b]
        out[f"samp_{b}_nbr"], out[f"samp_{b}_eid"], out[f"samp_{b}_et"] = nbr, eid, et
    out["emb_batches"] = np.asarray(emb_batches)

    # ---- state after the last batch: rows of the nodes touched last
    touched = np.unique(np.concatenate([g.sources[: nb * bs], g.destinations[: nb * bs]]))
    rs = np.random.RandomState(1)
    pick = np.sort(rs.choice(touched, size=min(128, len(touched)), replace=False))
    out["state_nodes"] = pick.astype(np.int32)
    mem = tgn.memory
    out["state_memory"] = mem.memory[pick].numpy()
    out["state_last_update"] = mem.last_update[pick].numpy()
    out["state_messages"] = mem.messages[pick[:32]].numpy()
    out["state_msg_ts"] = mem.timestamps[pick].numpy()
    out["state_flags"] = mem.nodes[pick].astype(np.uint8)
    out["sum_memory"] = np.float64(mem.memory.double().sum().item())
    out["sum_abs_memory"] = np.float64(mem.memory.double().abs().sum().item())
    out["sum_messages"] = np.float64(mem.messages.double().sum().item())
    if spec.n_layers > 1:
        h = tgn.embedding_module.histories[0]
        out["state_history"] = h.emb[pick].numpy()
        out["sum_abs_history"] = np.float64(h.emb.double().abs().sum().item())
        out["cache_flag_nodes"] = np.nonzero(h.cache_flag)[0].astype(np.int32)

    # ---- AP over the batches that ran (evaluation/evaluation.py:39-45)
    from sklearn.metrics import average_precision_score
    aps = []
    for b in range(nb):
        n = min(g.n_edges, (b + 1) * bs) - b * bs
        pred = np.concatenate([scores[b, 0, :n], scores[b, 1, :n]])
        lab = np.concatenate([np.ones(n), np.zeros(n)])
        aps.append(average_precision_score(lab, pred))
    out["ap"] = np.float64(np.mean(aps))
    out["versions"] = np.array([f"numba {numba.__version__}", f"torch {torch.__version__}",
                                f"numpy {np.__version__}"])
    path = os.path.join(HERE, f"{case}.npz")
    np.savez_compressed(path, **out)
    print(case, "->", path, "%.1f KB" % (os.path.getsize(path) / 1024), "AP %.6f" % out["ap"])


def run_other_recursion(case, g, data, nf, args, mode, n_run, out):
    """Scores and state slices of the unlimited-reuse (budget 0) and no-reuse recursions."""
    spec = g.spec
    args.budget = 0
    args.reuse = mode == "reuse0"
    torch.use_deterministic_algorithms(True)
    torch.manual_seed(0)
    tgn = TGN(neighbor_finder=nf, node_features=None, edge_features=g.edge_features,
              device=torch.device("cpu"), n_layers=spec.n_layers, n_heads=2, dropout=0.1,
              use_memory=True, node_dimension=172, time_dimension=172, memory_dimension=172,
              embedding_module_type="graph_attention", message_function="identity",
              aggregator_type="last", memory_updater_type="gru", n_neighbors=spec.n_degree,
              args=args)
    sd = {k: torch.from_numpy(v) for k, v in params.random_state_dict(spec.n_layers, seed=0).items()}
    sd["embedding_module.time_encoder.w.weight"] = sd["time_encoder.w.weight"]
    sd["embedding_module.time_encoder.w.bias"] = sd["time_encoder.w.bias"]
    tgn.load_state_dict(sd, strict=True)
    tgn.test_mode = False
    tgn.eval()
    neg_all = synthetic.negative_destinations(g, seed=0)
    nb, bs = n_run, spec.bs
    scores = np.full((nb, 2, bs), np.nan, dtype=np.float32)
    with torch.no_grad():
        for b in range(nb):
            s, e = b * bs, min(g.n_edges, (b + 1) * bs)
            p, n = tgn.compute_edge_probabilities(g.sources[s:e], g.destinations[s:e], neg_all[s:e],
                                                  g.timestamps[s:e], g.edge_idxs[s:e], spec.n_degree,
                                                  mode == "reuse0", False, None)
            scores[b, 0, :e - s] = p.numpy().ravel()
            scores[b, 1, :e - s] = n.numpy().ravel()
    out["scores"] = scores
    out["neg"] = neg_all[: nb * bs].astype(np.int32)
    touched = np.unique(np.concatenate([g.sources[: nb * bs], g.destinations[: nb * bs]]))
    pick = np.sort(np.random.RandomState(1).choice(touched, size=min(128, len(touched)), replace=False))
    out["state_nodes"] = pick.astype(np.int32)
    out["state_memory"] = tgn.memory.memory[pick].numpy()
    if mode == "reuse0":
        out["state_history"] = tgn.embedding_module.histories[0].emb[pick].numpy()
    out["versions"] = np.array([f"numba {numba.__version__}", f"torch {torch.__version__}",
                                f"numpy {np.__version__}"])
    path = os.path.join(HERE, f"{case}.npz")
    np.savez_compressed(path, **out)
    print(case, "->", path, "%.1f KB" % (os.path.getsize(path) / 1024))


if __name__ == "__main__":
    names = sys.argv[1:] or list(CASES)
    for c in names:
        run_case(c)
