"""Seeded synthetic temporal graphs that stand in for the datasets the reference is run on.

The real interaction logs (JODIE Wikipedia/Reddit/MOOC, SNAP AskUbuntu/SuperUser/Wiki-Talk) are
not shipped with the reference, so every test and benchmark here draws a graph with the same
node/edge counts and id conventions instead.  The id conventions follow the reference's
pre-processing (utils/preprocess_data.py:41-63, 78-79): node 0 and edge 0 are padding, sources are
1..NS, bipartite destinations NS+1..NS+ND, edge ids 1..E, edge-feature row 0 is all zeros and
``n_nodes = max id + 1``.

Draw order from one ``numpy.random.RandomState(seed)``: sources, destinations, timestamps,
features.  ``Zipf(s)`` over m ids means p_i proportional to (i+1)^-s, id = first_id + i.
"""
from __future__ import annotations

import dataclasses
import hashlib

import numpy as np

FEAT_DIM = 172


@dataclasses.dataclass
class GraphSpec:
    """Shape and run parameters of one synthetic workload."""
    name: str
    n_src: int            # bipartite: number of sources; non-bipartite: number of nodes
    n_dst: int            # bipartite: number of destinations; 0 for non-bipartite graphs
    n_edges: int
    zipf_src: float
    zipf_dst: float
    ts_law: str           # "uniform" | "exp" | "bursty"
    ts_span: float
    dst_law: str = "zipf"  # "zipf" | "prefatt"
    random_feats: bool = True
    n_layers: int = 2
    n_degree: int = 10
    bs: int = 200
    budget: int = 1000
    strategy: str = "MRD"

    @property
    def bipartite(self) -> bool:
        return self.n_dst > 0

    @property
    def n_nodes(self) -> int:
        return self.n_src + self.n_dst + 1


# The five workloads the headline metric is defined on (index = position in the config list),
# plus small variants used by the parity tests.
SPECS = {
    "c1": GraphSpec("c1", 1000, 500, 20000, 1.1, 1.1, "uniform", 1e5, n_layers=1),
    "c2": GraphSpec("c2", 8227, 1000, 157474, 1.2, 1.5, "exp", 2.7e6),
    "c3": GraphSpec("c3", 10000, 984, 672447, 1.3, 1.3, "exp", 2.7e6, n_degree=20, bs=600,
                    budget=2000, strategy="LRU"),
    "c4": GraphSpec("c4", 194085, 0, 1443339, 1.5, 1.5, "bursty", 2.3e8, random_feats=False,
                    bs=1000, budget=1000, strategy="2Q"),
    "c5": GraphSpec("c5", 1140149, 0, 7833140, 1.6, 0.0, "exp", 2.0e8, dst_law="prefatt",
                    random_feats=False, bs=2000, budget=10000, strategy="MRD"),
    # small parity cases
    "t_bip2": GraphSpec("t_bip2", 600, 200, 6000, 1.1, 1.3, "exp", 1e5, bs=200, budget=150),
    "t_nb2": GraphSpec("t_nb2", 1500, 0, 6000, 1.3, 1.3, "bursty", 1e6, bs=200, budget=100),
    "t_lru": GraphSpec("t_lru", 700, 150, 6000, 1.1, 1.2, "exp", 1e5, n_degree=20, bs=300,
                       budget=60, strategy="LRU"),
    "t_2q": GraphSpec("t_2q", 1500, 0, 6000, 1.2, 1.2, "exp", 1e6, random_feats=False, bs=200,
                      budget=80, strategy="2Q"),
}


@dataclasses.dataclass
class Graph:
    spec: GraphSpec
    sources: np.ndarray       # int64 [E]
    destinations: np.ndarray  # int64 [E]
    timestamps: np.ndarray    # float64 [E], non-decreasing
    edge_idxs: np.ndarray     # int64 [E] = 1..E
    edge_features: np.ndarray  # float32 [E+1, 172], row 0 zero

    @property
    def n_nodes(self) -> int:
        return self.spec.n_nodes

    @property
    def n_edges(self) -> int:
        return len(self.sources)

    @property
    def n_batches(self) -> int:
        return (self.n_edges + self.spec.bs - 1) // self.spec.bs

    def sha256(self) -> str:
        h = hashlib.sha256()
        for a in (self.sources, self.destinations, self.timestamps, self.edge_idxs):
            h.update(np.ascontiguousarray(a).tobytes())
        h.update(np.ascontiguousarray(self.edge_features[: min(1024, len(self.edge_features))]).tobytes())
        return h.hexdigest()


def _zipf(rng, m, s, size):
    p = 1.0 / np.arange(1, m + 1, dtype=np.float64) ** s
    p /= p.sum()
    return rng.choice(m, size=size, p=p).astype(np.int64)


def _resolve_copies(base, ptr):
    """dst[i] = dst[ptr[i]] where ptr[i] >= 0, else base[i]; ptr[i] < i.  Pointer doubling."""
    val = base.copy()
    ptr = ptr.copy()
    todo = np.nonzero(ptr >= 0)[0]
    while len(todo):
        p = ptr[todo]
        done = ptr[p] < 0
        val[todo[done]] = val[p[done]]
        ptr[todo[done]] = -1
        ptr[todo[~done]] = ptr[p[~done]]
        todo = todo[~done]
    return val


def make_graph(spec: GraphSpec | str, seed: int = 0, n_edges: int | None = None) -> Graph:
    """Draw the graph for ``spec`` (a name from SPECS or a GraphSpec).

    ``n_edges`` truncates the edge stream (the first edges of the same draw are NOT guaranteed;
    a different E changes the draw), and is meant for quick tests only.
    """
    if isinstance(spec, str):
        spec = SPECS[spec]
    if n_edges is not None:
        spec = dataclasses.replace(spec, n_edges=n_edges)
    rng = np.random.RandomState(seed)
    E = spec.n_edges
    if spec.bipartite:
        src = 1 + _zipf(rng, spec.n_src, spec.zipf_src, E)
        dst = 1 + spec.n_src + _zipf(rng, spec.n_dst, spec.zipf_dst, E)
    else:
        n = spec.n_src
        src = 1 + _zipf(rng, n, spec.zipf_src, E)
        if spec.dst_law == "zipf":
            dst = 1 + _zipf(rng, n, spec.zipf_dst, E)
        else:
            # preferential attachment: with prob 0.8 copy a uniformly chosen endpoint of a
            # uniformly chosen earlier edge, else a uniform node
            copy = rng.random_sample(E) < 0.8
            j = np.floor(rng.random_sample(E) * np.arange(E)).astype(np.int64)
            which = rng.randint(0, 2, E)
            unif = 1 + rng.randint(0, n, E).astype(np.int64)
            copy[0] = False
            base = np.where(copy & (which == 0), src[j], unif)
            ptr = np.where(copy & (which == 1), j, -1)
            dst = _resolve_copies(base, ptr)
        while True:  # no self loops
            bad = np.nonzero(dst == src)[0]
            if len(bad) == 0:
                break
            dst[bad] = 1 + rng.randint(0, n, len(bad))
    if spec.ts_law == "uniform":
        ts = np.sort(rng.uniform(0, spec.ts_span, E))
    elif spec.ts_law == "exp":
        ts = np.cumsum(rng.exponential(spec.ts_span / E, E))
    elif spec.ts_law == "bursty":
        scale = np.where((np.arange(E) // 10000) % 2 == 0, 0.1, 1.9) * (spec.ts_span / E)
        ts = np.cumsum(rng.exponential(1.0, E) * scale)
    else:
        raise ValueError(spec.ts_law)
    if spec.random_feats:
        feats = np.empty((E + 1, FEAT_DIM), dtype=np.float32)
        feats[0] = 0
        # drawn in blocks so that the fp64 temporaries stay small
        blk = 1 << 16
        for s in range(0, E, blk):
            e = min(E, s + blk)
            feats[1 + s:1 + e] = rng.randn(e - s, FEAT_DIM).astype(np.float32)
    else:
        feats = np.zeros((E + 1, FEAT_DIM), dtype=np.float32)
    return Graph(spec, src, dst, ts.astype(np.float64), np.arange(1, E + 1, dtype=np.int64), feats)


def negative_destinations(graph: Graph, seed: int = 0) -> np.ndarray:
    """One uniform negative destination per positive edge, batch by batch, drawn the way the
    reference's eval loop draws them (utils/util.py:68-87 with evaluation/evaluation.py:32): per
    batch the sampler draws `size` source indices first (discarded) and then `size` destination
    indices, both from one ``RandomState(seed)`` over the unique sorted id lists."""
    rs = np.random.RandomState(seed)
    src_list = np.unique(graph.sources)
    dst_list = np.unique(graph.destinations)
    out = np.empty(graph.n_edges, dtype=np.int64)
    bs = graph.spec.bs
    for s in range(0, graph.n_edges, bs):
        e = min(graph.n_edges, s + bs)
        rs.randint(0, len(src_list), e - s)
        out[s:e] = dst_list[rs.randint(0, len(dst_list), e - s)]
    return out
