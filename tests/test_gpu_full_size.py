"""Full-size run (the 1.14 M-node configuration) checked through properties that do not need the CPU
oracle: sampled neighbours respect time order and padding, the appended uncached rows are what the
definition says, scores are probabilities, a batch touches only the state rows of its own nodes, and the
same inputs give the same bits twice."""
import numpy as np
import pytest
import torch

from helpers import graph
from test_gpu_model import make_model

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def big():
    g = graph("c5")
    return g, make_model(g)


def test_sampler_properties_at_full_size(big):
    g, tgn = big
    spec = g.spec
    nf = tgn.embedding_module.neighbor_finder
    lo = (g.n_batches // 2) * spec.bs
    src, dst, ts = g.sources[lo:lo + spec.bs], g.destinations[lo:lo + spec.bs], g.timestamps[lo:lo + spec.bs]
    nodes = np.r_[src, dst]
    qts = np.r_[ts, ts]
    nbr, eid, et, dt = (x.cpu().numpy() for x in nf.sample_device(nodes, qts, spec.n_degree, want_delta=True))
    valid = nbr != 0
    # right-aligned: once a slot is valid every later slot is
    assert np.all(valid[:, 1:] | ~valid[:, :-1])
    assert np.all((eid != 0) == valid)
    # non-decreasing along the row (the float32 copies round monotonically)
    assert np.all((np.diff(et, axis=1) >= 0) | ~valid[:, :-1])
    assert np.array_equal(dt, (qts[:, None] - et.astype(np.float64)).astype(np.float32))
    # every sampled edge really joins the query node and its neighbour, at that time
    e = eid[valid].astype(np.int64) - 1
    q = np.repeat(nodes, spec.n_degree).reshape(nbr.shape)[valid]
    other = np.where(g.sources[e] == q, g.destinations[e], g.sources[e])
    assert np.array_equal(other, nbr[valid])
    assert np.array_equal(g.timestamps[e].astype(np.float32), et[valid])
    # strictly earlier than the query (in the stream's own float64 times)
    assert np.all(g.timestamps[e] < qts[:, None].repeat(spec.n_degree, 1)[valid])
    # rows of nodes with at least K earlier interactions are full
    deg_before = np.array([np.searchsorted(nf_ts, t) for nf_ts, t in
                           ((g.timestamps[(g.sources == n) | (g.destinations == n)], t)
                            for n, t in zip(nodes[:20], qts[:20]))])
    assert np.array_equal(valid[:20].sum(1), np.minimum(deg_before, spec.n_degree))


def test_batches_at_full_size(big):
    g, tgn = big
    spec = g.spec
    first = g.n_batches // 2
    rng = np.random.RandomState(1)

    def run(model, n_batches):
        out = []
        for b in range(first, first + n_batches):
            lo = b * spec.bs
            src, dst = g.sources[lo:lo + spec.bs], g.destinations[lo:lo + spec.bs]
            ts, eidx = g.timestamps[lo:lo + spec.bs], g.edge_idxs[lo:lo + spec.bs]
            neg = np.roll(dst, 7)
            plan = np.unique(np.r_[src, dst])[: spec.budget]         # any plan will do: the batch's own nodes
            mem_before = model.memory.memory.clone()
            p, q = model.compute_edge_probabilities(src, dst, neg, ts, eidx, spec.n_degree, True, False, plan)
            n1, n_pos, _ = model.check_status()
            out.append(torch.cat([p, q]).clone())
            # probabilities
            assert torch.isfinite(out[-1]).all() and (out[-1] > 0).all() and (out[-1] < 1).all()
            assert n_pos == len(np.unique(np.r_[src, dst])) and n1 >= 3 * len(src)
            # only the batch's own nodes may change in the memory table
            changed = (model.memory.memory != mem_before).any(dim=1).nonzero().flatten().cpu().numpy()
            assert np.isin(changed, np.r_[src, dst]).all()
            # cache flags = the plan
            h = model.embedding_module.histories[0]
            assert np.array_equal(np.nonzero(h.cache_flag)[0], np.sort(plan))
        return torch.stack(out)

    a = run(tgn, 3)
    fresh = make_model(g)
    b = run(fresh, 3)
    assert torch.equal(a, b)        # same inputs, same state: same bits
    del rng
