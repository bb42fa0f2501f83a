"""Kernel-level parity on the GPU: every entry point of the C ABI against the CPU oracle on the
same seeded inputs.  Integer outputs must be identical; floating-point outputs within the stated
tolerance (fp32 kernels: 1e-4 relative to a 0.05 floor)."""
import numpy as np
import pytest
import torch

from helpers import graph, max_rel, state_dict
from oracle import tgn_oracle

pytestmark = pytest.mark.gpu

D = 172
TOL = 1e-4       # fp32 kernels
TOL_TC = 1e-3    # tensor-core projections (split TF32, truncating fp32 accumulation in tensor memory)


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


def _i32(a, dev):
    return torch.as_tensor(np.asarray(a), dtype=torch.int32).to(dev)


def _finder(g):
    from orca_b200.neighbor_finder import get_neighbor_finder
    return get_neighbor_finder(g)


def _adj(g):
    return tgn_oracle.Adjacency(g.sources, g.destinations, g.edge_idxs, g.timestamps, g.n_nodes)


# ------------------------------------------------------------------------------- sampling
@pytest.mark.parametrize("spec,k", [("t_nb2", 10), ("t_bip2", 10), ("t_lru", 20), ("c1", 10), ("t_nb2", 1),
                                    ("t_nb2", 32), ("t_nb2", 16), ("t_nb2", 17)])
def test_sampler_bit_exact(spec, k):
    g = graph(spec)
    nf, adj = _finder(g), _adj(g)
    rs = np.random.RandomState(7)
    q = 3000
    nodes = rs.randint(0, g.n_nodes, q)               # includes node 0 and nodes without edges
    ts = rs.uniform(-1.0, g.timestamps[-1] * 1.1, q)
    # queries exactly at edge times exercise the strictly-before rule
    pick = rs.randint(0, g.n_edges, q // 2)
    nodes[: q // 2] = g.sources[pick]
    ts[: q // 2] = g.timestamps[pick]
    want = tgn_oracle.sample_neighbors(adj, nodes, ts, k)
    got = nf.get_temporal_neighbor(nodes, ts, k)
    for a, w in zip(got, want):
        assert a.dtype == w.dtype and a.shape == w.shape
        assert a.tobytes() == w.tobytes()
    # fused time differences
    _, _, et, dt = nf.sample_device(nodes, ts, k, want_delta=True)
    want_dt = (ts[:, None] - want[2]).astype(np.float32)
    assert dt.cpu().numpy().tobytes() == want_dt.tobytes()


def test_sampler_duplicate_timestamps_and_hub():
    # one hub with 200k interactions at few distinct times: long equal runs inside the search
    rs = np.random.RandomState(3)
    E = 200000
    src = np.ones(E, dtype=np.int64)
    dst = rs.randint(2, 50, E).astype(np.int64)
    ts = np.sort(rs.randint(0, 300, E)).astype(np.float64)

    class Data:
        sources, destinations, timestamps, edge_idxs = src, dst, ts, np.arange(1, E + 1)

    from orca_b200.neighbor_finder import get_neighbor_finder
    nf = get_neighbor_finder(Data)
    adj = tgn_oracle.Adjacency(src, dst, Data.edge_idxs, ts, 50)
    nodes = np.concatenate([np.ones(400, dtype=np.int64), rs.randint(0, 50, 400)])
    qts = np.concatenate([rs.randint(-1, 302, 400).astype(np.float64), rs.uniform(0, 300, 400)])
    want = tgn_oracle.sample_neighbors(adj, nodes, qts, 10)
    got = nf.get_temporal_neighbor(nodes, qts, 10)
    for a, w in zip(got, want):
        assert a.tobytes() == w.tobytes()
    a = nf.find_before(1, 150.0)
    i = np.searchsorted(ts, 150.0)
    assert len(a[0]) == i and np.array_equal(a[2], ts[:i])


def test_sampler_empty_inputs():
    g = graph("t_nb2")
    nf = _finder(g)
    nbr, eid, et = nf.get_temporal_neighbor(np.zeros(0, dtype=np.int64), np.zeros(0), 10)
    assert nbr.shape == (0, 10) and eid.shape == (0, 10) and et.shape == (0, 10)


# ------------------------------------------------------------------------------- uncached set
@pytest.mark.parametrize("n_nodes", [1501, 70000, 1700000])
def test_find_uncached(dev, n_nodes):
    from orca_b200 import _lib
    L = _lib.lib()
    rs = np.random.RandomState(n_nodes)
    for trial in range(3):
        nq, k = 600, 10
        nbr = rs.randint(1, min(n_nodes, 5000), size=(nq, k)).astype(np.int32)
        if trial != 1:
            nbr[rs.rand(nq, k) < 0.2] = 0           # padding present -> node 0 heads the list
        src = rs.randint(1, min(n_nodes, 5000), nq).astype(np.int32)
        ts = rs.uniform(0, 1e5, nq)
        flag = (rs.rand(n_nodes) < 0.3).astype(np.uint8)
        flag[0] = 0
        want = tgn_oracle.find_uncached(src, nbr, flag.astype(np.float64))
        u_cap = nq * k
        nodes_io = torch.zeros(nq + u_cap, dtype=torch.int32, device=dev)
        nodes_io[:nq] = _i32(src, dev)
        ts_io = torch.zeros(nq + u_cap, dtype=torch.float64, device=dev)
        ts_io[:nq] = torch.as_tensor(ts).to(dev)
        n_total = torch.zeros(1, dtype=torch.int32, device=dev)
        status = torch.zeros(4, dtype=torch.int32, device=dev)
        scratch = torch.zeros(max(int(L.orca_find_uncached_scratch_bytes(n_nodes)), 16), dtype=torch.uint8, device=dev)
        d_nbr, d_flag = _i32(nbr, dev), torch.as_tensor(flag).to(dev)   # keep the inputs alive
        _lib.check(L.orca_find_uncached(d_nbr.data_ptr(), nq, k, d_flag.data_ptr(),
                                        n_nodes, nodes_io.data_ptr(), ts_io.data_ptr(), u_cap, n_total.data_ptr(),
                                        scratch.data_ptr(), status.data_ptr(), _lib.stream_ptr(dev)))
        _lib.check(L.orca_read_status(None, status.data_ptr(), None, _lib.stream_ptr(dev)))
        n = int(n_total.item())
        assert n == nq + len(want)
        assert np.array_equal(nodes_io[nq:n].cpu().numpy(), want)
        assert np.all(ts_io[nq:n].cpu().numpy() == ts.max())
        assert np.array_equal(nodes_io[:nq].cpu().numpy(), src)


def test_find_uncached_capacity_is_reported(dev):
    from orca_b200 import _lib
    L = _lib.lib()
    nbr = np.arange(1, 101, dtype=np.int32).reshape(10, 10)
    src = np.full(10, 500, dtype=np.int32)
    nodes_io = torch.zeros(10 + 5, dtype=torch.int32, device=dev)
    nodes_io[:10] = _i32(src, dev)
    ts_io = torch.zeros(15, dtype=torch.float64, device=dev)
    n_total = torch.zeros(1, dtype=torch.int32, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    flag = torch.zeros(1000, dtype=torch.uint8, device=dev)
    scratch = torch.zeros(16, dtype=torch.uint8, device=dev)
    d_nbr = _i32(nbr, dev)
    _lib.check(L.orca_find_uncached(d_nbr.data_ptr(), 10, 10, flag.data_ptr(), 1000, nodes_io.data_ptr(),
                                    ts_io.data_ptr(), 5, n_total.data_ptr(), scratch.data_ptr(), status.data_ptr(),
                                    _lib.stream_ptr(dev)))
    with pytest.raises(_lib.OrcaError) as e:
        _lib.check(L.orca_read_status(None, status.data_ptr(), None, _lib.stream_ptr(dev)))
    assert e.value.code == 4
    assert int(n_total.item()) == 15
    assert np.array_equal(nodes_io[10:].cpu().numpy(), np.arange(2, 7))   # first entry (1) is dropped


# ------------------------------------------------------------------------------- last occurrence
def test_last_occurrence(dev):
    from orca_b200 import _lib
    L = _lib.lib()
    rs = np.random.RandomState(5)
    n_nodes = 300
    last_pos = torch.zeros(n_nodes, dtype=torch.int64, device=dev)
    base = 1
    for n in (1, 77, 1024, 1025, 4000):
        ids = rs.randint(1, n_nodes, n).astype(np.int32)
        uniq, pos = tgn_oracle.last_occurrence(ids)
        is_last = torch.zeros(n, dtype=torch.uint8, device=dev)
        compact = torch.zeros(n, dtype=torch.int32, device=dev)
        n_c = torch.zeros(1, dtype=torch.int32, device=dev)
        d_ids = _i32(ids, dev)
        _lib.check(L.orca_last_occurrence(d_ids.data_ptr(), n, None, n_nodes, last_pos.data_ptr(), base,
                                          is_last.data_ptr(), compact.data_ptr(), n_c.data_ptr(),
                                          _lib.stream_ptr(dev)))
        base += n
        want_flag = np.zeros(n, dtype=np.uint8)
        want_flag[pos] = 1
        assert np.array_equal(is_last.cpu().numpy(), want_flag)
        assert int(n_c.item()) == len(uniq)
        assert np.array_equal(compact[:len(uniq)].cpu().numpy(), np.sort(pos))


# ------------------------------------------------------------------------------- attention layer
def _attention_case(seed, n, k, n_tab=400):
    rs = np.random.RandomState(seed)
    table = rs.randn(n_tab, D).astype(np.float32)
    table[0] = 0
    etab = rs.randn(n_tab * 2, D).astype(np.float32)
    etab[0] = 0
    src_ids = rs.randint(1, n_tab, n).astype(np.int32)
    nbr = rs.randint(1, n_tab, size=(n, k)).astype(np.int32)
    eid = rs.randint(1, n_tab * 2, size=(n, k)).astype(np.int32)
    dt = np.abs(rs.randn(n, k) * 10 ** rs.uniform(0, 8, size=(n, k))).astype(np.float32)
    pad = rs.rand(n, k) < 0.3
    pad[0] = True
    if n > 2:
        pad[1] = False
        pad[2, :-1] = True
    nbr[pad] = 0
    eid[pad] = 0
    return table, etab, src_ids, nbr, eid, dt


@pytest.fixture
def fp32_projections():
    """Runs the projections on the plain fp32 SIMT tiles (the debug reference of the tensor-core path)."""
    from orca_b200 import _lib
    _lib.check(_lib.lib().orca_ctx_set(None, _lib.OPT_PROJECTION_MODE, 1))
    yield
    _lib.check(_lib.lib().orca_ctx_set(None, _lib.OPT_PROJECTION_MODE, 0))


def test_attention_layer_fp32_projections(dev, fp32_projections, capsys):
    test_attention_layer(dev, 10, 333, 0)
    test_attention_layer(dev, 20, 70, 1)
    for line in capsys.readouterr().out.splitlines():
        assert float(line.split()[-1]) < TOL


@pytest.mark.parametrize("k,n", [(10, 333), (20, 70), (1, 50), (32, 40), (10, 1), (10, 128), (10, 129)])
@pytest.mark.parametrize("layer", [0, 1])
def test_attention_layer(dev, k, n, layer):
    from orca_b200 import _lib, weights
    L = _lib.lib()
    sd = state_dict(2)
    p = {kk: torch.as_tensor(v) for kk, v in sd.items()}
    table, etab, src_ids, nbr, eid, dt = _attention_case(k * 100 + n, n, k)
    want = tgn_oracle.attention_layer(p, layer, torch.as_tensor(table[src_ids]), torch.as_tensor(table[nbr]),
                                      torch.as_tensor(etab[eid]), torch.as_tensor(dt), nbr).numpy()
    w = {kk: torch.from_numpy(v).to(dev) for kk, v in weights.prepare_attention(sd, layer).items()}
    ws = _lib.attn_struct(w)
    tw = torch.from_numpy(weights.prepare_time(sd)).to(dev)
    cap = n + 13                                       # capacity larger than the device-side row count
    n_dev = torch.tensor([n], dtype=torch.int32, device=dev)
    t_tab, t_etab = torch.from_numpy(table).to(dev), torch.from_numpy(etab).to(dev)
    pad_rows = lambda a: np.concatenate([a, np.zeros((cap - n,) + a.shape[1:], a.dtype)])
    d_src, d_nbr, d_eid = _i32(pad_rows(src_ids), dev), _i32(pad_rows(nbr), dev), _i32(pad_rows(eid), dev)
    d_dt = torch.from_numpy(pad_rows(dt)).to(dev)
    qt = torch.zeros(cap, 1056, device=dev)
    hidden = torch.zeros(cap, D, device=dev)
    ctx = torch.full((cap, 1032), float("nan"), device=dev)
    valid = torch.full((cap,), 7, dtype=torch.uint8, device=dev)
    out = torch.zeros(cap, D, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    s = _lib.stream_ptr(dev)
    _lib.check(L.orca_ctx_set_status_word(None, status.data_ptr()))
    _lib.check(L.orca_attn_query(ws, t_tab.data_ptr(), d_src.data_ptr(), cap, n_dev.data_ptr(), qt.data_ptr(), s))
    _lib.check(L.orca_attn_gather(qt.data_ptr(), t_tab.data_ptr(), t_etab.data_ptr(), tw.data_ptr(), d_nbr.data_ptr(),
                                  d_eid.data_ptr(), d_dt.data_ptr(), k, cap, n_dev.data_ptr(), ctx.data_ptr(),
                                  valid.data_ptr(), status.data_ptr(), s))
    push_table = torch.zeros_like(t_tab)
    win = torch.ones(cap, dtype=torch.uint8, device=dev)
    win[5] = 0
    _lib.check(L.orca_attn_output(ws, ctx.data_ptr(), valid.data_ptr(), t_tab.data_ptr(), d_src.data_ptr(), cap,
                                  n_dev.data_ptr(), out.data_ptr(), push_table.data_ptr(), d_src.data_ptr(),
                                  win.data_ptr(), hidden.data_ptr(), s))
    _lib.check(L.orca_read_status(None, status.data_ptr(), None, s))
    _lib.check(L.orca_ctx_set_status_word(None, None))
    got = out[:n].cpu().numpy()
    err = max_rel(got, want, floor=0.05)
    print(f"attention layer k={k} n={n} layer={layer}: max rel err {err:.2e}")
    assert err < TOL_TC
    v = valid.cpu().numpy()
    assert np.array_equal(v[:n], (~(nbr == 0).all(axis=1)).astype(np.uint8))
    assert np.all(v[n:] == 7) and torch.all(out[n:] == 0)      # rows beyond the device count untouched
    # pushed rows: every row but #5 reached the table (duplicates: some occurrence's value)
    pt = push_table.cpu().numpy()
    for r in (0, 1, 2, 17):
        if r < n and (src_ids[:n] == src_ids[r]).sum() == 1 and r != 5:
            assert np.array_equal(pt[src_ids[r]], got[r])


# ------------------------------------------------------------------------------- history
def test_history_push_pull_flags(dev):
    from orca_b200.history import History
    rs = np.random.RandomState(11)
    n = 500
    h = History(n, D, dev, history_budget=50)
    ids = rs.randint(1, n, 300)
    x = torch.from_numpy(rs.randn(300, D).astype(np.float32)).to(dev)
    h.push(x, ids)
    uniq, pos = tgn_oracle.last_occurrence(ids)
    want = np.zeros((n, D), dtype=np.float32)
    want[uniq] = x.cpu().numpy()[pos]
    assert np.array_equal(h.emb.cpu().numpy(), want)
    pull_ids = rs.randint(0, n, 777)
    assert np.array_equal(h.pull(torch.as_tensor(pull_ids).to(dev)).cpu().numpy(), want[pull_ids])
    # flags: plan replaces plan; plan-less accumulates
    h.update_flag(np.array([3, 4, 5]), None)
    h.update_flag(np.array([5, 9]), None)
    assert np.array_equal(np.nonzero(h.cache_flag)[0], [5, 9])
    h.update_flag(None, np.array([1, 2]))
    assert np.array_equal(np.nonzero(h.cache_flag)[0], [1, 2, 5, 9])
    h.update_flag(np.array([7]), None)
    assert np.array_equal(np.nonzero(h.cache_flag)[0], [7])
    assert h.cache_flag.dtype == np.float64


# ------------------------------------------------------------------------------- scorer, GRU, messages
def test_score(dev):
    from orca_b200 import _lib, weights
    L = _lib.lib()
    sd = state_dict(1)
    p = {kk: torch.as_tensor(v) for kk, v in sd.items()}
    rs = np.random.RandomState(2)
    for b in (1, 37, 200, 1000):
        emb = rs.randn(3 * b, D).astype(np.float32)
        s, d, n = (torch.as_tensor(emb[i * b:(i + 1) * b]) for i in range(3))
        want = torch.sigmoid(tgn_oracle.affinity(p, torch.cat([s, s]), torch.cat([d, n]))).numpy().ravel()
        w = weights.prepare_score(sd)
        t = {kk: torch.from_numpy(v).to(dev) for kk, v in w.items() if kk != "b2"}
        ws = _lib.ScoreWeights(t["W1t"].data_ptr(), t["b1"].data_ptr(), t["w2"].data_ptr(), w["b2"],
                               t["W1t_tc"].data_ptr())
        prob = torch.zeros(2 * b, device=dev)
        d_emb = torch.from_numpy(emb).to(dev)
        _lib.check(L.orca_score(ws, d_emb.data_ptr(), b, prob.data_ptr(), _lib.stream_ptr(dev)))
        assert max_rel(prob.cpu().numpy(), want, floor=0.05) < TOL_TC


def test_message_store_and_gru(dev):
    from orca_b200 import _lib, weights
    from orca_b200.memory import GRUMemoryUpdater, Memory
    L = _lib.lib()
    sd = state_dict(1)
    rs = np.random.RandomState(4)
    n_nodes, n_e, b = 300, 900, 150
    efeat = rs.randn(n_e, D).astype(np.float32)

    # oracle side
    orc = tgn_oracle.OracleTGN(None, efeat, sd, n_nodes, n_layers=1)
    orc.memory = torch.from_numpy(rs.randn(n_nodes, D).astype(np.float32))
    orc.last_update = torch.from_numpy(rs.uniform(0, 100, n_nodes).astype(np.float32))
    mem = Memory(n_nodes, D, 4 * D, 4 * D, device=dev)
    mem.memory.copy_(orc.memory)
    mem.last_update.copy_(orc.last_update)
    upd = GRUMemoryUpdater(4 * D, D, dev).to(dev)
    upd.memory_updater.load_state_dict({k.split(".")[-1]: torch.as_tensor(v) for k, v in sd.items()
                                        if k.startswith("memory_updater.memory_updater.")})

    src = rs.randint(1, 60, b)              # non-bipartite and repetitive: a node is often both roles
    dst = rs.randint(1, 60, b)
    ts = np.sort(rs.uniform(100, 5e6, b))
    eidx = rs.randint(1, n_e, b)
    cat_src, cat_dst = np.concatenate([src, dst]), np.concatenate([dst, src])
    uniq = orc.store_messages(cat_src, cat_dst, np.concatenate([ts, ts]), np.concatenate([eidx, eidx]))

    s = _lib.stream_ptr(dev)
    d_cs, d_cd = _i32(cat_src, dev), _i32(cat_dst, dev)
    last_pos = torch.zeros(n_nodes, dtype=torch.int64, device=dev)
    is_last = torch.zeros(2 * b, dtype=torch.uint8, device=dev)
    win_pos = torch.zeros(2 * b, dtype=torch.int32, device=dev)
    n_win = torch.zeros(1, dtype=torch.int32, device=dev)
    win_nodes = torch.zeros(2 * b, dtype=torch.int32, device=dev)
    _lib.check(L.orca_last_occurrence(d_cs.data_ptr(), 2 * b, None, n_nodes, last_pos.data_ptr(), 1, is_last.data_ptr(),
                                      win_pos.data_ptr(), n_win.data_ptr(), s))
    tw = torch.from_numpy(weights.prepare_time(sd)).to(dev)
    d_ef = torch.from_numpy(efeat).to(dev)
    d_ts, d_eidx = torch.as_tensor(ts).to(dev), _i32(eidx, dev)
    _lib.check(L.orca_message_store(mem.c_struct(), d_ef.data_ptr(), tw.data_ptr(), d_cs.data_ptr(), d_cd.data_ptr(),
                                    d_ts.data_ptr(), d_eidx.data_ptr(), b,
                                    win_pos.data_ptr(), 2 * b, n_win.data_ptr(), win_nodes.data_ptr(), s))
    assert int(n_win.item()) == len(uniq)
    assert np.array_equal(np.sort(win_nodes[:len(uniq)].cpu().numpy()), uniq)
    assert np.array_equal(mem.nodes, orc.msg_flag)
    assert np.array_equal(mem.timestamps.cpu().numpy(), orc.msg_ts.numpy())
    got, want = mem.messages.cpu().numpy(), orc.messages.numpy()
    assert np.array_equal(got[:, :3 * D], want[:, :3 * D])            # gathered parts are copies
    assert max_rel(got[:, 3 * D:], want[:, 3 * D:], floor=0.05) < TOL   # cos of the same fp32 argument

    # GRU over the unique positives, flags survive update_memory and are cleared by the caller
    positives = np.unique(cat_src)
    orc.update_memory(positives)
    upd.update_memory(mem, positives)
    assert max_rel(mem.memory.cpu().numpy(), orc.memory.numpy(), floor=0.05) < TOL_TC
    assert np.array_equal(mem.last_update.cpu().numpy(), orc.last_update.numpy())
    assert mem.nodes.sum() == len(uniq)
    # flush path: every flagged node, flags cleared afterwards
    orc.flush_pending()
    upd.update_memory_in_test(mem)
    assert max_rel(mem.memory.cpu().numpy(), orc.memory.numpy(), floor=0.05) < TOL_TC
    assert mem.nodes.sum() == 0


@pytest.mark.parametrize("n_nodes", [1501, 70000, 1700000])
def test_find_uncached_marked_by_sampler(dev, n_nodes):
    """The two-kernel form: the sampling launch marks the candidates, a light single block finishes."""
    from orca_b200 import _lib
    from orca_b200.neighbor_finder import get_neighbor_finder
    L = _lib.lib()
    rs = np.random.RandomState(n_nodes + 1)
    E = 20000
    hi = min(n_nodes, 4000)

    class Data:
        sources, destinations = rs.randint(1, hi, E).astype(np.int64), rs.randint(1, hi, E).astype(np.int64)
        timestamps, edge_idxs = np.sort(rs.uniform(0, 1e5, E)), np.arange(1, E + 1)

    nf = get_neighbor_finder(Data, max_node_idx=n_nodes - 1)
    adj = tgn_oracle.Adjacency(Data.sources, Data.destinations, Data.edge_idxs, Data.timestamps, n_nodes)
    bitmap = torch.zeros((n_nodes + 31) // 32, dtype=torch.int32, device=dev)
    for trial in range(3):
        nq, k = 600, 10
        src = rs.randint(1, hi, nq).astype(np.int32)
        ts = rs.uniform(0, 1.2e5, nq) if trial else np.full(nq, 2e5)     # trial 0: no padded slot at all? mostly
        flag = (rs.rand(n_nodes) < 0.3).astype(np.uint8)
        flag[0] = 0
        nbr_want, _, _ = tgn_oracle.sample_neighbors(adj, src, ts, k)
        want = tgn_oracle.find_uncached(src, nbr_want, flag.astype(np.float64))
        u_cap = nq * k
        nodes_io = torch.zeros(nq + u_cap, dtype=torch.int32, device=dev)
        nodes_io[:nq] = _i32(src, dev)
        ts_io = torch.zeros(nq + u_cap, dtype=torch.float64, device=dev)
        ts_io[:nq] = torch.as_tensor(ts).to(dev)
        nbr = torch.zeros(nq, k, dtype=torch.int32, device=dev)
        eid = torch.zeros(nq, k, dtype=torch.int32, device=dev)
        n_total = torch.zeros(1, dtype=torch.int32, device=dev)
        status = torch.zeros(4, dtype=torch.int32, device=dev)
        d_flag = torch.as_tensor(flag).to(dev)
        s = _lib.stream_ptr(dev)
        _lib.check(L.orca_sample_topk_mark(nf.indptr.data_ptr(), nf.adj_nbr.data_ptr(), nf.adj_eid.data_ptr(),
                                           nf.adj_ts.data_ptr(), n_nodes, nodes_io.data_ptr(), ts_io.data_ptr(), nq,
                                           None, k, nbr.data_ptr(), eid.data_ptr(), None, None, status.data_ptr(),
                                           d_flag.data_ptr(), bitmap.data_ptr(), s))
        _lib.check(L.orca_find_uncached_marked(bitmap.data_ptr(), nq, n_nodes, nodes_io.data_ptr(), ts_io.data_ptr(),
                                               u_cap, n_total.data_ptr(), status.data_ptr(), s))
        _lib.check(L.orca_read_status(None, status.data_ptr(), None, s))
        n = int(n_total.item())
        assert np.array_equal(nbr.cpu().numpy(), nbr_want)
        assert n == nq + len(want)
        assert np.array_equal(nodes_io[nq:n].cpu().numpy(), want)
        assert np.all(ts_io[nq:n].cpu().numpy() == ts.max())
        assert not bitmap.any()            # clean for the next batch
