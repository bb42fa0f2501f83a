"""Two-GPU parity of the sharded batch path (needs at least two GPUs; skipped otherwise): both ranks
run the whole fixture stream through TGN.compute_edge_probabilities in distributed mode (NCCL) and
must reproduce the reference's scores, agree with each other bit for bit, and end with identical
state tables."""
import os
import socket

import numpy as np
import pytest
import torch

from helpers import batches, golden, graph, max_rel, unpack

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, case, out_dir):
    import torch.distributed as dist
    from test_gpu_model import make_model
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        gold = golden(case)
        g = graph(str(gold["spec"]))
        spec = g.spec
        plan = unpack(gold[f"plan_{spec.strategy}_flat"], gold[f"plan_{spec.strategy}_off"])
        tgn = make_model(g, device=f"cuda:{rank}")
        tgn.set_distributed(rank, world)
        # planned once on rank 0 by the product planner, received by broadcast on the other rank
        import argparse
        from orca_b200.cache import get_cache_plan
        ns = argparse.Namespace(bs=spec.bs, n_degree=spec.n_degree, budget=spec.budget)
        shared = get_cache_plan(ns, g, tgn.embedding_module.neighbor_finder, g.n_nodes, spec.strategy,
                                broadcast_from=0)
        assert len(shared) == len(plan)
        for a, w in zip(shared, plan):
            assert np.array_equal(a, w)
        neg, scores = gold["neg"], gold["scores"]
        got = []
        worst = 0.0
        for b, src, dst, ts, eidx in batches(g, scores.shape[0]):
            n = len(src)
            ng = neg[b * spec.bs: b * spec.bs + n]
            if b == 5:
                # reconfigured in mid-stream: from the split by layer to the split by rows (the first exchange
                # buffers are released after a barrier, the peers' mappings closed, new ones opened)
                tgn.set_distributed(rank, world, split="rows")
            if b == 3:
                # the embedding API advances the state exactly like the scoring API
                s_e, d_e, n_e = tgn.compute_temporal_embeddings(src, dst, ng, ts, eidx, spec.n_degree, True, False,
                                                                plan[b])
                assert s_e.shape == (n, 172) and d_e.shape == (n, 172) and n_e.shape == (n, 172)
                got.append(s_e.cpu().numpy().ravel())
                tgn.check_status()
                continue
            p, q = tgn.compute_edge_probabilities(src, dst, ng, ts, eidx, spec.n_degree, True, False, plan[b])
            tgn.check_status()
            p, q = p.cpu().numpy().ravel(), q.cpu().numpy().ravel()
            got.append(np.r_[p, q])
            worst = max(worst, max_rel(p, scores[b, 0, :n]), max_rel(q, scores[b, 1, :n]))
        assert worst < 1e-3, worst
        np.save(os.path.join(out_dir, f"scores_{rank}.npy"), np.concatenate(got))
        np.save(os.path.join(out_dir, f"memory_{rank}.npy"), tgn.memory.memory.cpu().numpy())
        np.save(os.path.join(out_dir, f"hist_{rank}.npy"), tgn.embedding_module.histories[0].emb.cpu().numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("case", ["t_nb2", "t_lru"])
def test_two_gpus_match_reference_and_each_other(case, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port(), case, str(tmp_path)), nprocs=2, join=True)
    for name in ("scores", "memory", "hist"):
        a, b = np.load(tmp_path / f"{name}_0.npy"), np.load(tmp_path / f"{name}_1.npy")
        assert np.array_equal(a, b), name
