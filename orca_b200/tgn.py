"""``TGN`` with the constructor, methods and state-dict names of the reference's model
(model/tgn_model.py:13-195), running the per-batch temporal-embedding path on the GPU through the
C ABI of liborca_b200.so.

The torch modules below (``nn.MultiheadAttention``, ``nn.GRUCell``, ``nn.Linear`` ...) are parameter
containers only: they give ``state_dict()`` / ``load_state_dict()`` the reference's names, their
``forward`` is never called.  The kernels read re-associated copies of the parameters
(orca_b200/weights.py) that are rebuilt whenever the parameters change.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch
from torch import nn

from . import _lib, shard, weights
from .history import History
from .memory import Memory, get_memory_updater

# recursion modes of the fused batch entry point (ORCA_MODE_* of the C header)
MODE_BUDGET, MODE_REUSE_ALL, MODE_NO_REUSE = 0, 1, 2


class MergeLayer(nn.Module):
    """utils/util.py:12-24 (parameter container; used as the merger and as the link scorer)."""

    def __init__(self, dim1, dim2, dim3, dim4):
        super().__init__()
        self.fc1 = nn.Linear(dim1 + dim2, dim3)
        self.fc2 = nn.Linear(dim3, dim4)
        self.act = nn.ReLU()
        nn.init.xavier_normal_(self.fc1.weight)
        nn.init.xavier_normal_(self.fc2.weight)


class TimeEncode(nn.Module):
    """model/time_encoding.py:6-28: frozen frequencies 10^(-9 i/(d-1)), zero bias."""

    def __init__(self, dimension):
        super().__init__()
        self.dimension = dimension
        self.w = nn.Linear(1, dimension)
        w = (1 / 10 ** np.linspace(0, 9, dimension, dtype=np.float32)).reshape(dimension, -1)
        self.w.weight = nn.Parameter(torch.from_numpy(w), requires_grad=False)
        self.w.bias = nn.Parameter(torch.zeros(dimension), requires_grad=False)


class TemporalAttentionLayer(nn.Module):
    """model/temporal_attention.py:6-22 (parameter container)."""

    def __init__(self, n_node_features, n_neighbors_features, n_edge_features, time_dim, output_dimension,
                 n_head=2, dropout=0.1):
        super().__init__()
        self.n_head = n_head
        self.feat_dim = n_node_features
        self.time_dim = time_dim
        self.query_dim = n_node_features + time_dim
        self.key_dim = n_neighbors_features + time_dim + n_edge_features
        self.merger = MergeLayer(self.query_dim, n_node_features, n_node_features, output_dimension)
        self.multi_head_target = nn.MultiheadAttention(embed_dim=self.query_dim, kdim=self.key_dim,
                                                       vdim=self.key_dim, num_heads=n_head, dropout=dropout)
        self.norm = nn.LayerNorm(output_dimension)


class GraphAttentionEmbedding(nn.Module):
    """modules/embedding_module.py:64-113, 294-329: attention layers plus one History per layer
    below the top; history maintenance calls used by the reference's driver keep their names."""

    def __init__(self, neighbor_finder, time_encoder, n_layers, n_node_features, n_edge_features,
                 n_time_features, embedding_dimension, device, n_heads=2, dropout=0.1, reuse=False,
                 history_budget=0, args=None, num_nodes=-1):
        super().__init__()
        self.neighbor_finder = neighbor_finder
        self.time_encoder = time_encoder
        self.n_layers = n_layers
        self.device = device
        self.args = args
        self.budget = history_budget
        if reuse:
            self.histories = nn.ModuleList([History(num_nodes, embedding_dimension, device, history_budget)
                                            for _ in range(n_layers - 1)])
        self.attention_models = nn.ModuleList([
            TemporalAttentionLayer(n_node_features, n_node_features, n_edge_features, n_time_features,
                                   n_node_features, n_head=n_heads, dropout=dropout)
            for _ in range(n_layers)])

    def backup_history(self):
        return [self.histories[i].emb.clone() for i in range(self.n_layers - 1)]

    def restore_history(self, backup):
        for i in range(self.n_layers - 1):
            self.histories[i].emb = backup[i]

    def reset_history(self):
        for i in range(self.n_layers - 1):
            self.histories[i].reset_parameters()

    def detach_history(self):
        for i in range(self.n_layers - 1):
            self.histories[i].detach_history()


class _Staging:
    """Ring of pinned host buffers for the per-batch inputs; a buffer is reused only after the
    copy that read it has completed."""

    def __init__(self, n_slots=8):
        self.slots = [None] * n_slots
        self.views = [None] * n_slots     # numpy views of the pinned buffers (made once per buffer)
        self.events = [None] * n_slots
        self.i = 0

    def get(self, nbytes):
        i = self.i
        self.i = (i + 1) % len(self.slots)
        if self.events[i] is not None:
            self.events[i].synchronize()
        buf = self.slots[i]
        if buf is None or buf.numel() < nbytes:
            buf = torch.empty(max(nbytes, 1 << 16), dtype=torch.uint8, pin_memory=True)
            self.slots[i] = buf
            self.views[i] = buf.numpy()
        return i, buf, self.views[i]

    def mark(self, i, stream=None):
        ev = self.events[i]
        if ev is None:
            ev = torch.cuda.Event()
            self.events[i] = ev
        ev.record(stream)


class TGN(nn.Module):
    def __init__(self, neighbor_finder, node_features, edge_features, device, n_layers=2,
                 n_heads=2, dropout=0.1, use_memory=True, node_dimension=100, time_dimension=100,
                 memory_dimension=100, embedding_module_type="graph_attention",
                 message_function="mlp", n_neighbors=None, aggregator_type="last",
                 memory_updater_type="gru",
                 use_destination_embedding_in_message=False,
                 use_source_embedding_in_message=False,
                 args=None):
        super().__init__()
        self.device = _lib.require_cuda(device)
        if embedding_module_type != "graph_attention":
            raise ValueError("Embedding Module {} not supported".format(embedding_module_type))
        if message_function != "identity":
            # the reference's "mlp" branch cannot be constructed (model/tgn_model.py:52 reads a
            # local before assignment); identity is the only working value
            raise ValueError("message_function must be 'identity'")
        if aggregator_type != "last":
            raise ValueError("Message aggregator {} not supported".format(aggregator_type))
        if not use_memory or use_destination_embedding_in_message or use_source_embedding_in_message:
            raise ValueError("only the memory-based message of the default configuration is supported")
        if n_heads != 2 or node_dimension != _lib.DIM or time_dimension != _lib.DIM or memory_dimension != _lib.DIM:
            raise ValueError("orca_b200 is built for 2 heads and 172-wide node/time/memory features")
        if n_layers not in (1, 2):
            raise ValueError("n_layers must be 1 or 2")
        self.batch_counter = 0
        self.n_layers = n_layers
        self.neighbor_finder = neighbor_finder
        self.args = args
        ef = np.asarray(edge_features, dtype=np.float32)
        if ef.shape[1] != _lib.DIM:
            raise ValueError("orca_b200 is built for 172-wide edge features")
        self.edge_raw_features = torch.from_numpy(np.ascontiguousarray(ef)).to(self.device)
        self.n_edge_features = ef.shape[1]
        self.n_nodes = args.n_nodes
        self.time_dimension = time_dimension
        self.memory_dimension = memory_dimension
        self.embedding_dimension = node_dimension
        self.n_node_features = node_dimension
        self.n_neighbors = n_neighbors
        self.embedding_module_type = embedding_module_type
        self.use_memory = use_memory
        self.time_encoder = TimeEncode(dimension=time_dimension)
        msg_dim = 2 * memory_dimension + self.n_edge_features + time_dimension
        self.memory = Memory(n_nodes=self.n_nodes, memory_dimension=memory_dimension, input_dimension=msg_dim,
                             message_dimension=msg_dim, device=self.device)
        self.memory_updater = get_memory_updater(memory_updater_type, msg_dim, memory_dimension, self.device)
        self.embedding_module = GraphAttentionEmbedding(
            neighbor_finder=neighbor_finder, time_encoder=self.time_encoder, n_layers=n_layers,
            n_node_features=node_dimension, n_edge_features=self.n_edge_features,
            n_time_features=time_dimension, embedding_dimension=node_dimension, device=self.device,
            n_heads=n_heads, dropout=dropout, reuse=args.reuse, history_budget=args.budget, args=args,
            num_nodes=self.n_nodes)
        self.affinity_score = MergeLayer(node_dimension, node_dimension, node_dimension, 1)
        self.test_mode = False
        self.to(self.device)
        # kernel-side state
        self._prepared = None
        self._ws = None
        self._ws_key = None
        self._stage = _Staging()
        self._copy_stream = None       # created with the device ring on the first batch
        self._status_host = None       # pinned copy of the status word, refreshed after every batch
        self._status_event = None
        self._status_pending = False
        self._status = torch.zeros(4, dtype=torch.int32, device=self.device)
        # last-occurrence records: push winners of even / odd batches, message winners
        self._last_pos = torch.zeros(3 * self.n_nodes, dtype=torch.int64, device=self.device)
        # this model's context in the library: its auxiliary streams, switches and tracer
        with torch.cuda.device(self.device):
            ctx = C.c_void_p(0)
            _lib.check(_lib.lib().orca_ctx_create(C.byref(ctx)))
        self._ctx = ctx
        self._input_stream = None      # stream the batch inputs are made ready on (None: the current stream)
        # candidate bitmap of the uncached set, followed by the candidate list (length word + entries)
        self._cand_bitmap = torch.zeros((self.n_nodes + 31) // 32 + 1 + _lib.CAND_CAP, dtype=torch.int32,
                                        device=self.device)
        self._epoch = np.ones(1, dtype=np.int64)
        self._dummy_prev = np.full(1, -1, dtype=np.int32)
        self.last_counts = None
        self._rank, self._world, self._group = 0, 1, None
        self._layer1_ranks = 0         # multi-GPU split by layer: ranks that compute layer 1 (0: split by rows only)
        self._exchange = None          # direct exchange buffers of the multi-GPU split (set_distributed)
        self._mode = MODE_BUDGET

    def __del__(self):
        ctx = self.__dict__.get("_ctx")
        if ctx is not None and ctx.value:
            self.__dict__["_ctx"] = None
            try:
                _lib.lib().orca_ctx_destroy(ctx)
                for base, off in self.__dict__.get("_ipc_open") or []:
                    _lib.lib().orca_ipc_close(base, off)
                self.__dict__["_ipc_open"] = []
            except Exception:      # interpreter shutdown
                pass

    def set_option(self, option, value):
        """Switch of this model's context (_lib.OPT_*: projection mode, overlap, dependent launch,
        look-ahead, wait limit, trace)."""
        _lib.check(_lib.lib().orca_ctx_set(self._ctx, int(option), int(value)))

    def last_layer1_nodes(self, n_rows):
        """Node ids of the last batch's layer-1 row list [src | dst | neg | uncached] (its first n_rows
        entries), read back from the batch workspace.  Synchronises."""
        L = _lib.lib()
        b, u_cap, k = self._ws_key
        off = L.orca_eval_workspace_row_list(b, u_cap, k, self.n_nodes, L.orca_ctx_last_parity(self._ctx))
        torch.cuda.synchronize(self.device)
        return self._ws[off: off + 4 * n_rows].view(torch.int32).cpu().numpy()

    def set_distributed(self, rank, world, group=None, exchange="direct", split="layers", layer1_ranks=None):
        """Shard every batch's attention rows and link scores over `world` GPUs of one node (one
        process per GPU, torch.distributed initialised by the caller, NCCL).  Every rank keeps full
        replicas and must be fed the same batches; results are identical on all ranks.

        exchange="direct": the layer-1 rows travel by peer stores over NVLink into exchange buffers that
        the ranks map into each other through CUDA IPC (handles are swapped here, once);
        exchange="nccl": one all-gather per batch instead.
        split="layers" (direct exchange only): the first `layer1_ranks` ranks (default world // 2) compute
        layer 1 and the memory update, the others the top layer and the scores, a batch apart;
        split="rows": every rank computes its share of the rows of both layers."""
        self._release_exchange()
        self._rank, self._world, self._group = int(rank), int(world), group
        self._layer1_ranks = 0
        self._ws_key = None
        self._desc_ref = None
        self._exchange = None
        if self._world > 1 and exchange == "direct":
            import torch.distributed as dist
            cap = self.exchange_floats(int(self.args.bs), self._world, int(self.args.n_degree), self.n_nodes)
            gcap = 2 * int(self.args.bs) * _lib.DIM
            # one allocation per rank: EXCHANGE_SLOTS * cap floats of layer-1 rows, 2 * gcap floats of memory
            # rows, then the flag words
            xbuf = torch.zeros(_lib.EXCHANGE_SLOTS * cap + 2 * gcap + _lib.FLAG_WORDS, dtype=torch.float32,
                               device=self.device)
            torch.cuda.synchronize(self.device)
            L = _lib.lib()
            rows, flags, grus, keep, err = [], [], [], [xbuf], None
            try:
                handle = (C.c_ubyte * 64)()
                off = C.c_int64(0)
                _lib.check(L.orca_ipc_export(xbuf.data_ptr(), handle, C.byref(off)))
                mine = (bytes(handle), int(off.value))
            except _lib.OrcaError as e:
                mine, err = None, e
            handles = [None] * self._world
            dist.all_gather_object(handles, mine, group=group)
            if err is None and all(h is not None for h in handles):
                try:
                    for r in range(self._world):
                        if r == self._rank:
                            base = xbuf.data_ptr()
                        else:
                            h = (C.c_ubyte * 64).from_buffer_copy(handles[r][0])
                            out = C.c_void_p(0)
                            _lib.check(L.orca_ipc_open(h, handles[r][1], C.byref(out)))
                            base = out.value
                            self._ipc_open.append((base, handles[r][1]))
                        rows.append(base)
                        grus.append(base + 4 * _lib.EXCHANGE_SLOTS * cap)
                        flags.append(base + 4 * (_lib.EXCHANGE_SLOTS * cap + 2 * gcap))
                except _lib.OrcaError as e:
                    err = e
            else:
                err = err or RuntimeError("a peer could not export its exchange buffer")
            # all ranks take the same route: peer stores only if every rank mapped every buffer
            ok = torch.tensor([0 if err else 1], device=self.device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
            if int(ok.item()) == 0:
                import warnings
                warnings.warn(f"orca_b200: peer exchange buffers could not be shared ({err}); the layer-1 rows "
                              "are all-gathered with NCCL instead")
                return
            self.set_exchange(rows, flags, cap, keep, grus, gcap)
            if split == "layers":
                a = self._world // 2 if layer1_ranks is None else int(layer1_ranks)
                if not 0 < a < self._world:
                    raise ValueError("layer1_ranks must lie between 1 and world - 1")
                self._layer1_ranks = a
            dist.barrier(group=group)

    def _release_exchange(self):
        """Lets go of the exchange buffers of an earlier set_distributed call: every rank first finishes
        what it has enqueued (peers may still be storing into this rank's buffer, and this rank into
        theirs), then the mappings of the peers' buffers are closed and the own buffer is dropped."""
        opened = self.__dict__.get("_ipc_open") or []
        if self.__dict__.get("_exchange") is not None:
            torch.cuda.synchronize(self.device)
            if self._world > 1:
                import torch.distributed as dist
                if dist.is_available() and dist.is_initialized():
                    dist.barrier(group=self._group)
        if opened:
            L = _lib.lib()
            with torch.cuda.device(self.device):
                for base, off in opened:
                    L.orca_ipc_close(base, off)
        self.__dict__["_ipc_open"] = []
        self.__dict__["_exchange"] = None

    @staticmethod
    def exchange_floats(bs, world, k, n_nodes):
        """Floats per slot of an exchange buffer for batches of up to `bs` edges: one block of
        rows_per_rank(3*bs + u_cap) rows per computing rank (at most `world` of them), u_cap =
        min(3*bs*k, n_nodes) being the most uncached neighbours a batch can have (a cold cache on the first
        batch reaches it)."""
        return (3 * bs + min(3 * bs * k, n_nodes) + world) * _lib.DIM

    def set_exchange(self, row_ptrs, flag_ptrs, cap, keep_alive=(), gru_ptrs=None, gru_cap=0):
        """Device addresses, as seen by this process, of every rank's exchange buffer (EXCHANGE_SLOTS *
        cap floats), flag words (int32[FLAG_WORDS], zeroed) and -- optional, for the node-split memory
        update -- memory-row buffer (2 * gru_cap floats)."""
        self._exchange = (list(row_ptrs), list(flag_ptrs), int(cap), list(keep_alive),
                          list(gru_ptrs) if gru_ptrs else None, int(gru_cap))
        self._exchange_seq = np.zeros(1, dtype=np.int64)
        self._desc_ref = None

    # ---- weights ------------------------------------------------------------------------------
    def load_state_dict(self, state_dict, strict=True, **kw):
        r = super().load_state_dict(state_dict, strict=strict, **kw)
        self.refresh_weights()
        return r

    def refresh_weights(self):
        """Call after changing parameters in place; load_state_dict does it itself."""
        self._prepared = None
        self.memory_updater.invalidate()

    def _weights(self):
        if self._prepared is None:
            sd = {k: v.detach().cpu().numpy() for k, v in self.state_dict().items()}
            dev = self.device
            up = lambda d: {k: (torch.from_numpy(v).to(dev) if isinstance(v, np.ndarray) else v) for k, v in d.items()}
            self._prepared = {
                "time_w": torch.from_numpy(weights.prepare_time(sd)).to(dev),
                "attn": [up(weights.prepare_attention(sd, l)) for l in range(self.n_layers)],
                "score": up(weights.prepare_score(sd)),
            }
        return self._prepared

    def attn_struct(self, layer):
        a = self._weights()["attn"][layer]
        return _lib.attn_struct(a)

    def score_struct(self):
        s = self._weights()["score"]
        return _lib.ScoreWeights(s["W1t"].data_ptr(), s["b1"].data_ptr(), s["w2"].data_ptr(), s["b2"],
                                 s["W1t_tc"].data_ptr())

    def set_neighbor_finder(self, neighbor_finder):
        self.neighbor_finder = neighbor_finder
        self.embedding_module.neighbor_finder = neighbor_finder

    # ---- model descriptor for the fused batch entry point ----------------------------------------
    def _descriptor(self, k):
        """The model descriptor of the fused batch entry.  Graph, weights and scratch pointers are filled
        once per (neighbour finder, prepared weights, k); the state tables can be replaced between calls
        (restore_memory, restore_history) and are refreshed every time."""
        nf = self.embedding_module.neighbor_finder
        w = self._weights()
        gw = self.memory_updater.prepared()
        ref = getattr(self, "_desc_ref", None)   # the objects themselves are kept: identities cannot be reused
        if ref is not None and ref[0] is nf and ref[1] is w and ref[2] is gw and ref[3] == k:
            t = self._desc
            t.mem = self.memory.c_struct()
            if self.n_layers == 2 and hasattr(self.embedding_module, "histories"):
                h = self.embedding_module.histories[0]
                t.hist_emb = h.emb.data_ptr()
                t.cache_flag = h.cache_flag_dev.data_ptr()
                t.prev_plan = h.prev_plan.data_ptr()
                t.n_prev_plan = h.n_prev.ctypes.data_as(C.POINTER(C.c_int32))
                t.plan_cap = h.prev_plan.numel()
            t.rank, t.world = self._rank, self._world
            t.layer1_ranks = self._layer1_ranks
            t.mode = self._mode
            t.input_stream = self._input_stream
            return t
        t = _lib.TgnT()
        if getattr(self, "_exchange", None) is not None:
            rows, flags, cap, _, grus, gcap = self._exchange
            for r in range(len(rows)):
                t.peer_rows[r] = rows[r]
                t.peer_flags[r] = flags[r]
                if grus:
                    t.peer_gru[r] = grus[r]
            t.exchange_cap = cap
            t.gru_cap = gcap if grus else 0
            t.exchange_seq = self._exchange_seq.ctypes.data_as(C.POINTER(C.c_int64))
        self._desc_ref, self._desc = (nf, w, gw, k), t
        t.indptr, t.adj_nbr, t.adj_eid, t.adj_ts = (nf.indptr.data_ptr(), nf.adj_nbr.data_ptr(),
                                                    nf.adj_eid.data_ptr(), nf.adj_ts.data_ptr())
        t.edge_table = self.edge_raw_features.data_ptr()
        t.n_nodes = self.n_nodes
        t.n_edge_rows = self.edge_raw_features.shape[0]
        t.time_w = w["time_w"].data_ptr()
        for l in range(self.n_layers):
            t.attn[l] = self.attn_struct(l)
        t.score = self.score_struct()
        t.gru = self.memory_updater.c_struct()
        t.n_layers = self.n_layers
        t.k = k
        t.mem = self.memory.c_struct()
        if self.n_layers == 2 and hasattr(self.embedding_module, "histories"):
            h = self.embedding_module.histories[0]
            t.hist_emb = h.emb.data_ptr()
            t.cache_flag = h.cache_flag_dev.data_ptr()
            t.prev_plan = h.prev_plan.data_ptr()
            t.n_prev_plan = h.n_prev.ctypes.data_as(C.POINTER(C.c_int32))
            t.plan_cap = h.prev_plan.numel()
        else:
            t.n_prev_plan = self._dummy_prev.ctypes.data_as(C.POINTER(C.c_int32))
        t.last_pos = self._last_pos.data_ptr()
        t.epoch_base = self._epoch.ctypes.data_as(C.POINTER(C.c_int64))
        t.rank, t.world = self._rank, self._world
        t.layer1_ranks = self._layer1_ranks
        t.cand_bitmap = self._cand_bitmap.data_ptr()
        t.mode = self._mode
        t.ctx = self._ctx
        t.input_stream = self._input_stream
        return t

    def _workspace(self, b, k):
        u_cap = min(3 * b * k, self.n_nodes) if self.n_layers == 2 else 0
        if self.n_layers == 2 and self._mode == MODE_NO_REUSE:
            u_cap = 3 * b * k          # one layer-1 row per neighbour slot
        key = (b, u_cap, k)
        if self._ws_key != key:
            # the workspace layout follows (b, u_cap, k): batches of another size get a workspace of their own
            # (kept, so that a stream whose last batch is short does not reallocate twice); the library's
            # side streams may still be reading the old one, hence the synchronisation
            cache = self.__dict__.setdefault("_ws_cache", {})
            if self._ws is not None:
                torch.cuda.synchronize(self.device)
                cache[self._ws_key] = self._ws
            ws = cache.get(key)
            if ws is None:
                nbytes = _lib.lib().orca_eval_workspace_bytes(b, u_cap, k, self.n_nodes)
                ws = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            self._ws, self._ws_key = ws, key
        return self._ws, u_cap

    # ---- one eval batch ----------------------------------------------------------------------------
    def _eval_batch(self, source_nodes, destination_nodes, negative_nodes, edge_times, edge_idxs, n_neighbors,
                    cache_plan, want_emb):
        L = _lib.lib()
        b = len(source_nodes)
        k = int(n_neighbors)
        if self._mode != MODE_BUDGET:
            cache_plan = None
        if self.n_layers == 2 and cache_plan is not None:
            h = self.embedding_module.histories[0]
            if len(cache_plan) > h.prev_plan.numel():
                h.prev_plan = torch.zeros(len(cache_plan), dtype=torch.int32, device=self.device)
                h.n_prev[0] = -1
        n_plan = len(cache_plan) if cache_plan is not None else 0
        n_i32 = 4 * b + n_plan
        off_ts = (n_i32 * 4 + 15) // 16 * 16
        total = off_ts + 8 * b
        slot, host, hn = self._stage.get(total)
        hi = hn[:n_i32 * 4].view(np.int32)
        hi[0:b] = source_nodes
        hi[b:2 * b] = destination_nodes
        hi[2 * b:3 * b] = negative_nodes
        hi[3 * b:4 * b] = edge_idxs
        if n_plan:
            hi[4 * b:] = cache_plan
        hn[off_ts:total].view(np.float64)[:] = edge_times
        # The staged batch goes to the device on a copy stream of its own, into a ring of device buffers:
        # the copy of this batch runs while the kernels of the previous one are still busy.  A device
        # buffer is overwritten only after the batch that read it has finished (ev_free), the kernels
        # start only after the copy (ev_copied).
        cur = torch.cuda.current_stream(self.device)
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(self.device)
            self._dev_ring = [None] * 4
            self._ev_free = [None] * 4
            self._ev_copied = [torch.cuda.Event() for _ in range(4)]
            self._dev_i = 0
        ds = self._dev_i
        self._dev_i = (ds + 1) % 4
        dev = self._dev_ring[ds]
        if dev is None or dev.numel() < total:
            dev = torch.empty(max(total, 1 << 16), dtype=torch.uint8, device=self.device)
            self._dev_ring[ds] = dev
            self._copy_stream.wait_stream(cur)      # a fresh buffer: ordered after everything enqueued so far
        elif self._ev_free[ds] is not None:
            self._copy_stream.wait_event(self._ev_free[ds])
        _lib.check(L.orca_stage_h2d(dev.data_ptr(), host.data_ptr(), total, self._copy_stream.cuda_stream))
        self._ev_copied[ds].record(self._copy_stream)
        self._stage.mark(slot, self._copy_stream)
        cur.wait_event(self._ev_copied[ds])
        self._input_stream = self._copy_stream.cuda_stream     # the library orders its side streams after the copy
        stream = cur.cuda_stream
        ws, u_cap = self._workspace(b, k)
        prob = torch.empty(2 * b, device=self.device)
        emb = torch.empty(3 * b, _lib.DIM, device=self.device) if want_emb else None
        desc = self._descriptor(k)
        base = dev.data_ptr()
        d_plan = base + 16 * b if cache_plan is not None else None
        if self._world > 1:
            prob, emb = self._eval_batch_sharded(desc, base, base + off_ts, b, d_plan, n_plan, u_cap, ws, want_emb)
            self.last_scores = prob
            self._release_dev(ds, cur)
            return prob, emb
        _lib.check(L.orca_tgn_eval_batch(desc, base, base + off_ts, b, d_plan, n_plan, u_cap, ws.data_ptr(),
                                         ws.numel(), prob.data_ptr(), _lib.ptr(emb), self._status.data_ptr(),
                                         stream))
        self.last_scores = prob     # [2b] = [pos | neg]: one contiguous tensor for callers that copy both
        self._release_dev(ds, cur)
        return prob, emb

    def _release_dev(self, ds, stream):
        ev = self._ev_free[ds]
        if ev is None:
            ev = self._ev_free[ds] = torch.cuda.Event()
        ev.record(stream)
        # The status word follows the batch to pinned host memory without a synchronisation; the next call
        # that finds the copy complete raises what the kernels reported (_raise_reported).
        if self._status_host is None:
            self._status_host = torch.zeros(4, dtype=torch.int32).pin_memory()
            self._status_event = torch.cuda.Event()
        self._status_host.copy_(self._status, non_blocking=True)
        self._status_event.record(stream)
        self._status_pending = True

    def _raise_reported(self):
        """Raises the device-side error of an earlier batch once its status copy has landed (capacity of the
        uncached set, ids outside a table, a bounded wait that gave up): the reference API has no status
        call, so the error surfaces at the start of a later call instead of being dropped."""
        if self._status_pending and self._status_event.query():
            self._status_pending = False
            code = int(self._status_host[0])
            if code != 0:
                raise _lib.OrcaError(code, f"a kernel of an earlier batch reported error {code} "
                                           f"(detail {int(self._status_host[3])}); results since then are invalid")

    def _eval_batch_sharded(self, desc, d_i32, d_ts, b, d_plan, n_plan, u_cap, ws, want_emb):
        if self.n_layers != 2:
            raise NotImplementedError("the multi-GPU split is built for the two-layer model")
        L = _lib.lib()
        world = self._world
        wa = self._layer1_ranks                 # split by layer: only ranks wa.. hold scores
        rpr = shard.rows_per_rank(3 * b + u_cap, wa if wa else world)
        b_max = shard.rows_per_rank(b, world - wa)
        s = _lib.stream_ptr(self.device)
        direct = getattr(self, "_exchange", None) is not None
        prob_local = torch.zeros(2 * b_max, device=self.device)
        emb2_local = torch.zeros(3 * b_max, _lib.DIM, device=self.device) if want_emb else None
        if direct:
            # the library moves the layer-1 rows itself (peer stores): the whole batch is one call
            _lib.check(L.orca_tgn_eval_batch_sharded(desc, 0, d_i32, d_ts, b, d_plan, n_plan, u_cap, ws.data_ptr(),
                                                     ws.numel(), None, None, prob_local.data_ptr(),
                                                     _lib.ptr(emb2_local), self._status.data_ptr(), s))
        else:
            emb1_local = torch.empty(rpr, _lib.DIM, device=self.device)
            _lib.check(L.orca_tgn_eval_batch_sharded(desc, 1, d_i32, d_ts, b, d_plan, n_plan, u_cap, ws.data_ptr(),
                                                     ws.numel(), emb1_local.data_ptr(), None, None, None,
                                                     self._status.data_ptr(), s))
            emb1_all = shard.all_gather_rows(emb1_local, self._group)
            _lib.check(L.orca_tgn_eval_batch_sharded(desc, 2, d_i32, d_ts, b, d_plan, n_plan, u_cap, ws.data_ptr(),
                                                     ws.numel(), None, emb1_all.data_ptr(), prob_local.data_ptr(),
                                                     _lib.ptr(emb2_local), self._status.data_ptr(), s))
        prob = shard.assemble_edges(shard.all_gather_rows(prob_local, self._group)[wa:], b, 2)
        emb = shard.assemble_edges(shard.all_gather_rows(emb2_local, self._group)[wa:], b, 3) if want_emb else None
        return prob, emb

    def check_status(self):
        """Synchronises and raises if a kernel reported an error since the last check; returns
        (rows at layer 1, unique positives, kernel launches) of the last batch."""
        h = np.zeros(4, dtype=np.int32)
        self._status_pending = False       # (this call reads, reports and clears the word itself)
        _lib.check(_lib.lib().orca_read_status(self._ctx, self._status.data_ptr(), h.ctypes.data,
                                               _lib.stream_ptr(self.device)))
        self.last_counts = (int(h[1]), int(h[2]), int(h[3]))
        return self.last_counts

    def _enter(self, reuse, train):
        self._raise_reported()
        if train:
            raise NotImplementedError("the training path (train=True) is not part of this build")
        # model/tgn_model.py:114-120: the call's `reuse` and the budget choose the recursion
        mode = MODE_NO_REUSE if not reuse else (MODE_BUDGET if self.args.budget != 0 else MODE_REUSE_ALL)
        if mode != MODE_NO_REUSE and self.n_layers == 2 and not hasattr(self.embedding_module, "histories"):
            raise AttributeError("reuse=True needs a model built with args.reuse (no history tables)")
        if mode != MODE_BUDGET and self._world > 1:
            raise NotImplementedError("the multi-GPU split is built for the budgeted recursion only")
        self._mode = mode
        self.batch_counter += 1
        if self.test_mode is False:
            # model/tgn_model.py:109-111: pending messages are flushed when eval starts
            self.update_memory_in_test(self.memory)
            self.test_mode = True

    # ---- model/tgn_model.py:95-147
    @torch.no_grad()
    def compute_temporal_embeddings(self, source_nodes, destination_nodes, negative_nodes, edge_times, edge_idxs,
                                    n_neighbors, reuse, train, cache_plan):
        self._enter(reuse, train)
        b = len(source_nodes)
        _, emb = self._eval_batch(source_nodes, destination_nodes, negative_nodes, edge_times, edge_idxs,
                                  n_neighbors, cache_plan, want_emb=True)
        return emb[:b], emb[b:2 * b], emb[2 * b:]

    # ---- model/tgn_model.py:150-157
    @torch.no_grad()
    def compute_edge_probabilities(self, source_nodes, destination_nodes, negative_nodes, edge_times, edge_idxs,
                                   n_neighbors, reuse, train, cache_plan):
        self._enter(reuse, train)
        b = len(source_nodes)
        prob, _ = self._eval_batch(source_nodes, destination_nodes, negative_nodes, edge_times, edge_idxs,
                                   n_neighbors, cache_plan, want_emb=False)
        return prob[:b].unsqueeze(1), prob[b:].unsqueeze(1)

    # ---- a whole stream of batches in one library call (the loop of evaluation/evaluation.py:18-37)
    @torch.no_grad()
    def eval_epoch(self, sources, destinations, negatives, timestamps, edge_idxs, n_neighbors, batch_size,
                   cache_plan=None, reuse=True):
        """Scores every batch of the stream (edges [i*batch_size, (i+1)*batch_size)) exactly as one
        compute_edge_probabilities call per batch would, without a Python call or a host round trip per
        batch: the batches are packed into pinned host memory, and the library copies each batch to the
        device, runs it and copies its scores back, batch after batch, asynchronously.
        cache_plan: list with one id array per batch (or None: the plan-less flag rule).
        Returns (pos, neg): float32 numpy arrays with one score per edge."""
        L = _lib.lib()
        E = len(sources)
        bs, k = int(batch_size), int(n_neighbors)
        nb = (E + bs - 1) // bs
        if nb == 0:
            return np.zeros(0, np.float32), np.zeros(0, np.float32)
        self._enter(reuse, False)
        self.batch_counter += nb - 1
        if self._mode != MODE_BUDGET:
            cache_plan = None
        world, rank = self._world, self._rank
        if world > 1 and getattr(self, "_exchange", None) is None:
            raise NotImplementedError("eval_epoch on several GPUs needs the direct exchange (set_distributed)")
        b = np.full(nb, bs, dtype=np.int32)
        b[-1] = E - (nb - 1) * bs
        n_plan = np.full(nb, -1, dtype=np.int32)
        if cache_plan is not None:
            n_plan[:] = [len(cache_plan[i]) for i in range(nb)]
        ints = 4 * b.astype(np.int64) + np.maximum(n_plan, 0)
        off_i32 = np.zeros(nb, dtype=np.int64)
        np.cumsum(ints[:-1], out=off_i32[1:])
        off_ts = np.arange(nb, dtype=np.int64) * bs
        wa = self._layer1_ranks if world > 1 else 0     # split by layer: ranks wa.. hold the scores
        wb, rb = world - wa, rank - wa
        if world == 1:
            b_loc = b.astype(np.int64)
        elif rb < 0:
            b_loc = np.zeros(nb, dtype=np.int64)
        else:
            b_loc = (b.astype(np.int64) - rb + wb - 1) // wb
        off_prob = np.zeros(nb, dtype=np.int64)
        np.cumsum(2 * b_loc[:-1], out=off_prob[1:])
        n_scores = int(2 * b_loc.sum())
        # pinned host images of the stream (kept and grown: pinning is slow)
        pin = self.__dict__.setdefault("_epoch_pin", {})

        def pinned(name, n, dtype):
            t = pin.get(name)
            if t is None or t.numel() < n or t.dtype != dtype:
                t = torch.empty(max(n, 1), dtype=dtype, pin_memory=True)
                pin[name] = t
            return t

        n_ints = int(ints.sum())
        h_i32 = pinned("i32", n_ints, torch.int32)
        h_ts = pinned("ts", E, torch.float64)
        h_prob = pinned("prob", n_scores, torch.float32)
        hi = h_i32.numpy()
        hts = h_ts.numpy()
        if self.n_layers == 2 and cache_plan is not None:
            h = self.embedding_module.histories[0]
            most = int(n_plan.max())
            if most > h.prev_plan.numel():
                h.prev_plan = torch.zeros(most, dtype=torch.int32, device=self.device)
                h.n_prev[0] = -1
        slot = (24 * bs + 4 * int(max(n_plan.max(), 0)) + 16 + 255) // 256 * 256
        dev = self.__dict__.setdefault("_epoch_dev", {})
        if dev.get("stage") is None or dev["stage"].numel() < 4 * slot:
            torch.cuda.synchronize(self.device)
            dev["stage"] = torch.empty(4 * slot, dtype=torch.uint8, device=self.device)
        if dev.get("prob") is None or dev["prob"].numel() < n_scores:
            torch.cuda.synchronize(self.device)
            dev["prob"] = torch.empty(max(n_scores, 1), dtype=torch.float32, device=self.device)
        ws, u_cap = self._workspace(bs, k)
        desc = self._descriptor(k)
        stream = torch.cuda.current_stream(self.device)
        # The stream goes to the library in chunks of a few batches: while the GPU works on one chunk the next
        # one is packed into its own part of the pinned image (the library never waits for the host).
        # (The first chunks are short -- 1, 2, 4 batches -- so that the GPU starts while most of the stream is
        # still being packed.)
        bounds, i0, chunk = [], 0, 1
        while i0 < nb:
            bounds.append((i0, min(nb, i0 + chunk)))
            i0 += chunk
            chunk = min(8, 2 * chunk)
        for i0, i1 in bounds:
            hts[i0 * bs:min(E, i1 * bs)] = timestamps[i0 * bs:min(E, i1 * bs)]
            if int(b[-1]) == bs and cache_plan is None:
                lo, up = i0 * bs, i1 * bs
                v = hi[int(off_i32[i0]):int(off_i32[i0]) + 4 * (up - lo)].reshape(i1 - i0, 4, bs)
                v[:, 0], v[:, 1], v[:, 2], v[:, 3] = (np.asarray(a[lo:up]).reshape(i1 - i0, bs) for a in
                                                       (sources, destinations, negatives, edge_idxs))
            else:
                for i in range(i0, i1):
                    o, n, lo = int(off_i32[i]), int(b[i]), i * bs
                    hi[o:o + n] = sources[lo:lo + n]
                    hi[o + n:o + 2 * n] = destinations[lo:lo + n]
                    hi[o + 2 * n:o + 3 * n] = negatives[lo:lo + n]
                    hi[o + 3 * n:o + 4 * n] = edge_idxs[lo:lo + n]
                    if n_plan[i] > 0:
                        hi[o + 4 * n:o + 4 * n + n_plan[i]] = cache_plan[i]
            ep = _lib.EpochT(h_i32.data_ptr(), h_ts.data_ptr(), off_i32[i0:].ctypes.data, off_ts[i0:].ctypes.data,
                             off_prob[i0:].ctypes.data, b[i0:].ctypes.data, n_plan[i0:].ctypes.data, i1 - i0)
            _lib.check(L.orca_tgn_eval_epoch(desc, C.byref(ep), u_cap, ws.data_ptr(), ws.numel(),
                                             dev["stage"].data_ptr(), dev["stage"].numel(), dev["prob"].data_ptr(),
                                             h_prob.data_ptr(), self._status.data_ptr(), stream.cuda_stream))
        stream.synchronize()
        local = h_prob.numpy()[:n_scores]
        pos = np.empty(E, dtype=np.float32)
        neg = np.empty(E, dtype=np.float32)
        if world == 1:
            if int(b[-1]) == bs:
                v = local.reshape(nb, 2, bs)
                pos[:], neg[:] = v[:, 0].reshape(-1), v[:, 1].reshape(-1)
            else:
                for i in range(nb):
                    o, n, lo = int(off_prob[i]), int(b[i]), i * bs
                    pos[lo:lo + n], neg[lo:lo + n] = local[o:o + n], local[o + n:o + 2 * n]
            return pos, neg
        # every scoring rank holds the scores of its edges (edge e of a batch: scoring rank e % wb): one exchange
        # per epoch
        import torch.distributed as dist
        most = 2 * int(((b.astype(np.int64) + wb - 1) // wb).sum())
        mine = torch.zeros(most, dtype=torch.float32, device=self.device)
        mine[:n_scores] = dev["prob"][:n_scores]
        every = shard.all_gather_rows(mine, self._group).cpu().numpy()
        for r in range(wb):
            bl = (b.astype(np.int64) - r + wb - 1) // wb
            o = 0
            for i in range(nb):
                n, lo = int(bl[i]), i * bs
                pos[lo + r:lo + int(b[i]):wb] = every[wa + r, o:o + n]
                neg[lo + r:lo + int(b[i]):wb] = every[wa + r, o + n:o + 2 * n]
                o += 2 * n
        return pos, neg

    def update_memory(self, memory, positives):
        self.memory_updater.update_memory(memory, positives)

    def update_memory_in_test(self, memory):
        self.memory_updater.update_memory_in_test(memory)
