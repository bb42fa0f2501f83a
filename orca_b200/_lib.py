"""ctypes binding of liborca_b200.so (the C ABI declared in include/orca_b200.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liborca_b200.so")

DIM = 172
QT_DIM = 1032
QT_LD = 1056
MSG_DIM = 688
CAND_CAP = 2048   # ORCA_CAND_CAP
EXCHANGE_SLOTS = 4  # ORCA_EXCHANGE_SLOTS
FLAG_WORDS = 48     # ORCA_FLAG_WORDS
# options of orca_ctx_set
OPT_PROJECTION_MODE, OPT_OVERLAP, OPT_DEPENDENT_LAUNCH, OPT_LOOKAHEAD, OPT_WAIT_LIMIT, OPT_TRACE = range(6)

c_f32p = C.c_void_p
c_i32p = C.c_void_p


class AttnWeights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("Mq", "cq", "G", "b1", "g", "W2t", "b2", "ln_w", "ln_b",
                                          "Mq_tc", "G_tc", "W2t_tc")]


class ScoreWeights(C.Structure):
    _fields_ = [("W1t", C.c_void_p), ("b1", C.c_void_p), ("w2", C.c_void_p), ("b2", C.c_float),
                ("W1t_tc", C.c_void_p)]


class GruWeights(C.Structure):
    _fields_ = [("Wg", C.c_void_p), ("bg", C.c_void_p), ("Wg_tc", C.c_void_p)]


class MemoryT(C.Structure):
    _fields_ = [("memory", C.c_void_p), ("last_update", C.c_void_p), ("messages", C.c_void_p),
                ("msg_ts", C.c_void_p), ("msg_flag", C.c_void_p), ("n_nodes", C.c_int64)]


class TgnT(C.Structure):
    _fields_ = [
        ("indptr", C.c_void_p), ("adj_nbr", C.c_void_p), ("adj_eid", C.c_void_p), ("adj_ts", C.c_void_p),
        ("edge_table", C.c_void_p), ("n_nodes", C.c_int64), ("n_edge_rows", C.c_int64),
        ("time_w", C.c_void_p),
        ("attn", AttnWeights * 2),
        ("score", ScoreWeights),
        ("gru", GruWeights),
        ("n_layers", C.c_int32), ("k", C.c_int32),
        ("mem", MemoryT),
        ("hist_emb", C.c_void_p), ("cache_flag", C.c_void_p),
        ("prev_plan", C.c_void_p), ("n_prev_plan", C.POINTER(C.c_int32)), ("plan_cap", C.c_int32),
        ("last_pos", C.c_void_p), ("epoch_base", C.POINTER(C.c_int64)),
        ("rank", C.c_int32), ("world", C.c_int32),
        ("cand_bitmap", C.c_void_p),
        ("mode", C.c_int32),
        ("peer_rows", C.c_void_p * 8),
        ("peer_flags", C.c_void_p * 8),
        ("exchange_cap", C.c_int64),
        ("peer_gru", C.c_void_p * 8),
        ("gru_cap", C.c_int64),
        ("exchange_seq", C.POINTER(C.c_int64)),
        ("ctx", C.c_void_p),
        ("input_stream", C.c_void_p),
        ("layer1_ranks", C.c_int32),
    ]


class EpochT(C.Structure):
    _fields_ = [("h_i32", C.c_void_p), ("h_ts", C.c_void_p), ("off_i32", C.c_void_p), ("off_ts", C.c_void_p),
                ("off_prob", C.c_void_p), ("b", C.c_void_p), ("n_plan", C.c_void_p), ("n_batches", C.c_int64)]


# every symbol the header declares: name -> (restype, argtypes)
_V, _I32, _I64 = C.c_void_p, C.c_int32, C.c_int64
SYMBOLS = {
    "orca_last_error": (C.c_char_p, []),
    "orca_version": (C.c_int, []),
    "orca_ctx_create": (C.c_int, [C.POINTER(C.c_void_p)]),
    "orca_ctx_destroy": (C.c_int, [_V]),
    "orca_ctx_set": (C.c_int, [_V, _I32, _I64]),
    "orca_ctx_set_status_word": (C.c_int, [_V, _V]),
    "orca_ctx_last_parity": (C.c_int, [_V]),
    "orca_csr_build_host": (C.c_int, [_V, _V, _V, _V, _I64, _I64, _V, _V, _V, _V]),
    "orca_sample_topk": (C.c_int, [_V, _V, _V, _V, _I64, _V, _V, _I32, _V, _I32, _V, _V, _V, _V, _V, _V]),
    "orca_sample_topk_mark": (C.c_int, [_V, _V, _V, _V, _I64, _V, _V, _I32, _V, _I32, _V, _V, _V, _V, _V, _V, _V, _V]),
    "orca_find_uncached_marked": (C.c_int, [_V, _I32, _I64, _V, _V, _I32, _V, _V, _V]),
    "orca_find_before": (C.c_int, [_V, _V, _I64, _V, _V, _I32, _V, _V]),
    "orca_find_uncached_scratch_bytes": (_I64, [_I64]),
    "orca_find_uncached": (C.c_int, [_V, _I32, _I32, _V, _I64, _V, _V, _I32, _V, _V, _V, _V]),
    "orca_last_occurrence": (C.c_int, [_V, _I32, _V, _I64, _V, _I64, _V, _V, _V, _V]),
    "orca_attn_query": (C.c_int, [C.POINTER(AttnWeights), _V, _V, _I32, _V, _V, _V]),
    "orca_attn_gather": (C.c_int, [_V, _V, _V, _V, _V, _V, _V, _I32, _I32, _V, _V, _V, _V, _V]),
    "orca_attn_gather_profile": (C.c_int, [_V, _I32, _V]),
    "orca_attn_gather_profile_read": (C.c_int, [_V, _V, _V]),
    "orca_attn_output": (C.c_int, [C.POINTER(AttnWeights), _V, _V, _V, _V, _I32, _V, _V, _V, _V, _V, _V, _V]),
    "orca_history_pull": (C.c_int, [_V, _V, _I64, _V, _V]),
    "orca_history_push": (C.c_int, [_V, _V, _V, _V, _I32, _V, _V]),
    "orca_history_set_flags": (C.c_int, [_V, _I64, _V, _I32, _V, _I32, _V]),
    "orca_score": (C.c_int, [C.POINTER(ScoreWeights), _V, _I32, _V, _V]),
    "orca_message_store": (C.c_int, [C.POINTER(MemoryT), _V, _V, _V, _V, _V, _V, _I32, _V, _I32, _V, _V, _V]),
    "orca_gru_update": (C.c_int, [C.POINTER(GruWeights), C.POINTER(MemoryT), _V, _I32, _V, _I32, _V, _V]),
    "orca_gru_scratch_bytes": (_I64, [_I32]),
    "orca_gru_update_static": (C.c_int, [C.POINTER(GruWeights), C.POINTER(MemoryT), _V, _I32, _V, _I32, _V]),
    "orca_plan_host": (C.c_int, [_I32, _V, _V, _I64, _I32, _I32, _V, _I64, _I32, C.c_uint32, _V, _I64, _V, _V]),
    "orca_csr_build_workspace_bytes": (_I64, [_I64, _I64]),
    "orca_csr_build": (C.c_int, [_V, _V, _V, _V, _I64, _I64, _V, _V, _V, _V, _V, _V, _I64, _V]),
    "orca_plan_mrd_workspace_bytes": (_I64, [_I64, _I32, _I32, _I64, _I32]),
    "orca_plan_mrd": (C.c_int, [_V, _I64, _I32, _I32, _V, _I64, _I32, _V, _I64, _V, _V, _V, _V, _I64, _V]),
    "orca_plan_device_workspace_bytes": (_I64, [_I32, _I64, _I32, _I32, _I64, _I32]),
    "orca_plan_device": (C.c_int, [_I32, _V, _I64, _I32, _I32, _V, _I64, _I32, C.c_uint32, _V, _I64, _V, _V, _V, _V,
                                   _I64, _V]),
    "orca_eval_workspace_bytes": (_I64, [_I32, _I32, _I32, _I64]),
    "orca_eval_workspace_row_list": (_I64, [_I32, _I32, _I32, _I64, _I32]),
    "orca_tgn_eval_batch": (C.c_int, [C.POINTER(TgnT), _V, _V, _I32, _V, _I32, _I32, _V, _I64, _V, _V, _V, _V]),
    "orca_tgn_eval_batch_sharded": (C.c_int, [C.POINTER(TgnT), _I32, _V, _V, _I32, _V, _I32, _I32, _V, _I64, _V, _V,
                                              _V, _V, _V, _V]),
    "orca_tgn_eval_epoch": (C.c_int, [C.POINTER(TgnT), C.POINTER(EpochT), _I32, _V, _I64, _V, _I64, _V, _V, _V, _V]),
    "orca_stage_h2d": (C.c_int, [_V, _V, C.c_int64, _V]),
    "orca_ipc_export": (C.c_int, [_V, _V, C.POINTER(C.c_int64)]),
    "orca_ipc_open": (C.c_int, [_V, C.c_int64, C.POINTER(C.c_void_p)]),
    "orca_ipc_close": (C.c_int, [_V, C.c_int64]),
    "orca_trace_phases": (C.c_int, []),
    "orca_trace_phase_name": (C.c_char_p, [_I32]),
    "orca_trace_read": (C.c_int, [_V, _V]),
    "orca_read_status": (C.c_int, [_V, _V, _V, _V]),
}

_lib = None


def lib():
    """The loaded library.  Raises if it has not been built (python -m orca_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m orca_b200.build` "
                              "(nvcc, sm_100a). There is no CPU fallback.")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


class OrcaError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"orca_b200 error {code}: {msg}")
        self.code = code


def check(rc):
    if rc != 0:
        raise OrcaError(rc, lib().orca_last_error().decode())


def ptr(t):
    """Device (or host) address of a torch tensor / numpy array, None -> NULL."""
    if t is None:
        return None
    if isinstance(t, torch.Tensor):
        return t.data_ptr()
    if isinstance(t, np.ndarray):
        return t.ctypes.data
    raise TypeError(type(t))


ATTN_FIELDS = ("Mq", "cq", "G", "b1", "g", "W2t", "b2", "ln_w", "ln_b", "Mq_tc", "G_tc", "W2t_tc")


def attn_struct(w):
    """AttnWeights from a dict of device tensors (weights.prepare_attention uploaded)."""
    return AttnWeights(*[w[k].data_ptr() for k in ATTN_FIELDS])


def stream_ptr(device=None):
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(device):
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError("orca_b200 runs on a CUDA device only (no CPU path); got device=%s" % device)
    if not torch.cuda.is_available():
        raise RuntimeError("orca_b200 needs a CUDA device and none is available (no CPU path)")
    return device
