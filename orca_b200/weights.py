"""Prepared weights: the reference's parameters re-associated for the kernels.

One query attends K keys that share the key/value projections, so both projections can be moved
off the K gathered rows (model/temporal_attention.py:41-55 with torch.nn.MultiheadAttention):

  logit_hj = s * q_h . (Wk_h k_j + bk_h) = (s * Wk_h^T q_h) . k_j + const   (const cancels in softmax)
  sum_j a_hj (Wv_h k_j + bv_h)           = Wv_h (sum_j a_hj k_j) + bv_h      (weights sum to one)

With q = Wq [h_src | cos(b_t)] + bq linear in h_src, the whole query side collapses to one matrix
``Mq`` and the whole output side (V projection, out projection, first merger layer) to one matrix
``G``.  The gather-attention kernel then touches no weights at all.  Composition is done in
float64 and rounded once to float32.

All matrices are stored row-major [in, out] as the C ABI expects (include/orca_b200.h).
"""
from __future__ import annotations

import math

import numpy as np

D = 172
HEADS = 2
QT_HEAD = 528     # column stride of one head of the projected query (516 used)
TC_BN, TC_BK = 176, 64


def _bf16_round(x):
    """float32 -> nearest bfloat16 (ties to even), returned as float32 with the low 16 bits zero."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32).view(np.float32)


def pack_tc(W, bn=None):
    """Packs a row-major [K, N] matrix for the tensor-core kernel (csrc/tc_gemm.cu).

    N is cut into tiles of `bn` (default 176) columns and K into blocks of 64 rows (both zero padded).
    One (tile, block) stage image is [head | tail], each [8 chunks][bn columns][8 bf16]: element
    (k, n) of the block sits at chunk k // 8, column n, position k % 8 -- the K-major, no-swizzle
    core-matrix layout the MMA reads from shared memory -- so that a stage is one contiguous bulk
    copy.  head = the value rounded to bf16, tail = the remainder rounded to bf16 (16 significant
    bits together).  Returned as uint16 [n_tiles, n_kblocks, 2, 8, bn, 8]."""
    W = np.asarray(W, dtype=np.float32)
    K, N = W.shape
    bn = bn or TC_BN
    nkb, nt = -(-K // TC_BK), -(-N // bn)
    P = np.zeros((nkb * TC_BK, nt * bn), dtype=np.float32)
    P[:K, :N] = W
    head = _bf16_round(P)
    tail = _bf16_round(P - head)

    def image(X):  # [nkb*64, nt*176] -> [nt, nkb, 8, 176, 8] of bf16 bit patterns
        bits = (X.view(np.uint32) >> 16).astype(np.uint16)
        return bits.reshape(nkb, TC_BK // 8, 8, nt, bn).transpose(3, 0, 1, 4, 2)

    return np.ascontiguousarray(np.stack([image(head), image(tail)], axis=2))


def _f64(x):
    return np.asarray(x, dtype=np.float64)


def prepare_attention(sd, layer: int, dim: int = D, heads: int = HEADS):
    p = f"embedding_module.attention_models.{layer}."
    Wq = _f64(sd[p + "multi_head_target.q_proj_weight"])
    Wk = _f64(sd[p + "multi_head_target.k_proj_weight"])
    Wv = _f64(sd[p + "multi_head_target.v_proj_weight"])
    bias = _f64(sd[p + "multi_head_target.in_proj_bias"])
    Wo = _f64(sd[p + "multi_head_target.out_proj.weight"])
    bo = _f64(sd[p + "multi_head_target.out_proj.bias"])
    W1 = _f64(sd[p + "merger.fc1.weight"])
    E = Wq.shape[0]                 # 344 = node + time
    kd = Wk.shape[1]                # 516 = node + edge + time
    hd = E // heads
    if dim != D or E != 2 * D or kd != 3 * D or heads != HEADS:
        raise ValueError("orca_b200 is built for 172-wide features and 2 heads")
    bq, bv = bias[:E], bias[2 * E:]
    src_t = np.cos(_f64(sd["time_encoder.w.bias"]))            # time encoding of a zero gap
    A = Wq[:, :dim]                                             # [344, 172]
    a = Wq[:, dim:] @ src_t + bq                                # [344]
    s = 1.0 / math.sqrt(hd)
    Mq = np.zeros((dim, heads * QT_HEAD))
    cq = np.zeros(heads * QT_HEAD)
    G = np.zeros((heads * kd + dim, dim))
    W1a, W1b = W1[:, :E], W1[:, E:]
    for h in range(heads):
        rows = slice(h * hd, (h + 1) * hd)
        Mq[:, h * QT_HEAD:h * QT_HEAD + kd] = s * (A[rows].T @ Wk[rows])  # [172, 516]
        cq[h * QT_HEAD:h * QT_HEAD + kd] = s * (Wk[rows].T @ a[rows])
        P_h = Wo[:, rows] @ Wv[rows]                                     # [344, 516]
        G[h * kd:(h + 1) * kd] = (W1a @ P_h).T                           # [516, 172]
    G[heads * kd:] = W1b.T
    c_o = Wo @ bv + bo
    out = {
        "Mq": Mq, "cq": cq, "G": G, "b1": _f64(sd[p + "merger.fc1.bias"]), "g": W1a @ c_o,
        "W2t": _f64(sd[p + "merger.fc2.weight"]).T, "b2": _f64(sd[p + "merger.fc2.bias"]),
        "ln_w": _f64(sd[p + "norm.weight"]), "ln_b": _f64(sd[p + "norm.bias"]),
    }
    out = {k: np.ascontiguousarray(v, dtype=np.float32) for k, v in out.items()}
    for k in ("Mq", "G", "W2t"):
        out[k + "_tc"] = pack_tc(out[k])
    return out


def prepare_gru(sd, dim: int = D):
    p = "memory_updater.memory_updater."
    Wih, Whh = _f64(sd[p + "weight_ih"]), _f64(sd[p + "weight_hh"])
    bih, bhh = _f64(sd[p + "bias_ih"]), _f64(sd[p + "bias_hh"])
    msg = Wih.shape[1]
    Wg = np.zeros((msg + dim, 4 * dim))
    bg = np.zeros(4 * dim)
    j = np.arange(dim)
    # unit j owns columns 4j..4j+3 = (r, z, n from the message, n from the memory)
    Wg[:msg, 4 * j + 0] = Wih[j].T
    Wg[msg:, 4 * j + 0] = Whh[j].T
    bg[4 * j + 0] = bih[j] + bhh[j]
    Wg[:msg, 4 * j + 1] = Wih[dim + j].T
    Wg[msg:, 4 * j + 1] = Whh[dim + j].T
    bg[4 * j + 1] = bih[dim + j] + bhh[dim + j]
    Wg[:msg, 4 * j + 2] = Wih[2 * dim + j].T
    bg[4 * j + 2] = bih[2 * dim + j]
    Wg[msg:, 4 * j + 3] = Whh[2 * dim + j].T
    bg[4 * j + 3] = bhh[2 * dim + j]
    Wg = np.ascontiguousarray(Wg, dtype=np.float32)
    bg_pad = np.zeros(4 * TC_BN, dtype=np.float32)
    bg_pad[:4 * dim] = bg
    return {"Wg": Wg, "bg": bg_pad, "Wg_tc": pack_tc(Wg)}


def prepare_score(sd):
    W1t = np.ascontiguousarray(_f64(sd["affinity_score.fc1.weight"]).T, dtype=np.float32)
    return {
        "W1t": W1t, "W1t_tc": pack_tc(W1t),
        "b1": np.asarray(sd["affinity_score.fc1.bias"], dtype=np.float32),
        "w2": np.ascontiguousarray(np.asarray(sd["affinity_score.fc2.weight"], dtype=np.float32).reshape(-1)),
        "b2": float(np.asarray(sd["affinity_score.fc2.bias"]).reshape(-1)[0]),
    }


def prepare_time(sd):
    if np.any(np.asarray(sd["time_encoder.w.bias"]) != 0):
        raise ValueError("the time encoder's bias is frozen at zero in the reference "
                         "(model/time_encoding.py:19-21); a nonzero bias is not supported")
    w = np.ascontiguousarray(np.asarray(sd["time_encoder.w.weight"], dtype=np.float32).reshape(-1))
    # The gather kernel picks the cosine variant of a whole group of 64 columns from the group's first
    # frequency: that is only right for the reference's frozen frequencies (positive, falling) and for
    # groups whose frequencies stay within a factor 2^23 of each other (fixed-point reduction needs
    # arguments above 2^-8 when the group's largest argument is below 2^30).
    if np.any(w <= 0) or np.any(np.diff(w) > 0):
        raise ValueError("the time encoder's frequencies must be positive and non-increasing, as the reference "
                         "freezes them (model/time_encoding.py:18); other frequencies are not supported")
    for lo in range(0, len(w), 64):
        if w[lo] / w[min(lo + 63, len(w) - 1)] >= 2.0 ** 23:
            raise ValueError("the time encoder's frequencies fall too fast within a group of 64 columns")
    return w
