"""The re-associated weights (host logic, no GPU): evaluating the kernels' formulas in numpy
float64 must reproduce the oracle's attention layer, GRU cell and scorer."""
import numpy as np
import torch

from orca_b200 import params, weights
from oracle import tgn_oracle

D = 172


def _rand_case(seed, n=37, k=10):
    rs = np.random.RandomState(seed)
    h_src = rs.randn(n, D).astype(np.float32)
    h_nbr = rs.randn(n, k, D).astype(np.float32)
    ef = rs.randn(n, k, D).astype(np.float32)
    dt = (rs.rand(n, k) * 1e5).astype(np.float32)
    nbr = rs.randint(1, 50, size=(n, k))
    nbr[0] = 0            # a row with no neighbour at all
    nbr[1, :7] = 0        # a partly padded row
    return h_src, h_nbr, ef, dt, nbr


def test_attention_reassociation():
    sd = params.random_state_dict(2, seed=3)
    p = {k: torch.as_tensor(v) for k, v in sd.items()}
    h_src, h_nbr, ef, dt, nbr = _rand_case(0)
    for layer in (0, 1):
        want = tgn_oracle.attention_layer(p, layer, torch.as_tensor(h_src), torch.as_tensor(h_nbr),
                                          torch.as_tensor(ef), torch.as_tensor(dt), nbr).numpy()
        w = {k: v.astype(np.float64) for k, v in weights.prepare_attention(sd, layer).items()}
        assert w["Mq"].shape == (172, 1056) and not w["Mq"][:, 516:528].any()
        tw = weights.prepare_time(sd).astype(np.float32)
        qt = h_src.astype(np.float64) @ w["Mq"] + w["cq"]                      # [n, 1032]
        tenc = np.cos((dt[..., None] * tw).astype(np.float32)).astype(np.float64)
        key = np.concatenate([h_nbr, ef, tenc], axis=2).astype(np.float64)      # [n, k, 516]
        mask = nbr == 0
        valid = ~mask.all(axis=1)
        ctx = np.zeros((len(h_src), 2 * 516))
        for h in range(2):
            logit = np.einsum("nc,nkc->nk", qt[:, h * 528:h * 528 + 516], key)
            logit[mask] = -np.inf
            logit[~valid] = 0
            a = np.exp(logit - logit.max(axis=1, keepdims=True))
            a /= a.sum(axis=1, keepdims=True)
            ctx[:, h * 516:(h + 1) * 516] = np.einsum("nk,nkc->nc", a, key)
        ctx[~valid] = 0
        hid = np.maximum(np.concatenate([ctx, h_src], axis=1) @ w["G"] + w["b1"] + valid[:, None] * w["g"], 0)
        y = hid @ w["W2t"] + w["b2"]
        y = (y - y.mean(1, keepdims=True)) / np.sqrt(y.var(1, keepdims=True) + 1e-5) * w["ln_w"] + w["ln_b"]
        assert np.max(np.abs(y - want)) < 2e-5


def test_gru_and_score_layout():
    sd = params.random_state_dict(1, seed=5)
    p = {k: torch.as_tensor(v) for k, v in sd.items()}
    rs = np.random.RandomState(1)
    x = rs.randn(9, 4 * D).astype(np.float32)
    h = rs.randn(9, D).astype(np.float32)
    want = tgn_oracle.gru_cell(p, torch.as_tensor(x), torch.as_tensor(h)).numpy()
    g = weights.prepare_gru(sd)
    acc = np.concatenate([x, h], 1).astype(np.float64) @ g["Wg"].astype(np.float64) + g["bg"][:4 * D]
    acc = acc.reshape(9, D, 4)
    sig = lambda v: 1 / (1 + np.exp(-v))
    r, z = sig(acc[..., 0]), sig(acc[..., 1])
    n = np.tanh(acc[..., 2] + r * acc[..., 3])
    assert np.max(np.abs((1 - z) * n + z * h - want)) < 1e-5

    a, b = rs.randn(6, D).astype(np.float32), rs.randn(6, D).astype(np.float32)
    want = torch.sigmoid(tgn_oracle.affinity(p, torch.as_tensor(a), torch.as_tensor(b))).numpy().ravel()
    s = weights.prepare_score(sd)
    hid = np.maximum(np.concatenate([a, b], 1).astype(np.float64) @ s["W1t"] + s["b1"], 0)
    assert np.max(np.abs(sig(hid @ s["w2"] + s["b2"]) - want)) < 1e-6


def test_tensor_core_weight_packing():
    """head + tail reproduces the matrix to ~2^-16 and the stage image puts element (k, n) at
    [tile n // 176][block k // 64][part][chunk (k % 64) // 8][column n % 176][k % 8]."""
    rs = np.random.RandomState(0)
    W = rs.randn(1204, 172).astype(np.float32)
    P = weights.pack_tc(W)
    assert P.shape == (1, 19, 2, 8, 176, 8) and P.dtype == np.uint16
    as_f32 = lambda bits: (bits.astype(np.uint32) << 16).view(np.float32)
    rec = (as_f32(P[:, :, 0]) + as_f32(P[:, :, 1])).transpose(1, 2, 4, 0, 3).reshape(19 * 64, 176)   # [k, n]
    assert np.max(np.abs(rec[:1204, :172] - W) / np.maximum(np.abs(W), 1e-30)) < 2 ** -15
    assert not rec[1204:].any() and not rec[:, 172:].any()
    k, n = 1000, 37
    got = as_f32(P[0, k // 64, 0, (k % 64) // 8, n, k % 8]) + as_f32(P[0, k // 64, 1, (k % 64) // 8, n, k % 8])
    assert got == rec[k, n]
    assert weights.pack_tc(rs.randn(172, 1056).astype(np.float32)).shape == (6, 3, 2, 8, 176, 8)
