"""Shared helpers for the parity tests."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_golden(name):
    z = np.load(os.path.join(GOLDEN, name))
    return {k: z[k] for k in z.files}


def rel_err(a, b):
    """max |a-b| / max |b|  (norm-wise relative error, the measure every tolerance in tests/ refers to)."""
    a = torch.as_tensor(a).double()
    b = torch.as_tensor(b).double()
    denom = b.abs().max().clamp_min(1e-30)
    return float((a - b).abs().max() / denom)


def listed_from_dense(g):
    """Turn a dense-vocabulary flash fixture into listed-slot operator inputs."""
    from oracle import ema_oracle as orc
    x = torch.from_numpy(g["x"]).long()
    B, L = x.shape
    H = int(g["H"])
    E_k = torch.from_numpy(g["E_k"])
    E_v = torch.from_numpy(g["E_v"])
    D = E_k.shape[1]
    hd = D // H
    unique, k_max = orc.build_unique_index(x)
    safe = unique.clamp_min(0)
    E_k_act = E_k[safe] * (unique >= 0).unsqueeze(-1)
    E_v_act = E_v[safe] * (unique >= 0).unsqueeze(-1)
    Q = torch.from_numpy(g["Q"]).view(B, L, H, hd).transpose(1, 2).contiguous()
    dO = torch.from_numpy(g["dO"]).view(B, L, H, hd).transpose(1, 2).contiguous()
    W_pe = torch.from_numpy(g["W_dn"]).t().contiguous()
    return dict(x=x, unique=unique, K_max=k_max, E_k=E_k_act.contiguous(), E_v=E_v_act.contiguous(), Q=Q, dO=dO,
                W_pe=W_pe, rhos=torch.from_numpy(g["rhos"]), V=int(g["V"]), H=H, hd=hd,
                use_silu=bool(int(g["use_silu"])))


def dense_grads_from_listed(inp, dE_act, used):
    """Scatter per-sample listed-slot gradients back to vocabulary rows and return the rows in ``used``."""
    unique = inp["unique"]
    V = inp["V"]
    D = dE_act.shape[-1]
    full = torch.zeros(V, D, dtype=dE_act.dtype)
    for b in range(unique.shape[0]):
        ok = unique[b] >= 0
        full.index_add_(0, unique[b][ok], dE_act[b][ok])
    return full[torch.as_tensor(used).long()]
