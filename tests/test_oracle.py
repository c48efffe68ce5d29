"""The CPU oracle against the reference's golden vectors and known-answer tests (no GPU)."""
import math

import numpy as np
import pytest
import torch

from oracle import ema_oracle as orc
from helpers import load_golden, rel_err, listed_from_dense, dense_grads_from_listed


# ---- known-answer vectors restated from the reference's scan tests -------------------------------
def test_scan_within_doc_closed_form():
    # tests/test_doc_boundary.py:75-105
    x = torch.tensor([[0, 1, 0, 2, 0, 1]])
    rhos = torch.tensor([0.9, 0.5])
    C = orc.query_scan(x, rhos, 3, doc_ids=torch.zeros(1, 6, dtype=torch.long))
    assert torch.allclose(C[0, 0], torch.zeros(2))
    assert torch.allclose(C[0, 2], rhos ** 2, atol=1e-6)
    assert torch.allclose(C[0, 4], (rhos ** 2 + 1.0) * rhos ** 2, atol=1e-6)


def test_scan_cross_doc_isolation():
    # tests/test_doc_boundary.py:22-72
    x = torch.tensor([[0, 1, 2, 0, 1, 0, 1, 3, 0, 1]])
    doc_ids = torch.tensor([[0, 0, 0, 0, 0, 1, 1, 1, 1, 1]])
    rhos = torch.tensor([0.9, 0.8, 0.7, 0.6])
    C = orc.query_scan(x, rhos, 5, doc_ids=doc_ids)
    C0 = orc.query_scan(x, rhos, 5)
    assert torch.allclose(C[0, 5], torch.zeros(4))
    assert C0[0, 5].abs().sum() > 0
    assert torch.allclose(C[0, 8], rhos ** 3, atol=1e-6)


def test_scan_c_base_returned_undecayed_at_t0():
    # tests/test_doc_boundary.py:108-134
    x = torch.tensor([[0, 1, 0, 2]])
    rhos = torch.tensor([0.9, 0.5])
    c_init = torch.tensor([[[2.0, 1.5], [0.0, 0.0], [0.0, 0.0]]])
    keys = torch.tensor([[0, 1, 2]])
    C = orc.query_scan(x, rhos, 3, c_init=c_init, c_init_keys=keys, doc_ids=torch.zeros(1, 4, dtype=torch.long))
    assert torch.allclose(C[0, 0], torch.tensor([2.0, 1.5]))


def test_scan_manual_recurrence_chunked():
    # tests/test_pipeline_thorough.py:191-271: tokens [1,2,1,3,1,2,1], N=4, chunked with c_base carry-over
    tokens = [1, 2, 1, 3, 1, 2, 1]
    N, V = 4, 4
    rhos = orc.make_rhos(N, 1.0, 16.0)
    full = orc.query_scan(torch.tensor([tokens]), rhos, V)[0]
    state = np.zeros((V, N), np.float32)
    last = np.full(V, -1)
    for t, v in enumerate(tokens):
        if last[v] >= 0:
            state[v] = state[v] * rhos.numpy() ** (t - last[v])
        assert np.allclose(full[t].numpy(), state[v], atol=1e-6)
        state[v] += 1.0
        last[v] = t
    # chunked: c_base = state after last occurrence decayed to the chunk start (mathbrain/data.py:128-140)
    for bs in (2, 3, 4):
        for start in range(0, len(tokens), bs):
            chunk = tokens[start:start + bs]
            keys = sorted(set(tokens[:start + bs]))
            c_base = torch.zeros(1, len(keys), N)
            for i, k in enumerate(keys):
                occ = [s for s in range(start) if tokens[s] == k]
                if occ:
                    c_base[0, i] = (full[occ[-1]] + 1.0) * rhos ** float(start - occ[-1])
            C = orc.query_scan(torch.tensor([chunk]), rhos, V, c_init=c_base, c_init_keys=torch.tensor([keys]))
            assert torch.allclose(C[0], full[start:start + len(chunk)], atol=1e-5)


# ---- fixtures generated from the unmodified reference ------------------------------------------
@pytest.mark.parametrize("name", ["scan_ref_a.npz", "scan_ref_docs.npz"])
def test_scan_matches_reference_fixture(name):
    g = load_golden(name)
    x = torch.from_numpy(g["x"])
    doc_ids = torch.from_numpy(g["doc_ids"]) if g["doc_ids"].size else None
    rhos = torch.from_numpy(g["rhos"])
    C = orc.query_scan(x, rhos, int(g["V"]), torch.from_numpy(g["c_init"]), torch.from_numpy(g["keys"]), doc_ids)
    assert rel_err(C, g["C_seq"]) < 1e-5          # EMA state tolerance: 1e-5 relative, fp32
    C2 = orc.query_scan(x, rhos, int(g["V"]), doc_ids=doc_ids)
    assert rel_err(C2, g["C_seq_nokeys"]) < 1e-5


def test_scan_equals_memory_state_at_own_slot():
    g = load_golden("scan_ref_a.npz")
    x = torch.from_numpy(g["x"])
    keys = torch.from_numpy(g["keys"])
    rhos = torch.from_numpy(g["rhos"])
    c_init = torch.from_numpy(g["c_init"])
    M = orc.memory_states(x, keys, rhos, c_init)
    C = torch.from_numpy(g["C_seq"])
    for b in range(x.shape[0]):
        for t in range(x.shape[1]):
            hit = (keys[b] == x[b, t]).nonzero()
            if hit.numel():
                assert torch.allclose(M[b, t, int(hit[0])], C[b, t], atol=2e-5, rtol=1e-5)


@pytest.mark.parametrize("name", ["flash_ref_silu.npz", "flash_ref_linear.npz", "flash_ref_small_w.npz"])
def test_flash_oracle_matches_reference_fixture(name):
    g = load_golden(name)
    inp = listed_from_dense(g)
    out = orc.flash_ema(inp["Q"], inp["x"], inp["E_k"], inp["E_v"], inp["W_pe"], inp["rhos"], inp["V"],
                        inp["unique"], use_silu=inp["use_silu"], dO=inp["dO"])
    B, H, L, hd = out["O"].shape
    O = out["O"].transpose(1, 2).reshape(B, L, H * hd)
    dQ = out["dQ"].transpose(1, 2).reshape(B, L, H * hd)
    tol = 1e-4                                     # fp32-mode tolerance: 1e-4 relative
    assert rel_err(O, g["O"]) < tol
    assert rel_err(dQ, g["dQ"]) < tol
    assert rel_err(dense_grads_from_listed(inp, out["dE_k"], g["used"]), g["dE_k_used"]) < tol
    assert rel_err(dense_grads_from_listed(inp, out["dE_v"], g["used"]), g["dE_v_used"]) < tol
    assert rel_err(out["dW_pe"].t(), g["dW_dn"]) < tol


def test_flash_listed_only_differs_from_full_vocab():
    g = load_golden("flash_ref_silu.npz")
    inp = listed_from_dense(g)
    a = orc.flash_ema(inp["Q"], inp["x"], inp["E_k"], inp["E_v"], inp["W_pe"], inp["rhos"], inp["V"], inp["unique"])
    b = orc.flash_ema(inp["Q"], inp["x"], inp["E_k"], inp["E_v"], inp["W_pe"], inp["rhos"], inp["V"], inp["unique"],
                      inactive_mass="listed_only")
    assert rel_err(a["O"], b["O"]) > 1e-2


@pytest.mark.parametrize("name", ["gate_ref_silu.npz", "gate_ref_linear.npz"])
def test_gating_oracle_matches_reference_fixture(name):
    g = load_golden(name)
    t = {k: torch.from_numpy(v) for k, v in g.items() if v.ndim > 0}
    out = orc.query_gating(t["x_q"], t["C_seq"], t["W_dn"], t["ln_w"], t["ln_b"], bool(int(g["use_silu"])), dY=t["dY"])
    for k in ("Y", "dx_q", "dW_dn", "dln_w", "dln_b"):
        ok = "dW_pe" if k == "dW_dn" else k
        assert rel_err(out[ok], g[k]) < 1e-5, k
    # inner operator (pre-activation as an input) must agree with the fused form
    bias = t["W_dn"].sum(1)
    p_pre = t["C_seq"] @ t["W_dn"].t()
    inner = orc.gating_from_ppre(t["x_q"], p_pre, bias, t["ln_w"], t["ln_b"], bool(int(g["use_silu"])), dY=t["dY"])
    assert rel_err(inner["Y"], g["Y"]) < 1e-5
    assert rel_err(inner["dx_q"], g["dx_q"]) < 1e-5


def test_rhos_definition():
    r = orc.make_rhos(64, 1024.0, 4096.0)
    assert abs(float(r[0]) - 2 ** (-1 / 1024)) < 1e-7 and abs(float(r[-1]) - 2 ** (-1 / 4096)) < 1e-7


def test_decode_step_equals_dense_loop():
    torch.manual_seed(0)
    B, V, N, D, H = 2, 30, 8, 32, 2
    hd = D // H
    rhos = orc.make_rhos(N, 2.0, 32.0)
    E = torch.randn(V, D) * 0.5
    W = torch.randn(N, D) * 0.5
    L = 12
    x = torch.randint(0, V, (B, L))
    Q = torch.randn(B, H, L, hd) * 0.5
    uniq = torch.arange(V).unsqueeze(0).expand(B, -1).contiguous()
    ref = orc.flash_ema(Q, x, E.expand(B, -1, -1), E.expand(B, -1, -1), W, rhos, V, uniq)
    Cq_ref = orc.query_scan(x, rhos, V)
    state = torch.zeros(B, V, N)
    last = torch.full((B, V), -1, dtype=torch.long)
    for t in range(L):
        O, Cq = orc.decode_step(state, last, t, x[:, t], Q[:, :, t], E, E, W, rhos, V)
        assert rel_err(O, ref["O"][:, :, t]) < 1e-5
        assert torch.allclose(Cq, Cq_ref[:, t], atol=1e-5)
