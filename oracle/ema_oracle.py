"""CPU oracle for the Per-Slot-EMA hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain PyTorch on the CPU, the arithmetic of the
reference's Per-Slot-EMA operators.  It exists to check the CUDA kernels; it is
never imported by the product package.  Only the test-suite, the smoke check and
the CPU-baseline leg of the benchmark may import it.

Parity status
-------------
* ``query_scan``            pinned: reproduces the reference's own scan tests
                            (closed-form vectors of tests/test_doc_boundary.py:22-134,
                            the manual recurrence of tests/test_pipeline_thorough.py:191-271)
                            and agrees with ``compute_query_ema_history_pt`` on seeded
                            random inputs (fixtures in tests/golden/).
* ``flash_ema`` fwd / bwd   pinned on outputs of the unmodified reference
                            ``mathbrain/flash_ema_attention.py::flash_ema_forward`` (forward
                            as shipped; backward by plain autograd through the shipped function,
                            given a pe_proj module that clones its input so the in-place state
                            update does not invalidate the saved tensor),
                            committed as tests/golden/flash_ref_*.npz together with the
                            generator.  The reference's own test-suite holds no vector for
                            this operator.
* ``query_gating``          pinned on outputs of the reference's fallback branch
                            (mathbrain/triton_fused_gating.py:187-197), same fixture scheme.

Conventions (all cited to the reference tree)
---------------------------------------------
* decay rates  rho_n = exp(-ln 2 / h_n), h = logspace(min_hl, max_hl, N)   (mathbrain/model.py:128-130)
* memory state seen at chunk step t ("compare -> update -> decay"):
      M_0[k] = c_base[k];  M_{t+1}[k] = rho * (M_t[k] + [x_t == k])
  (mathbrain/data.py:128-140, tests/test_gold_standard.py:196-221,
   mathbrain/flash_ema_attention.py:48,82 with c_base = 0)
* query-side state  C_seq[t] = M_t[x_t]                                   (mathbrain/triton_ema_query.py:94-111)
* gate  G_t[k] = SiLU(M_t[k] @ W_pe),  K = E_k * G,  V = E_v * G          (mathbrain/flash_ema_attention.py:51-59)
* per head: O_t = softmax_k(q_t . K_t[k] / sqrt(hd)) @ V_t over ALL vocabulary slots; a slot that is
  not listed, or whose state is zero, has score 0 and value 0, so it only adds exp(0 - max) to the
  normaliser                                                              (mathbrain/flash_ema_attention.py:76-79)
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------------------
# decay rates
# --------------------------------------------------------------------------------------
def make_rhos(n_scales: int, min_hl: float = 1.0, max_hl: float = 2048.0) -> torch.Tensor:
    """rho_n = exp(-ln2 / h_n) with log-spaced half-lives (mathbrain/model.py:128-130)."""
    half_lives = torch.logspace(math.log10(min_hl), math.log10(max_hl), n_scales)
    return torch.exp(-torch.log(torch.tensor(2.0)) / half_lives)


# --------------------------------------------------------------------------------------
# query-side scan
# --------------------------------------------------------------------------------------
def query_scan(x, rhos, vocab_size, c_init=None, c_init_keys=None, doc_ids=None, dtype=torch.float32):
    """State of token x_t just before step t (mathbrain/triton_ema_query.py:67-117).

    Differences from the reference twin, both deliberate:
      * duplicate keys in ``c_init_keys`` (the collate function pads the key list with token 0,
        mathbrain/data.py:220): the FIRST listed entry wins, where the reference's scatter is
        order-dependent;  key -1 is ignored.
      * ``dtype`` lets the tests run the same recurrence in float64.
    """
    x = x.long()
    B, L = x.shape
    N = rhos.shape[0]
    rhos = rhos.to(dtype)
    C_seq = torch.zeros(B, L, N, dtype=dtype)
    for b in range(B):
        last_t = {}
        last_c = {}
        last_d = {}
        if c_init is not None and c_init_keys is not None:
            keys = c_init_keys[b].tolist()
            for i, k in enumerate(keys):
                if k < 0 or k in last_t:
                    continue
                last_t[k] = 0
                last_c[k] = c_init[b, i].to(dtype).clone()
                if doc_ids is not None:
                    last_d[k] = int(doc_ids[b, 0])
        for t in range(L):
            v = int(x[b, t])
            if v in last_t:
                c = last_c[v] * rhos ** float(t - last_t[v])
                if doc_ids is not None and last_d.get(v, None) != int(doc_ids[b, t]):
                    c = torch.zeros(N, dtype=dtype)
            else:
                c = torch.zeros(N, dtype=dtype)
            if doc_ids is not None:
                last_d[v] = int(doc_ids[b, t])
            C_seq[b, t] = c
            last_c[v] = c + 1.0
            last_t[v] = t
    return C_seq


# --------------------------------------------------------------------------------------
# memory-side (slot-major) state
# --------------------------------------------------------------------------------------
def memory_states(x, unique, rhos, c_base=None, extra_decay=False, dtype=torch.float32):
    """Dense M[b, t, k, :] for the listed slots (tests/test_gold_standard.py:196-221).

    ``extra_decay`` reproduces the Triton kernels' convention, which applies one additional
    decay to the c_base term (mathbrain/triton_flash_ema.py:48-50,185).
    """
    B, L = x.shape
    K = unique.shape[1]
    N = rhos.shape[0]
    rhos = rhos.to(dtype)
    M = torch.zeros(B, L, K, N, dtype=dtype)
    C = torch.zeros(B, K, N, dtype=dtype) if c_base is None else c_base.to(dtype).clone()
    if extra_decay:
        C = C * rhos
    valid = unique >= 0
    C = C * valid.unsqueeze(-1)          # entries that are not slots carry no state
    for t in range(L):
        M[:, t] = C
        match = ((unique == x[:, t:t + 1]) & valid).to(dtype)
        C = (C + match.unsqueeze(-1)) * rhos
    return M


def tile_start_states(x, unique, rhos, tile, c_base=None, extra_decay=False, dtype=torch.float32):
    """State of every listed slot at the first step of each ``tile``-step time tile
    (the role of mathbrain/triton_flash_ema.py:29-113)."""
    M = memory_states(x, unique, rhos, c_base, extra_decay, dtype)
    return M[:, ::tile].contiguous()


# --------------------------------------------------------------------------------------
# flash-EMA attention, listed-slot form, forward + backward
# --------------------------------------------------------------------------------------
def flash_ema(Q, x, E_k, E_v, W_pe, rhos, V_total, unique, c_base=None, use_silu=True,
              inactive_mass="full_V", extra_decay=False, dO=None, dtype=torch.float32,
              round_bf16=False):
    """Flash-EMA gated cross-attention over the listed slots of every sample.

    Follows mathbrain/flash_ema_attention.py:46-82 one timestep at a time; the state is kept outside
    autograd and each step's graph is built from the leaf parameters, so the backward runs (the
    shipped function's in-place state update prevents it).

    Q        [B, H, L, hd]     E_k, E_v [B, K, D]     W_pe [N, D]     unique [B, K] (-1 = not a slot)
    inactive_mass: "full_V"     softmax over all V_total slots: the V_total - K_b unlisted slots enter
                                with score 0, value 0 (the PyTorch reference's behaviour)
                   "listed_only" softmax over listed valid slots only (what the Triton kernel computes)
    round_bf16: round the state and W_pe to bf16 before the gate product (the precision the tensor-core
                path computes the gate GEMM in); everything else stays in ``dtype``.
    Returns dict(O, LSE) and, when dO is given, dQ, dE_k, dE_v, dW_pe.
    """
    B, H, L, hd = Q.shape
    K = unique.shape[1]
    D = H * hd
    N = rhos.shape[0]
    scale = 1.0 / math.sqrt(hd)
    valid = unique >= 0                                   # [B, K]
    kb = valid.sum(1)                                     # [B]
    need_grad = dO is not None

    Qd = Q.detach().to(dtype)
    Ek = E_k.detach().to(dtype).clone().requires_grad_(need_grad)
    Ev = E_v.detach().to(dtype).clone().requires_grad_(need_grad)
    W = W_pe.detach().to(dtype).clone().requires_grad_(need_grad)
    rh = rhos.to(dtype)

    C = torch.zeros(B, K, N, dtype=dtype) if c_base is None else c_base.detach().to(dtype).clone()
    if extra_decay:
        C = C * rh

    O = torch.zeros(B, H, L, hd, dtype=dtype)
    LSE = torch.zeros(B, H, L, dtype=dtype)
    dQ = torch.zeros(B, H, L, hd, dtype=dtype) if need_grad else None

    for t in range(L):
        q_t = Qd[:, :, t, :].clone().requires_grad_(need_grad)          # [B, H, hd]
        Cg = C
        Wg = W
        if round_bf16:
            Cg = C.to(torch.bfloat16).to(dtype)
            Wg = W + (W.detach().to(torch.bfloat16).to(dtype) - W.detach())
        pre = Cg @ Wg                                                    # [B, K, D]
        gate = F.silu(pre) if use_silu else pre
        Kt = (Ek * gate).view(B, K, H, hd)
        Vt = (Ev * gate).view(B, K, H, hd)
        s = torch.einsum("bhd,bkhd->bhk", q_t, Kt) * scale               # [B, H, K]
        s = s.masked_fill(~valid.unsqueeze(1), float("-inf"))
        if inactive_mass == "full_V":
            rest = (V_total - kb).to(dtype).clamp_min(0.0)               # [B]
            m = torch.clamp(s.max(dim=-1).values, min=0.0).detach()
            m = torch.where(rest.unsqueeze(1) > 0, m, s.max(dim=-1).values.detach())
            e = torch.exp(s - m.unsqueeze(-1))
            denom = e.sum(-1) + rest.unsqueeze(1) * torch.exp(-m)
        elif inactive_mass == "listed_only":
            m = s.max(dim=-1).values.detach()
            e = torch.exp(s - m.unsqueeze(-1))
            denom = e.sum(-1)
        else:
            raise ValueError(inactive_mass)
        p = e / denom.unsqueeze(-1)                                      # [B, H, K]
        o_t = torch.einsum("bhk,bkhd->bhd", p, Vt)
        O[:, :, t] = o_t.detach()
        LSE[:, :, t] = (m + torch.log(denom)).detach()
        if need_grad:
            grads = torch.autograd.grad(o_t, [q_t, Ek, Ev, W], dO[:, :, t].to(dtype), allow_unused=True)
            dQ[:, :, t] = grads[0]
            for leaf, g in zip((Ek, Ev, W), grads[1:]):
                if g is not None:
                    leaf.grad = g if leaf.grad is None else leaf.grad + g
        match = ((unique == x[:, t:t + 1]) & valid).to(dtype)
        C = (C + match.unsqueeze(-1)) * rh

    out = {"O": O, "LSE": LSE}
    if need_grad:
        out.update(dQ=dQ,
                   dE_k=Ek.grad if Ek.grad is not None else torch.zeros_like(Ek),
                   dE_v=Ev.grad if Ev.grad is not None else torch.zeros_like(Ev),
                   dW_pe=W.grad if W.grad is not None else torch.zeros_like(W))
    return out


# --------------------------------------------------------------------------------------
# fused query gating
# --------------------------------------------------------------------------------------
def query_gating(x_q, C_seq, W_pe_dn, ln_w, ln_b, use_silu=True, eps=1e-5, dY=None, dtype=torch.float32):
    """Q_ln = LayerNorm(x_q * SiLU((C_seq + 1) @ W^T)) * ln_w + ln_b  with W = pe_proj.weight [D, N]
    (mathbrain/triton_fused_gating.py:179-195; the "+1" is the reference's bias W.sum(1)).

    Returns dict(Y) and, when dY is given, dx_q, dW_pe (w.r.t. the [D, N] weight), dln_w, dln_b.
    """
    need = dY is not None
    xq = x_q.detach().to(dtype).clone().requires_grad_(need)
    W = W_pe_dn.detach().to(dtype).clone().requires_grad_(need)
    lw = ln_w.detach().to(dtype).clone().requires_grad_(need)
    lb = ln_b.detach().to(dtype).clone().requires_grad_(need)
    bias = W.sum(dim=1)
    p_lin = C_seq.to(dtype) @ W.t() + bias
    gate = F.silu(p_lin) if use_silu else p_lin
    y = F.layer_norm(xq * gate, (xq.shape[-1],), lw, lb, eps)
    out = {"Y": y.detach()}
    if need:
        g = torch.autograd.grad(y, [xq, W, lw, lb], dY.to(dtype))
        out.update(dx_q=g[0], dW_pe=g[1], dln_w=g[2], dln_b=g[3])
    return out


def gating_from_ppre(x_q, p_pre, bias, ln_w, ln_b, use_silu=True, eps=1e-5, dY=None, dtype=torch.float32):
    """The inner operator of the reference (mathbrain/triton_fused_gating.py:122-177): the gate
    pre-activation is an input.  Returns Y and (dx_q, dp_pre, dbias, dln_w, dln_b)."""
    need = dY is not None
    leaves = [t.detach().to(dtype).clone().requires_grad_(need) for t in (x_q, p_pre, bias, ln_w, ln_b)]
    xq, pp, bb, lw, lb = leaves
    p_lin = pp + bb
    gate = F.silu(p_lin) if use_silu else p_lin
    y = F.layer_norm(xq * gate, (xq.shape[-1],), lw, lb, eps)
    out = {"Y": y.detach()}
    if need:
        g = torch.autograd.grad(y, leaves, dY.to(dtype))
        out.update(dx_q=g[0], dp_pre=g[1], dbias=g[2], dln_w=g[3], dln_b=g[4])
    return out


# --------------------------------------------------------------------------------------
# listed-slot index (fallback when the data loader supplies no slot list)
# --------------------------------------------------------------------------------------
def build_unique_index(x):
    """Per-row sorted unique tokens packed to the front, -1 padding, K_max = max(count, 16)
    (mathbrain/triton_flash_ema.py:475-507)."""
    B, L = x.shape
    rows = [torch.unique(x[b]) for b in range(B)]
    k_max = max(max(r.numel() for r in rows), 16)
    out = torch.full((B, k_max), -1, dtype=x.dtype)
    for b, r in enumerate(rows):
        out[b, : r.numel()] = r
    return out, k_max


# --------------------------------------------------------------------------------------
# streaming decode: one step with resident per-sequence state
# --------------------------------------------------------------------------------------
def decode_step(state, last_t, t_now, tok, q, E_k, E_v, W_pe, rhos, V_total, use_silu=True, dtype=torch.float32):
    """One iteration of the loop body of mathbrain/flash_ema_attention.py:46-82 for a single new token per
    sequence, with the [V, N] state resident and lazily decayed.

    state  [B, V, N]  value of each slot right after its last update (undecayed since then)
    last_t [B, V]     step of that update (-1: never seen; state row is zero)
    t_now  int        current step;  tok [B] the new token;  q [B, H, hd]
    E_k, E_v [V, D]   projected slot embeddings shared by all sequences
    Returns O [B, H, hd], C_q [B, N] (query-side state of ``tok`` before the update); updates state/last_t.
    """
    B, V, N = state.shape
    H, hd = q.shape[1], q.shape[2]
    rh = rhos.to(dtype)
    seen = last_t >= 0
    dt = (t_now - last_t).clamp_min(0).to(dtype)                         # [B, V]
    M = state.to(dtype) * rh.view(1, 1, N) ** dt.unsqueeze(-1)           # state seen at t_now
    M = M * seen.unsqueeze(-1)
    pre = M @ W_pe.to(dtype)                                             # [B, V, D]
    gate = F.silu(pre) if use_silu else pre
    Kt = (E_k.to(dtype).unsqueeze(0) * gate).view(B, V, H, hd)
    Vt = (E_v.to(dtype).unsqueeze(0) * gate).view(B, V, H, hd)
    s = torch.einsum("bhd,bvhd->bhv", q.to(dtype), Kt) / math.sqrt(hd)
    p = torch.softmax(s, dim=-1)
    O = torch.einsum("bhv,bvhd->bhd", p, Vt)
    ar = torch.arange(B)
    C_q = M[ar, tok].clone()
    state[ar, tok] = (C_q + 1.0).to(state.dtype)
    last_t[ar, tok] = t_now
    return O, C_q
