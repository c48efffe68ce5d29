"""One training-step loss of the reference's SlotTransformerLM with the steps around the operators done this library's way.

`model` is an instance of the reference's own class (mathbrain/model.py:121-186); its parameters and sub-modules are
used as they are.  What changes against `model(x, ...)` followed by `F.cross_entropy` (train.py:313-323):

  * the slot K/V rows are gathered, normalised and projected once per DISTINCT token of the batch (project_slot_rows)
    and the attention reads them through a row index (FlashEMARowsFunction), where the model projects
    `[B, K_max, D]` per layer (model.py:63-68);
  * the tied lm_head and the masked cross-entropy run over the valid positions only, a chunk of rows at a time
    (lm_head_cross_entropy), where the model materialises `[B*T, V]` logits (model.py:185-186).

Same mathematics, same parameters, same gradients (checked in tests/test_gpu_hosted_model.py).
"""
import torch

from .lmhead import lm_head_cross_entropy
from .ops import (FlashEMARowsFunction, compute_query_ema_history, fused_apply_symmetric_query_gating,
                  precompute_boundaries, project_slot_rows, shared_slot_rows)


def train_step_loss(model, x, y, unique_slots, c_base, pad_mask, ignore_index=-1):
    """Mean cross-entropy of `model` on the chunk batch (x, y): the value `F.cross_entropy(model(x, unique_slots=...,
    c_base=..., pad_mask=...).view(-1, V), y.view(-1), ignore_index=ignore_index)` has.  Call `.backward()` on it."""
    B, L = x.shape
    E = model.embed.weight
    D = E.shape[1]
    rhos = model.ema_rhos
    x_q = model.embed(x)
    C_seq = compute_query_ema_history(x, rhos, model.vocab_size, c_base, unique_slots)
    if model.ema_dropout > 0 and model.training:
        C_seq = torch.nn.functional.dropout(C_seq, p=model.ema_dropout, training=True)
    unique_tensor = unique_slots.clone()
    unique_tensor[~pad_mask] = -1
    K_max = max(int(pad_mask.sum(dim=1).max()), 16)                # the one host read the model makes too (model.py:169)
    unique_tensor = unique_tensor[:, :K_max].contiguous()
    c_base_kv = c_base[:, :K_max, :] if c_base is not None else None
    C_bounds = precompute_boundaries(x, unique_tensor, rhos, 64, c_init=c_base_kv)
    tokens, row_index = shared_slot_rows(unique_tensor)
    for block in model.layers:
        a = block.attn
        H = a.n_heads
        h_in = block.attn_norm(x_q)
        E_k_rows, E_v_rows = project_slot_rows(E, tokens, a.ln_kv, a.k_proj, a.v_proj)
        Q_t = fused_apply_symmetric_query_gating(h_in, C_seq, a.pe_proj, a.ln_q, a.q_proj, a.use_silu)
        Q_mha = Q_t.view(B, L, H, D // H).transpose(1, 2).contiguous()
        out = FlashEMARowsFunction.apply(Q_mha, x, E_k_rows, E_v_rows, row_index, a.pe_proj.weight.t().contiguous(), rhos,
                                         E.shape[0], unique_tensor, unique_tensor.shape[1], C_bounds, a.use_silu)
        out = out.transpose(1, 2).contiguous().view(B, L, D)
        h = x_q + a.resid_dropout(a.o_proj(out))
        x_q = h + block.ffn(block.ffn_norm(h))
    return lm_head_cross_entropy(model.final_norm(x_q), model.lm_head.weight, y, ignore_index=ignore_index)
