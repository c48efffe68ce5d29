"""Chunked tied lm_head + masked cross-entropy.

The reference computes `logits = lm_head(final_norm(x_q))` for all B*T positions (mathbrain/model.py:185-186: [B*T, V]
= 2.9 GB in bf16 at the 46M configuration) and then `F.cross_entropy(..., ignore_index=-100)` (train.py:320-323), in which
the padded positions are thrown away.  Here only the VALID rows are projected, a chunk of rows at a time: a library GEMM
fills a [chunk, V] buffer, `mbema_ce_rows` turns it into the rows' losses and, in place, into dlogits, and two more GEMMs
take it to `dh` and `dE`; the buffer is reused by the next chunk, so the full logits never exist and masked positions
cost nothing.  Forward and backward run together (the loss is a scalar whose gradient scales dh and dE).
"""
import torch

from . import _lib
from .ops import _dt, _ptr, _require_cuda, _stream


class LMHeadCrossEntropy(torch.autograd.Function):
    """loss = mean over valid rows of CE(h @ E^T, targets); rows with targets == ignore_index are skipped.

    forward(h [R, D], E [V, D] (the tied embedding / lm_head weight), targets [R] int64, ignore_index=-100,
            chunk_rows=4096) -> scalar float32.  Gradients reach h and E.  The GEMMs run in h's dtype (bf16 under
    autocast, else the dtype of h)."""

    @staticmethod
    def forward(ctx, h, E, targets, ignore_index=-100, chunk_rows=4096):
        _require_cuda(h, E, targets)
        lib = _lib.load()
        with torch.cuda.device(h.device):
            cdt = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else h.dtype
            if cdt not in (torch.float32, torch.bfloat16):
                cdt = torch.float32
            R, D = h.shape
            V = E.shape[0]
            ld = (V + 7) // 8 * 8
            valid = (targets != ignore_index).nonzero(as_tuple=True)[0]          # positions that count
            n = int(valid.numel())                                              # one host synchronisation per step
            dh = torch.zeros(R, D, dtype=torch.float32, device=h.device)
            dE = torch.zeros(ld, D, dtype=torch.float32, device=h.device)
            loss = torch.zeros((), dtype=torch.float32, device=h.device)
            if n:
                Ep = torch.zeros(ld, D, dtype=cdt, device=h.device)             # rows [V, ld) stay zero
                Ep[:V] = E.detach().to(cdt)
                hv = h.detach().index_select(0, valid).to(cdt)
                tv = targets.index_select(0, valid).contiguous()
                rows = min(int(chunk_rows), n)
                buf = torch.empty(rows, ld, dtype=cdt, device=h.device)
                loss_rows = torch.empty(n, dtype=torch.float32, device=h.device)
                for lo in range(0, n, rows):
                    hi = min(lo + rows, n)
                    logits = buf[:hi - lo]
                    torch.mm(hv[lo:hi], Ep.t(), out=logits)
                    rc = lib.mbema_ce_rows(_ptr(logits), _dt(logits), _ptr(tv[lo:hi]), 1.0 / n, _ptr(loss_rows[lo:hi]),
                                           hi - lo, V, ld, _stream())
                    _lib.check(rc, "mbema_ce_rows")
                    dh.index_copy_(0, valid[lo:hi], torch.mm(logits, Ep).float())
                    if cdt == torch.float32:
                        dE.addmm_(logits.t(), hv[lo:hi])
                    else:
                        dE.add_(torch.mm(logits.t(), hv[lo:hi]).float())
                loss = loss_rows.sum() / n
        ctx.save_for_backward(dh.to(h.dtype), dE[:V].to(E.dtype))
        return loss

    @staticmethod
    def backward(ctx, g):
        dh, dE = ctx.saved_tensors
        return dh * g, dE * g, None, None, None


def lm_head_cross_entropy(h, E, targets, ignore_index=-100, chunk_rows=4096):
    """Mean cross-entropy of the tied lm_head over the positions whose target is not `ignore_index`; h [..., D],
    targets [...] int64 (same leading shape)."""
    return LMHeadCrossEntropy.apply(h.reshape(-1, h.shape[-1]), E, targets.reshape(-1), ignore_index, chunk_rows)
