"""Generate the golden fixtures in this directory from the UNMODIFIED reference.

Run once, in a container that has the reference tree (it does not travel to the GPU box):

    python tests/golden/make_golden.py [/path/to/reference]

It imports the reference's own PyTorch code and stores its inputs and outputs:

  scan_ref_*.npz    mathbrain/triton_ema_query.py::compute_query_ema_history_pt
  flash_ref_*.npz   mathbrain/flash_ema_attention.py::flash_ema_forward, forward as shipped; its backward
                    through plain autograd.  The shipped function updates its state tensor in place after
                    pe_proj saved it, which autograd rejects, so the ``pe_proj`` argument handed to it is an
                    nn.Linear whose forward clones its input first (same arithmetic, private saved copy).
                    (torch.autograd.graph.allow_mutation_on_saved_tensors was tried instead and gave a wrong
                    dW_pe with use_silu=False, as central differences of the shipped forward show.)
  gate_ref_*.npz    the fallback branch of mathbrain/triton_fused_gating.py::fused_apply_symmetric_query_gating
                    up to (and excluding) q_proj

The fixtures are small (a few hundred KB in total) so that they can be committed.
"""
import os
import sys

import numpy as np
import torch
import torch.nn as nn

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MATHBRAIN_REFERENCE", "")
if not REF:
    sys.exit("usage: make_golden.py <reference checkout>  (or set MATHBRAIN_REFERENCE)")
sys.path.insert(0, REF)
HERE = os.path.dirname(os.path.abspath(__file__))

from mathbrain.flash_ema_attention import flash_ema_forward          # noqa: E402
from mathbrain.triton_ema_query import compute_query_ema_history_pt  # noqa: E402
from mathbrain.triton_fused_gating import fused_apply_symmetric_query_gating  # noqa: E402


def zipf_tokens(gen, shape, vocab, s=1.1):
    r = torch.arange(1, vocab + 1, dtype=torch.float64)
    p = r ** (-s)
    p = p / p.sum()
    idx = torch.multinomial(p, int(np.prod(shape)), replacement=True, generator=gen)
    return idx.view(*shape)


def make_rhos(n, min_hl, max_hl):
    import math
    hl = torch.logspace(math.log10(min_hl), math.log10(max_hl), n)
    return torch.exp(-torch.log(torch.tensor(2.0)) / hl)


def scan_case(name, seed, B, L, N, V, K, min_hl, max_hl, with_docs):
    g = torch.Generator().manual_seed(seed)
    x = zipf_tokens(g, (B, L), V)
    rhos = make_rhos(N, min_hl, max_hl)
    keys = torch.full((B, K), -1, dtype=torch.long)
    c_init = torch.zeros(B, K, N)
    for b in range(B):
        perm = torch.randperm(V, generator=g)[:K]
        nk = int(torch.randint(K // 2, K + 1, (1,), generator=g))
        keys[b, :nk] = perm[:nk]
        c_init[b, :nk] = torch.rand(nk, N, generator=g) * 3.0
    doc_ids = None
    if with_docs:
        doc_ids = torch.zeros(B, L, dtype=torch.long)
        for b in range(B):
            cut = int(torch.randint(1, L - 1, (1,), generator=g))
            doc_ids[b, cut:] = 1
    ref = compute_query_ema_history_pt(x, rhos, V, c_init=c_init, c_init_keys=keys, doc_ids=doc_ids)
    ref_nokeys = compute_query_ema_history_pt(x, rhos, V, doc_ids=doc_ids)
    np.savez_compressed(os.path.join(HERE, name), x=x.numpy(), rhos=rhos.numpy(), keys=keys.numpy(),
                        c_init=c_init.numpy(), doc_ids=(doc_ids.numpy() if with_docs else np.zeros(0)),
                        V=V, C_seq=ref.numpy(), C_seq_nokeys=ref_nokeys.numpy())


class CloningLinear(nn.Linear):
    """nn.Linear that keeps a private copy of its input for the weight gradient."""

    def forward(self, inp):
        return super().forward(inp.clone())


def flash_case(name, seed, B, L, V, D, H, N, min_hl, max_hl, use_silu, wscale):
    g = torch.Generator().manual_seed(seed)
    x = zipf_tokens(g, (B, L), V)
    rhos = make_rhos(N, min_hl, max_hl)
    E_k = (torch.randn(V, D, generator=g) * wscale).requires_grad_(True)
    E_v = (torch.randn(V, D, generator=g) * wscale).requires_grad_(True)
    pe = CloningLinear(N, D, bias=False)
    with torch.no_grad():
        pe.weight.copy_(torch.randn(D, N, generator=g) * wscale)
    Q = (torch.randn(B, L, D, generator=g) * wscale).requires_grad_(True)
    dO = torch.randn(B, L, D, generator=g) * wscale
    with torch.no_grad():
        O_fwd = flash_ema_forward(Q, x, E_k, E_v, rhos, pe, H, use_silu=use_silu)
    O = flash_ema_forward(Q, x, E_k, E_v, rhos, pe, H, use_silu=use_silu)
    O.backward(dO)
    assert torch.equal(O.detach(), O_fwd)
    # store only the rows of E that appear in the chunk (all other rows have exactly zero gradient)
    used = torch.unique(x)
    assert float(E_k.grad.abs().sum() - E_k.grad[used].abs().sum()) == 0.0
    np.savez_compressed(os.path.join(HERE, name), x=x.numpy(), rhos=rhos.numpy(), V=V, H=H,
                        use_silu=int(use_silu), E_k=E_k.detach().numpy(), E_v=E_v.detach().numpy(),
                        W_dn=pe.weight.detach().numpy(), Q=Q.detach().numpy(), dO=dO.numpy(),
                        O=O.detach().numpy(), dQ=Q.grad.numpy(), used=used.numpy(),
                        dE_k_used=E_k.grad[used].numpy(), dE_v_used=E_v.grad[used].numpy(),
                        dW_dn=pe.weight.grad.numpy())


def gate_case(name, seed, B, L, D, N, use_silu):
    g = torch.Generator().manual_seed(seed)
    x_q = torch.randn(B, L, D, generator=g).requires_grad_(True)
    C_seq = torch.rand(B, L, N, generator=g) * 4.0
    pe = nn.Linear(N, D, bias=False)
    ln = nn.LayerNorm(D)
    with torch.no_grad():
        pe.weight.copy_(torch.randn(D, N, generator=g) * 0.1)
        ln.weight.copy_(1.0 + 0.1 * torch.randn(D, generator=g))
        ln.bias.copy_(0.1 * torch.randn(D, generator=g))
    dY = torch.randn(B, L, D, generator=g)
    ident = nn.Identity()
    y = fused_apply_symmetric_query_gating(x_q, C_seq, pe, ln, ident, use_silu)   # CPU tensors -> fallback branch
    y.backward(dY)
    np.savez_compressed(os.path.join(HERE, name), x_q=x_q.detach().numpy(), C_seq=C_seq.numpy(),
                        W_dn=pe.weight.detach().numpy(), ln_w=ln.weight.detach().numpy(),
                        ln_b=ln.bias.detach().numpy(), dY=dY.numpy(), use_silu=int(use_silu),
                        Y=y.detach().numpy(), dx_q=x_q.grad.numpy(), dW_dn=pe.weight.grad.numpy(),
                        dln_w=ln.weight.grad.numpy(), dln_b=ln.bias.grad.numpy())


if __name__ == "__main__":
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    scan_case("scan_ref_a.npz", 1, B=3, L=96, N=8, V=40, K=24, min_hl=1.0, max_hl=64.0, with_docs=False)
    scan_case("scan_ref_docs.npz", 2, B=2, L=64, N=4, V=12, K=8, min_hl=2.0, max_hl=32.0, with_docs=True)
    flash_case("flash_ref_silu.npz", 3, B=2, L=40, V=96, D=128, H=2, N=16, min_hl=1.0, max_hl=64.0,
               use_silu=True, wscale=0.5)
    flash_case("flash_ref_linear.npz", 4, B=1, L=24, V=64, D=64, H=1, N=8, min_hl=2.0, max_hl=16.0,
               use_silu=False, wscale=0.5)
    flash_case("flash_ref_small_w.npz", 5, B=2, L=32, V=300, D=128, H=2, N=64, min_hl=1024.0, max_hl=4096.0,
               use_silu=True, wscale=0.02)
    gate_case("gate_ref_silu.npz", 6, B=2, L=24, D=128, N=16, use_silu=True)
    gate_case("gate_ref_linear.npz", 7, B=1, L=16, D=64, N=8, use_silu=False)
    print("golden fixtures written to", HERE)
