"""Parity of the CUDA operators (through the C ABI) with the CPU oracle and the reference fixtures.

Tolerances (norm-wise relative error, helpers.rel_err):
  EMA state                 1e-5   (fp32)
  attention outputs/grads   1e-4   (fp32 mode),  2e-2 (bf16 operands)
"""
import numpy as np
import pytest
import torch

from oracle import ema_oracle as orc
from helpers import load_golden, rel_err, listed_from_dense, dense_grads_from_listed

pytestmark = pytest.mark.gpu

TOL_STATE = 1e-5
TOL_FP32 = 1e-4
TOL_BF16 = 2e-2


@pytest.fixture(scope="module")
def mb():
    import mathbrain_b200 as m
    assert torch.cuda.is_available()
    m._lib.load()
    m.set_options(inactive_mass="full_V", cbase_extra_decay=False, mode="fp32")
    return m


def cu(t):
    return t.cuda() if t is not None else None


# ------------------------------------------------------------------------------------------ scan
@pytest.mark.parametrize("name", ["scan_ref_a.npz", "scan_ref_docs.npz"])
def test_scan_reference_fixture(mb, name):
    g = load_golden(name)
    x = torch.from_numpy(g["x"])
    rhos = torch.from_numpy(g["rhos"])
    doc = torch.from_numpy(g["doc_ids"]) if g["doc_ids"].size else None
    C = mb.compute_query_ema_history(cu(x), cu(rhos), int(g["V"]), cu(torch.from_numpy(g["c_init"])),
                                     cu(torch.from_numpy(g["keys"])), cu(doc))
    assert rel_err(C.cpu(), g["C_seq"]) < TOL_STATE
    C2 = mb.compute_query_ema_history(cu(x), cu(rhos), int(g["V"]), doc_ids=cu(doc))
    assert rel_err(C2.cpu(), g["C_seq_nokeys"]) < TOL_STATE


def test_scan_known_answers(mb):
    # closed forms of the reference's tests/test_doc_boundary.py:75-134
    x = torch.tensor([[0, 1, 0, 2, 0, 1]]).cuda()
    rhos = torch.tensor([0.9, 0.5]).cuda()
    C = mb.compute_query_ema_history(x, rhos, 3).cpu()
    r = rhos.cpu()
    assert torch.allclose(C[0, 0], torch.zeros(2))
    assert torch.allclose(C[0, 2], r ** 2, atol=1e-6)
    assert torch.allclose(C[0, 4], (r ** 2 + 1.0) * r ** 2, atol=1e-6)
    c_init = torch.tensor([[[2.0, 1.5], [0.0, 0.0], [0.0, 0.0]]]).cuda()
    keys = torch.tensor([[0, 1, 2]]).cuda()
    C = mb.compute_query_ema_history(torch.tensor([[0, 1, 0, 2]]).cuda(), rhos, 3, c_init, keys).cpu()
    assert torch.allclose(C[0, 0], torch.tensor([2.0, 1.5]))


@pytest.mark.parametrize("T,N,bursty", [(1, 4, False), (37, 1, False), (512, 64, False), (1024, 128, True), (3000, 33, True)])
def test_scan_vs_oracle(mb, T, N, bursty):
    from mathbrain_b200 import synth
    b = synth.make_chunk_batch(11 + T, B=3, T=T, N=N, vocab=2000, max_prefix=300, min_fill=max(1, T // 2),
                               bursty=bursty, min_hl=2.0, max_hl=512.0)
    ref = orc.query_scan(b["x"], b["rhos"], b["vocab"], b["c_base"], b["unique_slots"], dtype=torch.float64)
    # keys padded with 0 like the collate function does: the first entry of a repeated key must win
    C = mb.compute_query_ema_history(cu(b["x"]), cu(b["rhos"]), b["vocab"], cu(b["c_base"]), cu(b["unique_slots"]))
    assert rel_err(C.cpu(), ref) < TOL_STATE


def test_scan_empty_batch(mb):
    C = mb.compute_query_ema_history(torch.zeros(0, 8, dtype=torch.long).cuda(), torch.ones(4).cuda() * 0.9, 10)
    assert C.shape == (0, 8, 4)


# ------------------------------------------------------------------------------------------ snapshots
@pytest.mark.parametrize("T,N,extra", [(5, 4, False), (128, 16, False), (300, 64, True), (700, 128, False)])
def test_tile_states_vs_oracle(mb, T, N, extra):
    from mathbrain_b200 import synth
    b = synth.make_chunk_batch(5 + T, B=2, T=T, N=N, vocab=300, max_prefix=100, min_fill=max(1, T - 3),
                               min_hl=1.0, max_hl=256.0)
    unique = b["unique_slots"].clone()
    unique[~b["pad_mask"]] = -1
    unique[0, 1] = -1                      # a hole in the slot list
    with mb.options(cbase_extra_decay=extra):
        h = mb.precompute_boundaries(cu(b["x"]), cu(unique), cu(b["rhos"]), 64, c_init=cu(b["c_base"]))
    ref = orc.tile_start_states(b["x"], unique, b["rhos"], 128, b["c_base"], extra_decay=extra, dtype=torch.float64)
    assert h.tile_state.shape == ref.shape
    assert rel_err(h.tile_state.cpu(), ref) < TOL_STATE
    assert h.kcount[:2].cpu().tolist() == (unique >= 0).sum(1).tolist()
    order = h.kcount[2:].cpu().tolist()
    assert sorted(order) == [0, 1] and h.kcount[order[0]] >= h.kcount[order[1]]
    M = orc.memory_states(b["x"], unique, b["rhos"], b["c_base"], extra_decay=extra, dtype=torch.float64)
    tok = h.tok_state.cpu()
    for bb in range(2):
        for t in range(T):
            hit = (unique[bb] == b["x"][bb, t]).nonzero()
            if hit.numel():
                assert rel_err(tok[bb, t], M[bb, t, int(hit[0])]) < 1e-4 or float(M[bb, t, int(hit[0])].abs().max()) < 1e-6


# ------------------------------------------------------------------------------------------ query gate
@pytest.mark.parametrize("name", ["gate_ref_silu.npz", "gate_ref_linear.npz"])
def test_gating_reference_fixture(mb, name):
    g = load_golden(name)
    t = {k: torch.from_numpy(v).cuda() for k, v in g.items() if v.ndim > 0}
    silu = bool(int(g["use_silu"]))
    D, N = t["W_dn"].shape
    pe = torch.nn.Linear(N, D, bias=False).cuda()
    ln = torch.nn.LayerNorm(D).cuda()
    with torch.no_grad():
        pe.weight.copy_(t["W_dn"]); ln.weight.copy_(t["ln_w"]); ln.bias.copy_(t["ln_b"])
    xq = t["x_q"].clone().requires_grad_(True)
    y = mb.fused_apply_symmetric_query_gating(xq, t["C_seq"], pe, ln, torch.nn.Identity(), silu)
    y.backward(t["dY"])
    assert rel_err(y.detach().cpu(), g["Y"]) < 2e-5
    assert rel_err(xq.grad.cpu(), g["dx_q"]) < 2e-5
    assert rel_err(pe.weight.grad.cpu(), g["dW_dn"]) < 2e-5
    assert rel_err(ln.weight.grad.cpu(), g["dln_w"]) < 2e-5
    assert rel_err(ln.bias.grad.cpu(), g["dln_b"]) < 2e-5


@pytest.mark.parametrize("rows,D,dt", [(1, 4, torch.float32), (77, 512, torch.float32), (300, 1024, torch.float32),
                                       (64, 512, torch.bfloat16), (5, 192, torch.float32)])
def test_gating_inner_operator(mb, rows, D, dt):
    torch.manual_seed(rows + D)
    x = torch.randn(1, rows, D).to(dt); p = (torch.randn(1, rows, D) * 2).to(dt)
    bias = torch.randn(D); lw = torch.randn(D); lb = torch.randn(D); dy = torch.randn(1, rows, D).to(dt)
    ref = orc.gating_from_ppre(x.float(), p.float(), bias, lw, lb, True, dY=dy.float(), dtype=torch.float64)
    leaves = [v.cuda().requires_grad_(True) for v in (x, p, bias, lw, lb)]
    y = mb.FusedGatingFunction.apply(*leaves, True)
    y.backward(dy.cuda().float())
    tol = 2e-5 if dt == torch.float32 else 1e-2      # bf16 gradients are rounded to bf16 on return
    assert rel_err(y.detach().cpu(), ref["Y"]) < 2e-5
    for leaf, k in zip(leaves, ("dx_q", "dp_pre", "dbias", "dln_w", "dln_b")):
        assert rel_err(leaf.grad.float().cpu(), ref[k]) < tol, k


# ------------------------------------------------------------------------------------------ attention
def run_flash(mb, inp, c_base=None, seq_lens=None, dtype=torch.float32, with_grad=True):
    Q = cu(inp["Q"]).to(dtype).requires_grad_(with_grad)
    Ek = cu(inp["E_k"]).to(dtype).requires_grad_(with_grad)
    Ev = cu(inp["E_v"]).to(dtype).requires_grad_(with_grad)
    W = cu(inp["W_pe"]).requires_grad_(with_grad)
    x = cu(inp["x"]); unique = cu(inp["unique"]); rhos = cu(inp["rhos"])
    h = mb.precompute_boundaries(x, unique, rhos, 64, c_init=cu(c_base), seq_lens=cu(seq_lens))
    O = mb.FlashEMAFunction.apply(Q, x, Ek, Ev, W, rhos, inp["V"], unique, unique.shape[1], h, inp["use_silu"])
    out = {"O": O.detach().cpu()}
    if with_grad:
        O.backward(cu(inp["dO"]).float())
        out.update(dQ=Q.grad.float().cpu(), dE_k=Ek.grad.float().cpu(), dE_v=Ev.grad.float().cpu(), dW_pe=W.grad.cpu())
    return out


@pytest.mark.parametrize("name", ["flash_ref_silu.npz", "flash_ref_linear.npz", "flash_ref_small_w.npz"])
def test_flash_reference_fixture(mb, name):
    g = load_golden(name)
    inp = listed_from_dense(g)
    if inp["hd"] != 64:
        pytest.skip("head_dim 64 only")
    out = run_flash(mb, inp)
    B, H, L, hd = out["O"].shape
    O = out["O"].transpose(1, 2).reshape(B, L, H * hd)
    dQ = out["dQ"].transpose(1, 2).reshape(B, L, H * hd)
    assert rel_err(O, g["O"]) < TOL_FP32
    assert rel_err(dQ, g["dQ"]) < TOL_FP32
    assert rel_err(dense_grads_from_listed(inp, out["dE_k"], g["used"]), g["dE_k_used"]) < TOL_FP32
    assert rel_err(dense_grads_from_listed(inp, out["dE_v"], g["used"]), g["dE_v_used"]) < TOL_FP32
    assert rel_err(out["dW_pe"].t(), g["dW_dn"]) < TOL_FP32


def make_case(seed, B, T, N, H, vocab, max_prefix, min_hl, max_hl, std=0.3, bursty=False, min_fill=None, holes=True):
    from mathbrain_b200 import synth
    b = synth.make_chunk_batch(seed, B=B, T=T, N=N, vocab=vocab, max_prefix=max_prefix,
                               min_fill=min_fill if min_fill is not None else max(1, T // 2), bursty=bursty,
                               min_hl=min_hl, max_hl=max_hl)
    unique = b["unique_slots"].clone()
    unique[~b["pad_mask"]] = -1
    c_base = b["c_base"].clone()
    if holes and unique.shape[1] > 3:
        unique[0, 2] = -1
    D = 64 * H
    w = synth.make_layer_weights(seed + 1, B, unique.shape[1], D, N, T, H, std=std)
    inp = dict(x=b["x"], unique=unique, rhos=b["rhos"], V=vocab, use_silu=True, **w)
    return inp, c_base, b["fill"]


def oracle_flash(inp, c_base, **kw):
    return orc.flash_ema(inp["Q"].float(), inp["x"], inp["E_k"].float(), inp["E_v"].float(), inp["W_pe"], inp["rhos"],
                         inp["V"], inp["unique"], c_base=c_base, use_silu=inp["use_silu"], dO=inp["dO"].float(), **kw)


def compare_all(out, ref, tol, rows=None):
    for k in ("O", "dQ", "dE_k", "dE_v", "dW_pe"):
        a, b = out[k], ref[k]
        if rows is not None and k in ("O", "dQ"):
            for bb, n in enumerate(rows):
                assert rel_err(a[bb, :, :n], b[bb, :, :n]) < tol, (k, bb)
        else:
            assert rel_err(a, b) < tol, k


@pytest.mark.parametrize("T,N,H", [(1, 4, 1), (63, 16, 2), (200, 64, 2), (130, 128, 1), (384, 33, 1)])
def test_flash_vs_oracle_with_c_base(mb, T, N, H):
    inp, c_base, _ = make_case(100 + T, B=2, T=T, N=N, H=H, vocab=400, max_prefix=150, min_hl=1.0, max_hl=300.0)
    out = run_flash(mb, inp, c_base)
    ref = oracle_flash(inp, c_base)
    compare_all(out, ref, TOL_FP32)


def test_flash_hot_slots_bursty(mb):
    # many repeats inside a tile: exercises the in-tile restart of a slot's state
    inp, c_base, _ = make_case(7, B=2, T=260, N=16, H=1, vocab=12, max_prefix=40, min_hl=1.0, max_hl=64.0, bursty=True,
                               holes=False)
    out = run_flash(mb, inp, c_base)
    ref = oracle_flash(inp, c_base)
    compare_all(out, ref, TOL_FP32)


def test_flash_semantic_switches(mb):
    inp, c_base, _ = make_case(21, B=2, T=150, N=16, H=1, vocab=200, max_prefix=100, min_hl=2.0, max_hl=100.0)
    with mb.options(inactive_mass="listed_only", cbase_extra_decay=True):
        out = run_flash(mb, inp, c_base)
    ref = oracle_flash(inp, c_base, inactive_mass="listed_only", extra_decay=True)
    compare_all(out, ref, TOL_FP32)
    inp["use_silu"] = False
    out = run_flash(mb, inp, c_base)
    ref = oracle_flash(inp, c_base)
    compare_all(out, ref, TOL_FP32)


def test_flash_seq_lens_skip_padding(mb):
    inp, c_base, fill = make_case(33, B=3, T=300, N=16, H=1, vocab=300, max_prefix=100, min_hl=2.0, max_hl=100.0,
                                  min_fill=20)
    inp["dO"] = inp["dO"].clone()
    for b, n in enumerate(fill.tolist()):
        inp["dO"][b, :, n:] = 0          # padded positions are loss-masked
    out = run_flash(mb, inp, c_base, seq_lens=fill)
    ref = oracle_flash(inp, c_base)
    compare_all(out, ref, TOL_FP32, rows=fill.tolist())
    for b, n in enumerate(fill.tolist()):
        assert float(out["O"][b, :, n:].abs().max() if n < 300 else 0.0) == 0.0


def test_flash_config1_shape_fp32_and_bf16(mb):
    # the CPU-reference configuration: B=2, T=128, V=50257, D=512, H=8, N=64, half-lives 1024..4096, c_base=0
    from mathbrain_b200 import synth
    rng = np.random.Generator(np.random.PCG64(0))
    x = torch.from_numpy(np.stack([synth.Zipf().draw(rng, 128) for _ in range(2)]))
    unique, K = orc.build_unique_index(x)
    g = torch.Generator().manual_seed(0)
    E = torch.randn(synth.VOCAB, 512, generator=g) * 0.02
    Ea = E[unique.clamp_min(0)] * (unique >= 0).unsqueeze(-1)
    inp = dict(x=x, unique=unique, rhos=synth.make_rhos(64), V=synth.VOCAB, use_silu=True,
               Q=torch.randn(2, 8, 128, 64, generator=g) * 0.02, E_k=Ea, E_v=Ea.clone(),
               W_pe=torch.randn(64, 512, generator=g) * 0.02, dO=torch.randn(2, 8, 128, 64, generator=g) * 0.02)
    ref = oracle_flash(inp, None)
    out = run_flash(mb, inp)
    compare_all(out, ref, TOL_FP32)
    out16 = run_flash(mb, inp, dtype=torch.bfloat16)
    compare_all(out16, ref, TOL_BF16)


def test_flash_chunking_invariance(mb):
    """Size-independent property: one 512-step chunk equals two 256-step chunks whose second half carries the
    slot states of the first (the c_base contract of the data pipeline)."""
    inp, c_base, _ = make_case(55, B=2, T=512, N=64, H=2, vocab=3000, max_prefix=600, min_hl=16.0, max_hl=2048.0,
                               std=0.2, min_fill=512, holes=False)
    full = run_flash(mb, inp, c_base, with_grad=False)["O"]
    M = orc.memory_states(inp["x"], inp["unique"], inp["rhos"], c_base, dtype=torch.float64)
    halves = []
    for s in (0, 256):
        part = dict(inp)
        part["x"] = inp["x"][:, s:s + 256].contiguous()
        part["Q"] = inp["Q"][:, :, s:s + 256].contiguous()
        halves.append(run_flash(mb, part, M[:, s].float(), with_grad=False)["O"])
    assert rel_err(torch.cat(halves, 2), full) < TOL_FP32


def test_flash_slot_order_invariance(mb):
    inp, c_base, _ = make_case(77, B=1, T=140, N=16, H=1, vocab=200, max_prefix=80, min_hl=2.0, max_hl=64.0)
    a = run_flash(mb, inp, c_base)
    perm = torch.randperm(inp["unique"].shape[1], generator=torch.Generator().manual_seed(1))
    inp2 = dict(inp)
    inp2["unique"] = inp["unique"][:, perm].contiguous()
    inp2["E_k"] = inp["E_k"][:, perm].contiguous()
    inp2["E_v"] = inp["E_v"][:, perm].contiguous()
    b = run_flash(mb, inp2, c_base[:, perm].contiguous())
    assert rel_err(b["O"], a["O"]) < 1e-5
    assert rel_err(b["dE_k"], a["dE_k"][:, perm]) < 1e-4
    assert rel_err(b["dW_pe"], a["dW_pe"]) < 1e-4


def test_build_unique_index(mb):
    x = torch.randint(0, 50, (4, 64), generator=torch.Generator().manual_seed(0))
    u, k = mb._build_unique_index(x.cuda(), "cuda")
    ur, kr = orc.build_unique_index(x)
    assert k == kr and torch.equal(u.cpu(), ur)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_slot_grad_scatter_matches_embedding_backward(mb, dtype):
    """out[token] += dE_k + dE_v per listed slot: against autograd's backward of F.embedding over the same slot lists
    (mathbrain/model.py:63-64), with padded entries (-1), tokens listed by several samples and a second accumulating
    call."""
    g = torch.Generator().manual_seed(11)
    B, K, D, V = 5, 37, 64, 90
    unique = torch.randint(0, V, (B, K), generator=g)
    unique[:, 30:] = -1
    unique[2, 5] = -1
    dEk = torch.randn(B, K, D, generator=g).to(dtype)
    dEv = torch.randn(B, K, D, generator=g).to(dtype)
    E = torch.zeros(V, D, dtype=torch.float64, requires_grad=True)
    rows = torch.nn.functional.embedding(unique.clamp_min(0), E)
    mask = (unique >= 0).unsqueeze(-1).double()
    (rows * (dEk.double() + dEv.double()) * mask).sum().backward()
    out = torch.zeros(V, D, device="cuda")
    mb.slot_grad_scatter(dEk.cuda(), dEv.cuda(), unique.cuda(), out)
    assert rel_err(out.cpu(), E.grad) < 1e-6
    mb.slot_grad_scatter(dEk.cuda(), None, unique.cuda(), out)          # accumulates; dE_v optional
    E2 = torch.zeros(V, D, dtype=torch.float64, requires_grad=True)
    (torch.nn.functional.embedding(unique.clamp_min(0), E2) * dEk.double() * mask).sum().backward()
    assert rel_err(out.cpu(), E.grad + E2.grad) < 1e-6
    with pytest.raises(mb._lib.MbemaError):
        mb.slot_grad_scatter(dEk[..., :60].cuda(), None, unique.cuda(), torch.zeros(V, 60, device="cuda"))   # D % 8


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1e-2)])
def test_slot_rows_projection_matches_the_per_sample_reference(mb, dtype, tol):
    """embedding -> ln_kv -> k_proj / v_proj over the DISTINCT tokens of a batch (project_slot_rows) against the
    reference's per-sample formulation (mathbrain/model.py:63-68) in float64: the gathered rows are the same values,
    and the gradients of E, ln_kv, k_proj and v_proj are those of the per-sample graph."""
    g = torch.Generator().manual_seed(21)
    B, K, D, V = 4, 23, 128, 60
    unique = torch.randint(0, V, (B, K), generator=g)
    for b in range(B):                                    # distinct within a sample, like a slot list
        unique[b] = torch.randperm(V, generator=g)[:K]
    unique[:, 19:] = -1
    E = torch.randn(V, D, generator=g)
    ln = torch.nn.LayerNorm(D)
    kp, vp = torch.nn.Linear(D, D, bias=False), torch.nn.Linear(D, D, bias=False)
    with torch.no_grad():
        ln.weight.copy_(1 + 0.1 * torch.randn(D, generator=g))
        ln.bias.copy_(0.1 * torch.randn(D, generator=g))
    Rk, Rv = torch.randn(B, K, D, generator=g), torch.randn(B, K, D, generator=g)
    mask = (unique >= 0).unsqueeze(-1)

    def loss_of(Ek_act, Ev_act):
        return ((Ek_act * Rk.to(Ek_act)) + (Ev_act * Rv.to(Ek_act))).mul(mask.to(Ek_act.device)).sum()

    # reference: per sample, float64, on the CPU
    E64 = E.double().requires_grad_(True)
    ln64, kp64, vp64 = (torch.nn.LayerNorm(D).double(), torch.nn.Linear(D, D, bias=False).double(),
                        torch.nn.Linear(D, D, bias=False).double())
    ln64.load_state_dict(ln.state_dict()); kp64.load_state_dict(kp.state_dict()); vp64.load_state_dict(vp.state_dict())
    mem = ln64(torch.nn.functional.embedding(unique.clamp_min(0), E64))
    ref_k, ref_v = kp64(mem), vp64(mem)
    loss_of(ref_k, ref_v).backward()

    dev = "cuda"
    Ed = E.to(dev).requires_grad_(True)
    ln, kp, vp = ln.to(dev), kp.to(dev), vp.to(dev)
    tokens, row_index = mb.shared_slot_rows(unique.to(dev))
    with torch.autocast("cuda", dtype=torch.bfloat16, enabled=(dtype == torch.bfloat16)):
        Ek_rows, Ev_rows = mb.project_slot_rows(Ed, tokens, ln, kp, vp)
        assert Ek_rows.dtype == dtype and Ek_rows.shape == (tokens.numel(), D)
        Ek_act, Ev_act = Ek_rows[row_index.long()], Ev_rows[row_index.long()]       # what the attention kernel gathers
        Rk, Rv = Rk.to(dev), Rv.to(dev)
        loss_of(Ek_act.float(), Ev_act.float()).backward()
    m = mask.expand(-1, -1, D)
    assert rel_err(Ek_act.detach().float().cpu()[m], ref_k.detach()[m]) < tol
    assert rel_err(Ev_act.detach().float().cpu()[m], ref_v.detach()[m]) < tol
    assert rel_err(Ed.grad.cpu(), E64.grad) < tol
    assert rel_err(ln.weight.grad.cpu(), ln64.weight.grad) < tol and rel_err(ln.bias.grad.cpu(), ln64.bias.grad) < tol
    assert rel_err(kp.weight.grad.cpu(), kp64.weight.grad) < tol and rel_err(vp.weight.grad.cpu(), vp64.weight.grad) < tol


@pytest.mark.parametrize("N,with_docs", [(64, False), (33, True), (128, True), (4, False)])
def test_scan_long_chains(mb, N, with_docs):
    """Chains of hundreds of occurrences (a vocabulary of a few tokens, runs of one token as in the padding, half-lives
    from one step to thousands): the warp-shuffle segmented scan of long chains against the oracle, with listed keys,
    without, and across document boundaries."""
    from mathbrain_b200 import synth
    g = torch.Generator().manual_seed(N)
    B, T, V = 3, 700, 5
    x = torch.randint(0, V, (B, T), generator=g)
    x[0, 300:] = 0                                         # a run of 400 repeats (gaps of one step)
    x[1, ::2] = 3                                          # gaps of two
    rhos = synth.make_rhos(N, 1.0, 4096.0)
    keys = torch.tensor([[0, 1, 2, 3, 4, 0, 0], [4, 3, -1, 1, 0, 2, 0], [2, -1, -1, -1, -1, -1, -1]])
    c_init = torch.rand(B, 7, N, generator=g) * 3.0
    doc = None
    if with_docs:
        doc = torch.zeros(B, T, dtype=torch.long)
        doc[0, 350:] = 1
        doc[1, 100:] = 1
        doc[1, 433:] = 2
    ref = orc.query_scan(x, rhos, V, c_init, keys, doc_ids=doc, dtype=torch.float64)
    C = mb.compute_query_ema_history(cu(x), cu(rhos), V, cu(c_init), cu(keys), cu(doc))
    assert rel_err(C.cpu(), ref) < TOL_STATE
    ref0 = orc.query_scan(x, rhos, V, doc_ids=doc, dtype=torch.float64)
    C0 = mb.compute_query_ema_history(cu(x), cu(rhos), V, doc_ids=cu(doc))
    assert rel_err(C0.cpu(), ref0) < TOL_STATE


def test_snapshots_reuse_the_scan_index(mb):
    """precompute_boundaries right after compute_query_ema_history on the same chunk reuses the token order the scan left
    in its workspace (only the key links are rebuilt, for a different key list): same snapshots as a call of its own; a
    chunk modified in place, or another chunk, is sorted afresh."""
    from mathbrain_b200 import synth
    b = synth.make_chunk_batch(77, B=3, T=300, N=16, vocab=200, max_prefix=200, min_fill=100, min_hl=2.0, max_hl=200.0)
    x, rhos, c_base = cu(b["x"]), cu(b["rhos"]), cu(b["c_base"])
    unique = b["unique_slots"].clone()
    unique[~b["pad_mask"]] = -1
    unique = cu(unique)
    mb.ops._index_cache.update(key=None, ws=None, x=None)
    fresh = mb.precompute_boundaries(x, unique, rhos, 64, c_init=c_base)              # sorts by itself
    mb.compute_query_ema_history(x, rhos, b["vocab"], c_base, cu(b["unique_slots"]))   # 0-padded keys: another list
    assert mb.ops._index_cache["key"] == mb.ops._index_key(x)
    reused = mb.precompute_boundaries(x, unique, rhos, 64, c_init=c_base)             # key links only
    assert torch.equal(fresh.tile_state, reused.tile_state) and torch.equal(fresh.tok_state, reused.tok_state)
    assert torch.equal(fresh.kcount, reused.kcount)
    x.add_(1).remainder_(b["vocab"])                                                  # in place: the cached order is stale
    assert mb.ops._index_cache["key"] != mb.ops._index_key(x)
    again = mb.precompute_boundaries(x, unique, rhos, 64, c_init=c_base)
    ref = orc.tile_start_states(x.cpu(), unique.cpu(), b["rhos"], 128, c_base=b["c_base"], dtype=torch.float64)
    nT = ref.shape[1]
    got = again.tile_state.reshape(-1)[: 3 * nT * unique.shape[1] * 16].view(3, nT, unique.shape[1], 16)
    assert rel_err(got.cpu(), ref) < TOL_STATE
