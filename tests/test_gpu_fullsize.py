"""The BASELINE configurations at their full sizes: the tensor-core path against the fp32 kernels (which the small
cases pin on the oracle and the reference fixtures), plus size-independent properties.  One layer each."""
import pytest
import numpy as np
import torch

from helpers import rel_err

pytestmark = pytest.mark.gpu

TOL_BF16 = 2e-2


@pytest.fixture(scope="module")
def mb():
    import mathbrain_b200
    return mathbrain_b200


def _run(mb, batch, w, mode, fp32_backward=False, dO=None, with_grad=True):
    dev = "cuda"
    unique = batch["unique_slots"].clone()
    unique[~batch["pad_mask"]] = -1
    unique = unique.to(dev)
    x, rhos = batch["x"].to(dev), batch["rhos"].to(dev)
    K = unique.shape[1]
    with mb.options(mode=mode, fp32_backward=fp32_backward):
        Q = w["Q"].to(dev).requires_grad_(with_grad)
        Ek = w["E_k"].to(dev).requires_grad_(with_grad)
        Ev = w["E_v"].to(dev).requires_grad_(with_grad)
        W = w["W_pe"].to(dev).requires_grad_(with_grad)
        h = mb.precompute_boundaries(x, unique, rhos, 64, c_init=batch["c_base"].to(dev))
        O = mb.FlashEMAFunction.apply(Q, x, Ek, Ev, W, rhos, batch["vocab"], unique, K, h, True)
        out = {"O": O.detach().float().cpu()}
        if with_grad:
            O.backward((w["dO"] if dO is None else dO).to(dev).float())
            out.update(dQ=Q.grad.float().cpu(), dE_k=Ek.grad.float().cpu(), dE_v=Ev.grad.float().cpu(), dW_pe=W.grad.float().cpu())
    assert mb.device_status() == 0
    return out


def test_config2_full_size_layer(mb):
    """B=56, T=512, d=512, H=8, N=64, prefixes up to 8192 tokens, fills U(64, 512): tensor-core forward + backward of
    one layer against the fp32 kernels; the backward is linear in dO."""
    from mathbrain_b200 import synth
    batch = synth.make_chunk_batch(2024, 56, 512, 64)
    K = batch["K_max"]
    w = synth.make_layer_weights(7, 56, K, 512, 64, 512, 8, std=0.02, dtype=torch.bfloat16)
    # positions beyond a chunk's fill are loss-masked in training: no gradient enters there (their token-0 state runs
    # into the thousands, where bf16 operands have no meaning)
    steps = torch.arange(512).view(1, 1, 512, 1)
    w["dO"] = w["dO"] * (steps < batch["fill"].view(-1, 1, 1, 1)).to(w["dO"].dtype)
    tc = _run(mb, batch, w, "tc_bf16")
    ref = _run(mb, batch, w, "fp32")
    # slot states reach ~600 after an 8192-token prefix: the gate product runs on fp16 operands (11 significant bits);
    # with bf16 operands dW_pe was off by 2-4.5 % here (the pre-activations moved by ~0.1)
    for k in ref:
        assert torch.isfinite(tc[k]).all(), k
        assert rel_err(tc[k], ref[k]) < TOL_BF16, (k, rel_err(tc[k], ref[k]))
    assert rel_err(tc["O"], ref["O"]) < 3e-3 and rel_err(tc["dW_pe"], ref["dW_pe"]) < 1e-2
    # listed slots beyond a sample's count receive no gradient
    pad = ~batch["pad_mask"]
    assert float(tc["dE_k"][pad].abs().max()) == 0.0 and float(tc["dE_v"][pad].abs().max()) == 0.0
    # linearity: grads(3 dO) = 3 grads(dO) up to the rounding of the bf16 tiles
    tc3 = _run(mb, batch, w, "tc_bf16", dO=3.0 * w["dO"].float())
    for k in ("dQ", "dE_k", "dE_v", "dW_pe"):
        assert rel_err(tc3[k], 3.0 * tc[k]) < 1e-2, k


def test_config3_full_size_layer(mb):
    """Long-chunk stress shape: B=8, T=4096, N=128, bursty repeats.  Forward against the fp32 kernels; the gradients of
    the tensor-core backward against the fp32 backward of the same forward (all within 2e-2)."""
    from mathbrain_b200 import synth
    batch = synth.make_chunk_batch(31, 8, 4096, 128, bursty=True)
    K = batch["K_max"]
    w = synth.make_layer_weights(9, 8, K, 512, 128, 4096, 8, std=0.02, dtype=torch.bfloat16)
    tc = _run(mb, batch, w, "tc_bf16")
    mixed = _run(mb, batch, w, "tc_bf16", fp32_backward=True)
    assert float((tc["O"] - mixed["O"]).abs().max()) == 0.0          # same forward kernel, deterministic
    for k in ("dQ", "dE_k", "dE_v"):
        assert rel_err(tc[k], mixed[k]) < TOL_BF16, (k, rel_err(tc[k], mixed[k]))
    assert rel_err(tc["dW_pe"], mixed["dW_pe"]) < TOL_BF16
    ref = _run(mb, batch, w, "fp32", with_grad=False)
    assert rel_err(tc["O"], ref["O"]) < TOL_BF16


def test_config4_full_size_decode_step(mb):
    """64 sequences, V=50257, N=64, 4096 seen slots each: tensor-core attend against the fp32 kernel, then an update."""
    from mathbrain_b200 import synth
    from mathbrain_b200.decode import DecodeState
    g = torch.Generator().manual_seed(4)
    B, V, N, H, K = 64, synth.VOCAB, 64, 8, 4096
    D = 64 * H
    rhos = synth.make_rhos(N).cuda()
    st = DecodeState(B, V, rhos, capacity=K + 128)
    for b in range(B):
        seen = torch.randperm(V, generator=g)[:K].cuda()
        st.active[b, :K] = seen.to(torch.int32)
        st.last_t[b, seen] = torch.randint(0, 8192, (K,), generator=g).to(torch.int32).cuda()
        st.state[b, seen] = (torch.rand(K, N, generator=g) * 3 + 1).cuda()
    st.n_active.fill_(K)
    E_k = (torch.randn(V, D, generator=g) * 0.02).to(torch.bfloat16).cuda()
    E_v = (torch.randn(V, D, generator=g) * 0.02).to(torch.bfloat16).cuda()
    W = (torch.randn(N, D, generator=g) * 0.02).cuda()
    q = (torch.randn(B, H, 64, generator=g) * 0.02).to(torch.bfloat16).cuda()
    O_tc = st.attend(q, E_k, E_v, W, 8192, mode="tc_bf16")
    O_32 = st.attend(q, E_k, E_v, W, 8192, mode="fp32")
    assert rel_err(O_tc.cpu(), O_32.cpu()) < TOL_BF16
    assert int(st._ws[:4].view(torch.int32).item()) == 0
    tok = torch.randint(0, V, (B,), generator=g).cuda()
    st.update(tok, 8192)
    st.check_overflow()
    assert int(st.n_active.max()) <= K + 1


def _sample_inputs(batch, w, i):
    """Sample i of a batch on its own: its valid slots only, its own prefix state, all T steps."""
    kb = int(batch["pad_mask"][i].sum())
    sub = dict(batch)
    for key in ("x", "fill", "prefix_len"):
        if key in sub and torch.is_tensor(sub[key]) and sub[key].dim() > 0:
            sub[key] = sub[key][i:i + 1]
    sub["unique_slots"] = batch["unique_slots"][i:i + 1, :kb]
    sub["pad_mask"] = batch["pad_mask"][i:i + 1, :kb]
    sub["c_base"] = batch["c_base"][i:i + 1, :kb]
    sub["K_max"] = kb
    ws = {"Q": w["Q"][i:i + 1], "dO": w["dO"][i:i + 1], "E_k": w["E_k"][i:i + 1, :kb], "E_v": w["E_v"][i:i + 1, :kb],
          "W_pe": w["W_pe"]}
    return sub, ws


def _against_oracle(mb, sub, ws, tol):
    from oracle import ema_oracle as orc
    tc = _run(mb, sub, ws, "tc_bf16")
    unique = sub["unique_slots"].clone()
    unique[~sub["pad_mask"]] = -1
    f = lambda t: t.float()
    ref = orc.flash_ema(f(ws["Q"]), sub["x"], f(ws["E_k"]), f(ws["E_v"]), f(ws["W_pe"]), sub["rhos"], sub["vocab"],
                        unique, c_base=sub["c_base"], dO=f(ws["dO"]))
    for k in ("O", "dQ", "dE_k", "dE_v", "dW_pe"):
        assert rel_err(tc[k], ref[k]) < tol, (k, rel_err(tc[k], ref[k]))


def test_config2_samples_against_the_oracle(mb):
    """Whole samples of the full-size 46M batch, each run alone through the tensor-core kernels and through the CPU
    oracle (fp32, all 512 steps, its real prefix state): the samples with the fewest and the most listed slots, the longest
    prefix and the shortest fill.  Everything within 2e-2, dW_pe included (a sample's own contribution)."""
    from mathbrain_b200 import synth
    batch = synth.make_chunk_batch(2024, 56, 512, 64)
    w = synth.make_layer_weights(7, 56, batch["K_max"], 512, 64, 512, 8, std=0.02, dtype=torch.bfloat16)
    steps = torch.arange(512).view(1, 1, 512, 1)
    w["dO"] = w["dO"] * (steps < batch["fill"].view(-1, 1, 1, 1)).to(w["dO"].dtype)       # padded steps are loss-masked
    kb = batch["pad_mask"].sum(1)
    cmax = batch["c_base"].abs().amax(dim=(1, 2))
    picks = {int(kb.argmin()), int(kb.argmax()), int(cmax.argmax()), int(batch["fill"].argmin())}
    assert len(picks) >= 3
    for i in sorted(picks):
        sub, ws = _sample_inputs(batch, w, i)
        _against_oracle(mb, sub, ws, TOL_BF16)


def test_config3_sample_against_the_oracle(mb):
    """One whole sample of the long-chunk batch (T=4096, N=128, bursty repeats) against the CPU oracle."""
    from mathbrain_b200 import synth
    batch = synth.make_chunk_batch(31, 8, 4096, 128, bursty=True)
    w = synth.make_layer_weights(9, 8, batch["K_max"], 512, 128, 4096, 8, std=0.02, dtype=torch.bfloat16)
    steps = torch.arange(4096).view(1, 1, 4096, 1)
    w["dO"] = w["dO"] * (steps < batch["fill"].view(-1, 1, 1, 1)).to(w["dO"].dtype)      # padded steps are loss-masked
    i = int(batch["pad_mask"].sum(1).argmin())           # the sample with the fewest slots keeps the oracle in seconds
    sub, ws = _sample_inputs(batch, w, i)
    _against_oracle(mb, sub, ws, TOL_BF16)


def test_config4_decode_window_against_the_oracle(mb):
    """Streaming decode at the full vocabulary: 64 steps of one sequence with thousands of seen slots, tensor-core attend
    against the oracle's dense step on the active slots."""
    from oracle import ema_oracle as orc
    from mathbrain_b200 import synth
    from mathbrain_b200.decode import DecodeState
    g = torch.Generator().manual_seed(11)
    B, V, N, H, K = 1, synth.VOCAB, 64, 8, 3000
    D = 64 * H
    rhos = synth.make_rhos(N)
    st = DecodeState(B, V, rhos.cuda(), capacity=K + 128)
    seen = torch.randperm(V, generator=g)[:K]
    state = torch.zeros(B, V, N)
    last = torch.full((B, V), -1, dtype=torch.long)
    state[0, seen] = torch.rand(K, N, generator=g) * 3 + 1
    last[0, seen] = torch.randint(0, 8192, (K,), generator=g)
    st.active[0, :K] = seen.to(torch.int32).cuda()
    st.last_t[0, seen.cuda()] = last[0, seen].to(torch.int32).cuda()
    st.state[0, seen.cuda()] = state[0, seen].cuda()
    st.n_active.fill_(K)
    E_k = (torch.randn(V, D, generator=g) * 0.02).to(torch.bfloat16)
    E_v = (torch.randn(V, D, generator=g) * 0.02).to(torch.bfloat16)
    W = torch.randn(N, D, generator=g) * 0.02
    E_kc, E_vc, Wc = E_k.cuda(), E_v.cuda(), W.cuda()
    toks = torch.from_numpy(synth.Zipf(V).draw(np.random.Generator(np.random.PCG64(3)), 64)).view(64, 1)
    for j in range(64):
        t = 8192 + j
        q = (torch.randn(B, H, 64, generator=g) * 0.02).to(torch.bfloat16)
        O = st.attend(q.cuda(), E_kc, E_vc, Wc, t, mode="tc_bf16")
        st.update(toks[j].cuda(), t)
        O_ref, _ = orc.decode_step(state, last, t, toks[j], q.float(), E_k.float(), E_v.float(), W, rhos, V)
        assert rel_err(O.cpu(), O_ref) < TOL_BF16, j
    st.check_overflow()
    assert st.device_status() == 0
