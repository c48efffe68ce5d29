"""Tensor-core (tcgen05) attention path against the fp32 oracle; bf16 tolerance 2e-2 (norm-wise relative)."""
import numpy as np
import pytest
import torch

from oracle import ema_oracle as orc
from helpers import rel_err
from test_gpu_parity import make_case, oracle_flash, run_flash, compare_all, cu, TOL_BF16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mb():
    import mathbrain_b200 as m
    m._lib.load()
    m.set_options(inactive_mass="full_V", cbase_extra_decay=False, mode="fp32")
    return m


def run_tc(mb, inp, c_base=None, seq_lens=None, dtype=torch.bfloat16, with_grad=True, **opt):
    with mb.options(mode="tc_bf16", **opt):
        out = run_flash(mb, inp, c_base, seq_lens=seq_lens, dtype=dtype, with_grad=with_grad)
    assert mb.device_status() == 0
    return out


@pytest.mark.parametrize("T,H,bursty,vocab", [(64, 2, False, 400), (200, 2, True, 30), (384, 4, False, 2000)])
def test_tc_forward_vs_oracle(mb, T, H, bursty, vocab):
    inp, c_base, _ = make_case(300 + T, B=2, T=T, N=64, H=H, vocab=vocab, max_prefix=150, min_hl=1.0, max_hl=300.0,
                               bursty=bursty)
    out = run_tc(mb, inp, c_base, with_grad=False)
    ref = orc.flash_ema(inp["Q"], inp["x"], inp["E_k"], inp["E_v"], inp["W_pe"], inp["rhos"], inp["V"], inp["unique"],
                        c_base=c_base)
    assert rel_err(out["O"], ref["O"]) < TOL_BF16
    # against the oracle that rounds state and W_pe to bf16 once (the kernel rounds snapshot and decay power separately)
    q16 = lambda t: t.to(torch.bfloat16).float()
    ref16 = orc.flash_ema(q16(inp["Q"]), inp["x"], q16(inp["E_k"]), q16(inp["E_v"]), inp["W_pe"], inp["rhos"], inp["V"],
                          inp["unique"], c_base=c_base, round_bf16=True)
    assert rel_err(out["O"], ref16["O"]) < 1.5e-2


def test_tc_forward_backward_config1_shape(mb):
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
    out = run_tc(mb, inp)
    compare_all(out, ref, TOL_BF16)


def test_tc_semantic_switches_and_seq_lens(mb):
    # operand scale 0.1 (five times the model's init scale); at 0.3 the bf16 operands alone cost 2-3 %
    inp, c_base, fill = make_case(41, B=3, T=300, N=64, H=2, vocab=300, max_prefix=100, min_hl=2.0, max_hl=100.0,
                                  min_fill=20, std=0.1)
    inp["dO"] = inp["dO"].clone()
    for b, n in enumerate(fill.tolist()):
        inp["dO"][b, :, n:] = 0
    out = run_tc(mb, inp, c_base, seq_lens=fill, inactive_mass="listed_only", cbase_extra_decay=True)
    ref = oracle_flash(inp, c_base, inactive_mass="listed_only", extra_decay=True)
    compare_all(out, ref, TOL_BF16, rows=fill.tolist())
    inp["use_silu"] = False
    out = run_tc(mb, inp, c_base)
    ref = oracle_flash(inp, c_base)
    compare_all(out, ref, TOL_BF16)


def test_tc_n128_forward_and_mixed_backward(mb):
    # N = 128 (the long-chunk configuration): tensor-core forward and backward, fp16 gate operands as for N = 64
    # operand scale 0.1: with 128 products per pre-activation the error budget (2e-2) holds for |pre| of a few units
    inp, c_base, _ = make_case(77, B=2, T=300, N=128, H=2, vocab=500, max_prefix=200, min_hl=4.0, max_hl=500.0, std=0.1)
    out = run_tc(mb, inp, c_base)
    ref = oracle_flash(inp, c_base)
    for k in ("O", "dQ", "dE_k", "dE_v"):
        assert rel_err(out[k], ref[k]) < TOL_BF16, k
    assert rel_err(out["dW_pe"], ref["dW_pe"]) < TOL_BF16
    with mb.options(mode="tc_bf16", fp32_backward=True):
        mixed = run_flash(mb, inp, c_base, dtype=torch.bfloat16)
    assert rel_err(mixed["dW_pe"], ref["dW_pe"]) < 5e-3


def test_tc_long_chunk_property(mb):
    """T = 4096 with bursty repeats (long-chunk stress shape, reduced batch): one chunk equals two half chunks
    chained through the slot states, and matches the fp32 kernels."""
    inp, c_base, _ = make_case(91, B=1, T=4096, N=64, H=2, vocab=3000, max_prefix=0, min_hl=1024.0, max_hl=4096.0,
                               std=0.02, bursty=True, min_fill=4096, holes=False)   # weights at the model's init scale
    full = run_tc(mb, inp, c_base, with_grad=False)["O"]
    with mb.options(mode="fp32"):
        ref = run_flash(mb, inp, c_base, with_grad=False)["O"]
    assert rel_err(full, ref) < TOL_BF16
    M = orc.memory_states(inp["x"][:, :2049], inp["unique"], inp["rhos"], c_base, dtype=torch.float64)
    second = dict(inp)
    second["x"] = inp["x"][:, 2048:].contiguous()
    second["Q"] = inp["Q"][:, :, 2048:].contiguous()
    tail = run_tc(mb, second, M[:, 2048].float(), with_grad=False)["O"]
    assert rel_err(tail, full[:, :, 2048:]) < 5e-3


def test_tc_unsupported_shape_is_refused(mb):
    inp, c_base, _ = make_case(5, B=1, T=64, N=16, H=2, vocab=100, max_prefix=10, min_hl=2.0, max_hl=30.0)
    with pytest.raises(mb._lib.MbemaError):
        run_tc(mb, inp, c_base, with_grad=False)


@pytest.mark.parametrize("mode", ["tc_bf16", "fp32"])
def test_shared_embedding_rows_match_per_sample_tensors(mb, mode):
    """Slot-embedding rows shared between samples (one row per token listed anywhere in the batch): same output as the
    per-sample [B,K,D] tensors gathered from those rows, and row gradients equal to the scatter-sum of the per-sample ones."""
    inp, c_base, _ = make_case(23, B=4, T=260, N=64, H=2, vocab=150, max_prefix=120, min_hl=4.0, max_hl=300.0, std=0.1)
    dev = "cuda"
    unique = inp["unique"].to(dev)
    tokens, row_index = mb.shared_slot_rows(unique)
    U, D = tokens.numel(), inp["E_k"].shape[-1]
    g = torch.Generator().manual_seed(3)
    dt = torch.bfloat16 if mode == "tc_bf16" else torch.float32
    Ek_rows = (torch.randn(U, D, generator=g) * 0.1).to(dt).to(dev)
    Ev_rows = (torch.randn(U, D, generator=g) * 0.1).to(dt).to(dev)
    valid = (unique >= 0).unsqueeze(-1)
    Ek_b = (Ek_rows[row_index.long()] * valid).detach().clone().requires_grad_(True)
    Ev_b = (Ev_rows[row_index.long()] * valid).detach().clone().requires_grad_(True)
    Ek_r, Ev_r = Ek_rows.clone().requires_grad_(True), Ev_rows.clone().requires_grad_(True)
    x, rhos = inp["x"].to(dev), inp["rhos"].to(dev)
    K = unique.shape[1]
    dO = inp["dO"].to(dev).float()
    outs = []
    with mb.options(mode=mode):
        h = mb.precompute_boundaries(x, unique, rhos, 64, c_init=c_base.to(dev))
        for shared in (False, True):
            Q = inp["Q"].to(dev).to(dt).requires_grad_(True)
            W = inp["W_pe"].to(dev).requires_grad_(True)
            if shared:
                O = mb.FlashEMARowsFunction.apply(Q, x, Ek_r, Ev_r, row_index, W, rhos, inp["V"], unique, K, h, True)
            else:
                O = mb.FlashEMAFunction.apply(Q, x, Ek_b, Ev_b, W, rhos, inp["V"], unique, K, h, True)
            O.backward(dO)
            outs.append((O.detach().float().cpu(), Q.grad.float().cpu(), W.grad.float().cpu()))
    assert mb.device_status() == 0
    assert float((outs[0][0] - outs[1][0]).abs().max()) == 0.0                 # forward: the same rows, bit for bit
    assert rel_err(outs[1][1], outs[0][1]) < 1e-6                              # dQ
    assert rel_err(outs[1][2], outs[0][2]) < 1e-5                              # dW_pe (per-CTA partials, same order)
    for rows_grad, per_sample in ((Ek_r.grad, Ek_b.grad), (Ev_r.grad, Ev_b.grad)):
        ref = torch.zeros(U, D, device=dev)
        ref.index_add_(0, row_index.long().reshape(-1), (per_sample.float() * valid).reshape(-1, D))
        assert rel_err(rows_grad.float().cpu(), ref.cpu()) < (2e-2 if mode == "tc_bf16" else 1e-5)   # atomics: order differs


def test_bounded_wait_gives_up_cleanly(mb):
    """The give-up path of the tensor-core forward: with the library's test hook one hand-off between the kernel's warps
    is withheld and its waits expire after a few polls.  The launch must end by itself, the sticky status word must name
    the failed wait and stay set over later calls, and -- once cleared -- the next launch must run normally, which it can
    only do if the first one released its tensor memory.  Nothing here hangs or faults the GPU: every wait is bounded."""
    inp, c_base, _ = make_case(901, B=2, T=200, N=64, H=2, vocab=300, max_prefix=100, min_hl=4.0, max_hl=500.0)
    assert mb.device_status() == 0
    mb.ops._OPTIONS["_test_withhold_arrive"] = True
    try:
        with mb.options(mode="tc_bf16"):
            run_flash(mb, inp, c_base, dtype=torch.bfloat16, with_grad=False)
    finally:
        mb.ops._OPTIONS["_test_withhold_arrive"] = False
    torch.cuda.synchronize()
    st = mb.device_status()
    assert st & 1, hex(st)                       # a bounded wait gave up ...
    assert (st >> 8) in (1, 2, 3), hex(st)       # ... and the word says which one
    with pytest.raises(mb._lib.MbemaError):
        mb.ops.check_status()
    # sticky: a later call does not clear it (its CTAs see the word and skip their work)
    with mb.options(mode="tc_bf16"):
        run_flash(mb, inp, c_base, dtype=torch.bfloat16, with_grad=False)
    assert mb.device_status() == st
    mb.ops.clear_status()
    out = run_tc(mb, inp, c_base, with_grad=False)
    with mb.options(mode="fp32"):
        ref = run_flash(mb, inp, c_base, dtype=torch.bfloat16, with_grad=False)
    assert rel_err(out["O"], ref["O"]) < TOL_BF16


def test_bounded_wait_gives_up_cleanly_in_the_backward(mb):
    """The same for the tensor-core backward: the forward runs normally, the hook withholds one hand-off of the backward's
    gate product; the launch ends by itself, the status names a wait of the backward, no gradient of the failed CTAs is
    trusted (the status says so), and after clear_status() forward + backward are correct again."""
    inp, c_base, _ = make_case(902, B=2, T=200, N=64, H=2, vocab=300, max_prefix=100, min_hl=4.0, max_hl=500.0, std=0.1)
    assert mb.device_status() == 0
    dev = "cuda"
    unique = inp["unique"].to(dev)
    with mb.options(mode="tc_bf16"):
        h = mb.precompute_boundaries(inp["x"].to(dev), unique, inp["rhos"].to(dev), 64, c_init=c_base.to(dev))
        leaves = [inp[k].to(dev).to(torch.bfloat16 if k != "W_pe" else torch.float32).requires_grad_(True)
                  for k in ("Q", "E_k", "E_v", "W_pe")]
        O = mb.FlashEMAFunction.apply(leaves[0], inp["x"].to(dev), leaves[1], leaves[2], leaves[3], inp["rhos"].to(dev),
                                      inp["V"], unique, unique.shape[1], h, True)
        torch.cuda.synchronize()
        assert mb.device_status() == 0
        mb.ops._OPTIONS["_test_withhold_arrive"] = True
        try:
            O.backward(inp["dO"].to(dev).float())
        finally:
            mb.ops._OPTIONS["_test_withhold_arrive"] = False
    torch.cuda.synchronize()
    st = mb.device_status()
    assert st & 1, hex(st)
    assert 1 <= (st >> 8) <= 8, hex(st)
    with pytest.raises(mb._lib.MbemaError):
        mb.ops.check_status()
    mb.ops.clear_status()
    out = run_tc(mb, inp, c_base)
    ref = oracle_flash(inp, c_base)
    compare_all(out, ref, TOL_BF16)
