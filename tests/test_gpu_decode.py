"""Streaming decode kernels against the dense CPU oracle (one iteration of the reference's attention loop per step)."""
import pytest
import torch

from oracle import ema_oracle as orc
from helpers import rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,V,N,H,steps,dt", [(3, 40, 8, 1, 30, torch.float32), (2, 300, 64, 2, 150, torch.float32),
                                               (2, 120, 16, 2, 80, torch.bfloat16)])
def test_decode_matches_dense_loop(B, V, N, H, steps, dt):
    from mathbrain_b200.decode import DecodeState
    from mathbrain_b200 import synth
    torch.manual_seed(B + V)
    D = 64 * H
    rhos = synth.make_rhos(N, 2.0, 64.0)
    E_k = (torch.randn(V, D) * 0.3).to(dt)
    E_v = (torch.randn(V, D) * 0.3).to(dt)
    W = torch.randn(N, D) * 0.3
    x = torch.randint(0, V, (B, steps))
    Q = (torch.randn(B, H, steps, 64) * 0.3).to(dt)
    st = DecodeState(B, V, rhos.cuda(), capacity=64 if V > 64 else V)
    state = torch.zeros(B, V, N)
    last = torch.full((B, V), -1, dtype=torch.long)
    cap = st.cap
    for t in range(steps):
        if int((last >= 0).sum(1).max()) >= cap and not bool(((last[torch.arange(B), x[:, t]]) >= 0).all()):
            break                                    # the next token would overflow the active list of this small test
        O = st.attend(Q[:, :, t].cuda(), E_k.cuda(), E_v.cuda(), W.cuda(), t, mode="fp32")      # the exact kernel
        Cq = st.update(x[:, t].cuda(), t)
        O_ref, Cq_ref = orc.decode_step(state, last, t, x[:, t], Q[:, :, t].float(), E_k.float(), E_v.float(), W, rhos, V)
        assert rel_err(O.cpu(), O_ref) < (1e-4 if dt == torch.float32 else 2e-2), t
        assert torch.allclose(Cq.cpu(), Cq_ref, atol=1e-5, rtol=1e-5), t
    st.check_overflow()


def test_decode_overflow_is_reported():
    from mathbrain_b200.decode import DecodeState
    from mathbrain_b200 import _lib, synth
    st = DecodeState(1, 10, synth.make_rhos(4, 2.0, 8.0).cuda(), capacity=2)
    for t, tok in enumerate([1, 2, 3]):
        st.update(torch.tensor([tok]).cuda(), t)
    with pytest.raises(_lib.MbemaError):
        st.check_overflow()


@pytest.mark.parametrize("B,V,H,steps,silu,dt", [(2, 700, 2, 300, True, torch.bfloat16), (3, 200, 4, 140, False, torch.float32),
                                                  (2, 500, 2, 260, True, torch.float32)])
def test_decode_tensor_core_matches_dense_loop(B, V, H, steps, silu, dt):
    """tcgen05 decode (bf16 operands) against the dense loop; several 128-slot tiles, the last one ragged."""
    from mathbrain_b200.decode import DecodeState
    from mathbrain_b200 import synth
    torch.manual_seed(V + H)
    N, D = 64, 64 * H
    rhos = synth.make_rhos(N, 2.0, 64.0)
    E_k = (torch.randn(V, D) * 0.2).to(dt)
    E_v = (torch.randn(V, D) * 0.2).to(dt)
    W = torch.randn(N, D) * 0.1
    x = torch.randint(0, V, (B, steps))
    Q = (torch.randn(B, H, steps, 64)).to(dt)
    st = DecodeState(B, V, rhos.cuda(), capacity=384)
    st_ref = DecodeState(B, V, rhos.cuda(), capacity=384)
    state = torch.zeros(B, V, N)
    last = torch.full((B, V), -1, dtype=torch.long)
    worst = 0.0
    for t in range(steps):
        q = Q[:, :, t].cuda()
        O = st.attend(q, E_k.cuda(), E_v.cuda(), W.cuda(), t, use_silu=silu, mode="tc_bf16")
        if t % 37 == 0 or t == steps - 1:
            O32 = st_ref.attend(q, E_k.cuda(), E_v.cuda(), W.cuda(), t, use_silu=silu, mode="fp32")
            assert rel_err(O.cpu(), O32.cpu()) < 2e-2, t
        st.update(x[:, t].cuda(), t)
        st_ref.update(x[:, t].cuda(), t)
        O_ref, _ = orc.decode_step(state, last, t, x[:, t], Q[:, :, t].float(), E_k.float(), E_v.float(), W, rhos, V,
                                   use_silu=silu)
        worst = max(worst, rel_err(O.cpu(), O_ref))
        assert worst < 2e-2, t
    st.check_overflow()
    assert int(st._ws[:4].view(torch.int32).item()) == 0


def test_decode_tensor_core_refuses_other_shapes():
    from mathbrain_b200.decode import DecodeState
    from mathbrain_b200 import _lib, synth
    st = DecodeState(1, 50, synth.make_rhos(16, 2.0, 8.0).cuda(), capacity=32)
    with pytest.raises(_lib.MbemaError):
        st.attend(torch.zeros(1, 2, 64).cuda(), torch.zeros(50, 128).cuda(), torch.zeros(50, 128).cuda(),
                  torch.zeros(16, 128).cuda(), 0, mode="tc_bf16")


def test_decode_tensor_core_many_tiles_per_cta():
    """Warm state with a different number of seen slots per sequence (up to 15 tiles of 128), enough sequences and
    heads that one CTA walks several tiles; compared with the fp32 kernel, which the dense loop checks above."""
    from mathbrain_b200.decode import DecodeState
    from mathbrain_b200 import synth
    g = torch.Generator().manual_seed(5)
    B, V, N, H, cap = 64, 3000, 64, 8, 2048
    D = 64 * H
    rhos = synth.make_rhos(N, 2.0, 256.0).cuda()
    st = DecodeState(B, V, rhos, capacity=cap)
    for b in range(B):
        K = int(torch.randint(1, 1900, (1,), generator=g)) if b else 1900
        seen = torch.randperm(V, generator=g)[:K].cuda()
        st.active[b, :K] = seen.to(torch.int32)
        st.last_t[b, seen] = torch.randint(0, 4000, (K,), generator=g).to(torch.int32).cuda()
        st.state[b, seen] = (torch.rand(K, N, generator=g) * 3 + 0.5).cuda()
        st.n_active[b] = K
    E_k = (torch.randn(V, D, generator=g) * 0.2).to(torch.bfloat16).cuda()
    E_v = (torch.randn(V, D, generator=g) * 0.2).to(torch.bfloat16).cuda()
    W = (torch.randn(N, D, generator=g) * 0.1).cuda()
    q = torch.randn(B, H, 64, generator=g).cuda()
    for silu in (True, False):
        O_tc = st.attend(q, E_k, E_v, W, 4000, use_silu=silu, mode="tc_bf16")
        O_32 = st.attend(q, E_k, E_v, W, 4000, use_silu=silu, mode="fp32")
        assert rel_err(O_tc.cpu(), O_32.cpu()) < 2e-2, silu
        assert int(st._ws[:4].view(torch.int32).item()) == 0
        O_tc2 = st.attend(q, E_k, E_v, W, 4000, use_silu=silu, mode="tc_bf16", listed_only=True)
        O_322 = st.attend(q, E_k, E_v, W, 4000, use_silu=silu, mode="fp32", listed_only=True)
        assert rel_err(O_tc2.cpu(), O_322.cpu()) < 2e-2, silu


def test_decode_step_replayed_from_a_cuda_graph():
    """A whole step (two layers of attend, update, advance) captured once and replayed, with the step number in device
    memory, against the same steps run eagerly on a second state."""
    from mathbrain_b200.decode import DecodeState
    from mathbrain_b200 import synth
    g = torch.Generator().manual_seed(11)
    B, V, N, H, L, steps = 5, 400, 64, 2, 2, 12
    D = 64 * H
    rhos = synth.make_rhos(N, 2.0, 64.0).cuda()
    E_k = [(torch.randn(V, D, generator=g) * 0.2).to(torch.bfloat16).cuda() for _ in range(L)]
    E_v = [(torch.randn(V, D, generator=g) * 0.2).to(torch.bfloat16).cuda() for _ in range(L)]
    W = [(torch.randn(N, D, generator=g) * 0.1).cuda() for _ in range(L)]
    toks = torch.randint(0, V, (steps + 3, B), generator=g).cuda()
    Q = torch.randn(steps + 3, L, B, H, 64, generator=g).cuda()
    st, ref = DecodeState(B, V, rhos, capacity=128), DecodeState(B, V, rhos, capacity=128)
    for t in range(3):                       # a few eager steps first, so that the captured step starts from a used state
        for s_ in (st, ref):
            s_.update(toks[t], t)
    st.use_device_step(3)
    q_static = [Q[3, l].clone() for l in range(L)]
    tok_static = toks[3].clone()
    graph, outs, C_q = st.capture_step(q_static, E_k, E_v, W, tok_static, mode="tc_bf16")
    for t in range(3, steps + 3):
        for l in range(L):
            q_static[l].copy_(Q[t, l])
        tok_static.copy_(toks[t])
        graph.replay()
        for l in range(L):
            O_ref = ref.attend(Q[t, l], E_k[l], E_v[l], W[l], t, mode="tc_bf16")
            assert rel_err(outs[l].cpu(), O_ref.cpu()) < 1e-5, (t, l)      # fp32 atomics: the order of the tile sums differs
        assert torch.equal(C_q, ref.update(toks[t], t)), t
    assert int(st.t_dev.item()) == steps + 3
    assert torch.equal(st.state, ref.state) and torch.equal(st.last_t, ref.last_t) and torch.equal(st.n_active, ref.n_active)
    st.check_overflow()
