"""GPU-side construction of unique_slots / pad_mask / c_base from resident per-document state (ChunkFeeder) against
the host-side definition: slot lists in the order of mathbrain/data.py:104-124 (chunk tokens sorted, then history-only
tokens sorted) and c_base as the closed-form state of the document's own prefix (mathbrain/data.py:128-140)."""
import numpy as np
import pytest
import torch

from helpers import rel_err

pytestmark = pytest.mark.gpu


def test_feeder_streams_documents_chunk_by_chunk():
    import mathbrain_b200 as mb
    from mathbrain_b200 import synth
    from mathbrain_b200.feeder import ChunkFeeder
    B, V, N, T = 4, 90, 8, 24
    rng = np.random.Generator(np.random.PCG64(5))
    rhos = synth.make_rhos(N, 2.0, 40.0)
    rhos64 = rhos.double().numpy()
    dev = "cuda"
    feeder = ChunkFeeder(B, V, rhos.to(dev), capacity=64)
    history = [np.zeros(0, np.int64) for _ in range(B)]
    zipf = synth.Zipf(V)
    for step in range(5):
        if step == 3:                                   # document 1 ends, a new one starts in its row
            feeder.reset([1])
            history[1] = np.zeros(0, np.int64)
        fill = rng.integers(1, T + 1, B)
        if step == 0:
            fill[0] = T
        x = np.zeros((B, T), np.int64)
        for b in range(B):
            x[b, :fill[b]] = zipf.draw(rng, int(fill[b]))
        xd, fd = torch.from_numpy(x).to(dev), torch.from_numpy(fill).to(dev)
        batch = feeder.next_batch(xd, fd)
        K = batch["K_max"]
        assert batch["unique_slots"].shape == (B, K) and batch["c_base"].shape == (B, K, N)
        for b in range(B):
            chunk = x[b, :fill[b]]
            cu = np.unique(chunk)
            hu = np.setdiff1d(np.unique(history[b]), cu)
            keys = np.concatenate([cu, hu])
            k = len(keys)
            assert int(batch["pad_mask"][b].sum()) == k and bool(batch["pad_mask"][b, :k].all())
            assert batch["unique_slots"][b, :k].cpu().numpy().tolist() == keys.tolist()
            assert int(batch["unique_slots"][b, k:].abs().sum()) == 0          # padded with token 0, as the collate function
            want = synth.prefix_state(history[b], keys, rhos64)
            got = batch["c_base"][b, :k].cpu()
            assert rel_err(got, torch.from_numpy(want)) < 1e-5 if want.any() else float(got.abs().max()) == 0.0
            assert float(batch["c_base"][b, k:].abs().max()) == 0.0 if k < K else True
        C_seq = mb.compute_query_ema_history(xd, rhos.to(dev), V, batch["c_base"], batch["unique_slots"])
        feeder.advance(xd, fd, C_seq)
        for b in range(B):
            history[b] = np.concatenate([history[b], x[b, :fill[b]]])
        assert feeder.t0.cpu().tolist() == [len(h) for h in history]
        assert feeder.n_seen.cpu().tolist() == [len(np.unique(h)) for h in history]


def test_feeder_refuses_a_full_list():
    import mathbrain_b200 as mb
    from mathbrain_b200 import synth
    from mathbrain_b200.feeder import ChunkFeeder
    rhos = synth.make_rhos(4, 2.0, 8.0).cuda()
    feeder = ChunkFeeder(1, 50, rhos, capacity=4)
    x = torch.arange(8, device="cuda").view(1, 8)
    fill = torch.tensor([8], device="cuda")
    batch = feeder.next_batch(x, fill)
    C_seq = mb.compute_query_ema_history(x, rhos, 50, batch["c_base"], batch["unique_slots"])
    with pytest.raises(mb._lib.MbemaError):
        feeder.advance(x, fill, C_seq)
