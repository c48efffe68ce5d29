"""Host-side data-parallel logic with two gloo ranks on the CPU (no GPU)."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    from mathbrain_b200 import dp
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(100 + rank)
        lin = torch.nn.Linear(4, 3)
        for p in lin.parameters():
            p.grad = torch.randn(p.shape, generator=g)
        local = [p.grad.clone() for p in lin.parameters()]
        unique = torch.tensor([[1, 3, -1], [0, 1, 2]])
        dE = [torch.randn(2, 3, 5, generator=g), torch.randn(2, 3, 5, generator=g)]
        table = dp.slot_embedding_grad(dE, unique, vocab=6)
        local_table = table.clone()
        dp.allreduce_gradients(list(lin.parameters()), extra=[table])
        # per-layer buckets: gradients accumulate straight into the flat buffer, reduced asynchronously
        lin2 = torch.nn.Linear(4, 3)
        bucket = dp.GradBucket(list(lin2.parameters()))
        bucket.zero()
        inp = torch.randn(5, 4, generator=g)
        lin2(inp).sum().backward()
        lin2(inp).sum().backward()                 # accumulates in place, the views stay views
        local2 = [p.grad.clone() for p in lin2.parameters()]
        assert all(p.grad.data_ptr() >= bucket.flat.data_ptr() for p in lin2.parameters())
        bucket.all_reduce_async()
        bucket.wait()
        assert torch.equal(torch.cat([p.grad.reshape(-1) for p in lin2.parameters()]), bucket.flat)
        q.put(("bucket", rank, local2, [p.grad.clone() for p in lin2.parameters()]))
        q.put((rank, [t.clone() for t in local], local_table, [p.grad.clone() for p in lin.parameters()], table.clone(),
               dp.shard_bounds(11, rank, world)))
    finally:
        dist.destroy_process_group()


def test_gradient_exchange_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=120) for _ in range(2 * len(procs))]
    bk = sorted([t[1:] for t in got if t[0] == "bucket"], key=lambda t: t[0])
    res = sorted([t for t in got if t[0] != "bucket"], key=lambda t: t[0])
    for a, b, c, d in zip(bk[0][1], bk[1][1], bk[0][2], bk[1][2]):
        assert torch.allclose(a + b, c) and torch.equal(c, d)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (_, l0, t0, r0, rt0, b0), (_, l1, t1, r1, rt1, b1) = res
    for a, b, c, d in zip(l0, l1, r0, r1):
        assert torch.allclose(a + b, c) and torch.allclose(c, d)
    assert torch.allclose(t0 + t1, rt0) and torch.allclose(rt0, rt1)
    assert b0 == (0, 6) and b1 == (6, 11)


def test_slot_embedding_grad_skips_non_slots():
    from mathbrain_b200 import dp
    unique = torch.tensor([[2, -1, 2]])
    g = torch.ones(1, 3, 4)
    out = dp.slot_embedding_grad([g], unique, vocab=5)
    assert out[2].tolist() == [2.0] * 4 and float(out.sum()) == 8.0


def test_balanced_shards_even_counts_and_lower_peak():
    import numpy as np
    from mathbrain_b200 import dp, synth
    rng = np.random.Generator(np.random.PCG64(3))
    costs = rng.integers(300, 2600, size=64).tolist()
    shards = dp.balanced_shards(costs, 8)
    assert sorted(i for s in shards for i in s) == list(range(64))
    assert all(len(s) == 8 for s in shards)
    peak = max(sum(costs[i] for i in s) for s in shards)
    naive = max(sum(costs[r * 8:(r + 1) * 8]) for r in range(8))
    mean = sum(costs) / 8
    assert peak <= naive and peak < 1.02 * mean
    with pytest.raises(ValueError):
        dp.balanced_shards(costs[:63], 8)
    batch = synth.make_chunk_batch(5, 8, 64, 8, vocab=200, max_prefix=100, min_fill=8)
    sub = synth.select_samples(batch, dp.balanced_shards(batch["pad_mask"].sum(1).tolist(), 2)[1])
    assert sub["x"].shape[0] == 4 and sub["unique_slots"].shape[1] == sub["K_max"] == max(16, int(sub["pad_mask"].sum(1).max()))
    assert bool((sub["unique_slots"][~sub["pad_mask"]] == 0).all())


def test_document_chunks_follow_the_reference_rule():
    from mathbrain_b200.data import document_chunks
    # lengths 0 and 1 are dropped; n tokens give ceil((n - 1) / block) chunks of at most block + 1 tokens
    assert document_chunks([0, 1], 4) == []
    assert document_chunks([2], 4) == [(0, 0, 2)]
    assert document_chunks([5], 4) == [(0, 0, 5)]
    assert document_chunks([6], 4) == [(0, 0, 5), (0, 4, 6)]
    assert document_chunks([9, 3], 4) == [(0, 0, 5), (0, 4, 9), (1, 0, 3)]
    assert document_chunks([10], 4) == [(0, 0, 5), (0, 4, 9), (0, 8, 10)]


def test_document_batch_carries_each_documents_own_prefix_state():
    from mathbrain_b200 import synth
    from oracle import ema_oracle as orc
    b = synth.make_document_batch(3, 12, 32, 4, vocab=50, median_len=60.0, sigma=0.8, min_hl=2.0, max_hl=16.0)
    assert b["x"].shape == (12, 32) and int(b["fill"].max()) <= 32
    # chunks of one document are consecutive and their prefixes advance by the block size
    for i in range(1, 12):
        if b["doc"][i] == b["doc"][i - 1]:
            assert int(b["prefix_len"][i]) == int(b["prefix_len"][i - 1]) + 32 and int(b["fill"][i - 1]) == 32
        else:
            assert int(b["prefix_len"][i]) == 0
    # the state handed to chunk c + 1 is what scanning chunk c from its own c_base leaves behind
    for i in range(1, 12):
        if b["doc"][i] != b["doc"][i - 1]:
            continue
        prev, cur = i - 1, i
        kp = int(b["pad_mask"][prev].sum())
        keys_prev = b["unique_slots"][prev:prev + 1, :kp]
        M = orc.memory_states(b["x"][prev:prev + 1], keys_prev, b["rhos"], b["c_base"][prev:prev + 1, :kp],
                              dtype=torch.float64)                       # [1, T, K, N]: state seen AT step t
        hit = (keys_prev[0] == b["x"][prev, 31]).double().unsqueeze(-1)
        after = (M[0, 31] + hit) * b["rhos"].double()                    # ... and after the last step
        end = {int(k): after[j] for j, k in enumerate(keys_prev[0].tolist())}
        kc = int(b["pad_mask"][cur].sum())
        for j, k in enumerate(b["unique_slots"][cur, :kc].tolist()):
            want = end.get(int(k), torch.zeros(4, dtype=torch.float64))
            assert torch.allclose(b["c_base"][cur, j].double(), want, rtol=1e-5, atol=1e-6)
