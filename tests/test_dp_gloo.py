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
    res = sorted([q.get(timeout=120) for _ in procs], key=lambda t: t[0])
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
