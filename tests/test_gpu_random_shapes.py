"""Seeded random shapes: the tensor-core path against the fp32 kernels over ragged sizes (T around the 128-step tile
boundaries, one to five samples, two to eight heads, both channel counts, with and without a prefix state)."""
import random

import pytest
import torch

from helpers import rel_err
from test_gpu_fullsize import _run

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mb():
    import mathbrain_b200
    return mathbrain_b200


@pytest.mark.parametrize("seed", range(12))
def test_tc_matches_fp32_kernels_on_random_shapes(mb, seed):
    from mathbrain_b200 import synth
    rnd = random.Random(seed)
    B = rnd.choice([1, 2, 3, 5])
    T = rnd.choice([1, 17, 127, 128, 129, 300, 513, 1000])
    H = rnd.choice([2, 4, 8])
    N = rnd.choice([64, 64, 128])
    batch = synth.make_chunk_batch(100 + seed, B, T, N, vocab=rnd.choice([40, 500, 50257]),
                                   max_prefix=rnd.choice([0, 50, 3000]), min_fill=1, bursty=rnd.random() < 0.4,
                                   min_hl=rnd.choice([1.0, 64.0, 1024.0]), max_hl=4096.0)
    # operand scale: pre-activations (state . W_pe over N channels) stay within a few tens, the range in which 16-bit
    # gate and gradient tiles hold the 2e-2 budget (states reach the hundreds after a 3000-token prefix)
    state_max = float(batch["c_base"].abs().max()) + T
    std = min(0.05, 25.0 / (state_max * N ** 0.5))
    w = synth.make_layer_weights(seed, B, batch["K_max"], 64 * H, N, T, H, std=std, dtype=torch.bfloat16)
    steps = torch.arange(T).view(1, 1, T, 1)
    w["dO"] = w["dO"] * (steps < batch["fill"].view(-1, 1, 1, 1)).to(w["dO"].dtype)   # padded steps are loss-masked
    tc = _run(mb, batch, w, "tc_bf16")
    ref = _run(mb, batch, w, "fp32")
    tol = 2e-2                                # fp16 gate operands for every N
    for k in ref:
        assert torch.isfinite(tc[k]).all(), k
        assert rel_err(tc[k], ref[k]) < tol, (k, rel_err(tc[k], ref[k]), dict(B=B, T=T, H=H, N=N))
