"""Chunked tied lm_head + masked cross-entropy against torch (float64): the reference's
`F.cross_entropy(lm_head(h).view(-1, V), y.view(-1), ignore_index=-100)` (mathbrain/model.py:185-186, train.py:320-323)."""
import pytest
import torch

from helpers import rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("V,chunk", [(1000, 64), (257, 4096), (50257, 96)])
def test_lm_head_cross_entropy(dtype, tol, V, chunk):
    from mathbrain_b200.lmhead import lm_head_cross_entropy
    g = torch.Generator().manual_seed(V)
    B, T, D = 3, 50, 64
    h = torch.randn(B, T, D, generator=g)
    E = torch.randn(V, D, generator=g) * 0.3
    y = torch.randint(0, V, (B, T), generator=g)
    y[0, 30:] = -100                                     # padded positions
    y[2, :] = -100                                       # a sample without a valid position
    y[1, 7] = V - 1
    h64, E64 = h.double().requires_grad_(True), E.double().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy((h64 @ E64.t()).view(-1, V), y.view(-1), ignore_index=-100)
    ref.backward()
    hd, Ed = h.cuda().requires_grad_(True), E.cuda().requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.bfloat16, enabled=(dtype == torch.bfloat16)):
        loss = lm_head_cross_entropy(hd, Ed, y.cuda(), chunk_rows=chunk)
    (loss * 3.0).backward()                              # the upstream factor reaches both gradients
    assert abs(float(loss.detach()) - float(ref.detach())) < tol * abs(float(ref.detach()))
    assert rel_err(hd.grad.cpu() / 3.0, h64.grad) < tol
    assert rel_err(Ed.grad.cpu() / 3.0, E64.grad) < tol
    assert float(hd.grad[2].abs().max()) == 0.0 and float(hd.grad[0, 30:].abs().max()) == 0.0


def test_lm_head_cross_entropy_all_masked():
    from mathbrain_b200.lmhead import lm_head_cross_entropy
    h = torch.randn(4, 8, device="cuda", requires_grad=True)
    E = torch.randn(20, 8, device="cuda", requires_grad=True)
    loss = lm_head_cross_entropy(h, E, torch.full((4,), -100, device="cuda"))
    loss.backward()
    assert float(loss.detach()) == 0.0 and float(h.grad.abs().max()) == 0.0 and float(E.grad.abs().max()) == 0.0
