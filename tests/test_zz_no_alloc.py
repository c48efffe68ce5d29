"""Allocation-free query scan (mbema_query_scan_static): for hosts that may not allocate device memory around the
call -- a fixed-budget serving loop, a plugin boundary without an allocator -- the scratch is a fixed array inside the
library.  Called straight through the C ABI, twice in a row with different inputs (the scratch keeps the first call's
contents), and compared with the workspace-taking entry point; the file sorts last so it runs after every other test.
"""
import ctypes

import pytest
import torch

from helpers import rel_err

pytestmark = pytest.mark.gpu

TOL_STATE = 1e-5      # EMA-state tolerance used throughout the suite


def _vp(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _scan_both(lib, batch):
    x = batch["x"].cuda()
    rhos = batch["rhos"].cuda()
    c_base = batch["c_base"].cuda()
    keys = batch["unique_slots"].cuda()
    B, T = x.shape
    N, K = rhos.shape[0], keys.shape[1]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ws = torch.empty(lib.mbema_query_scan_workspace_bytes(B, T), dtype=torch.uint8, device="cuda")
    ref = torch.empty(B, T, N, device="cuda")
    out = torch.full((B, T, N), float("nan"), device="cuda")
    rc = lib.mbema_query_scan(_vp(x), _vp(rhos), _vp(c_base), _vp(keys), None, _vp(ref), B, T, N, K, 0, _vp(ws),
                              ws.numel(), stream)
    assert rc == 0, lib.mbema_strerror(rc)
    rc = lib.mbema_query_scan_static(_vp(x), _vp(rhos), _vp(c_base), _vp(keys), None, _vp(out), B, T, N, K, 0, stream)
    assert rc == 0, lib.mbema_strerror(rc)
    torch.cuda.synchronize()
    return out.cpu(), ref.cpu()


def test_static_scan_matches_workspace_scan_twice():
    from mathbrain_b200 import _lib, synth
    lib = _lib.load()
    first = synth.make_chunk_batch(901, B=6, T=512, N=64, vocab=5000, max_prefix=600, min_fill=100)
    second = synth.make_chunk_batch(902, B=3, T=200, N=16, vocab=300, max_prefix=100, min_fill=50, min_hl=2.0, max_hl=64.0)
    for batch in (first, second):
        out, ref = _scan_both(lib, batch)
        assert torch.isfinite(out).all()
        assert rel_err(out, ref) < TOL_STATE


def test_static_scan_rejects_oversize():
    from mathbrain_b200 import _lib
    lib = _lib.load()
    x = torch.zeros(70, 512, dtype=torch.long, device="cuda")       # 35840 tokens > 32768
    rhos = torch.full((4,), 0.9, device="cuda")
    out = torch.empty(70, 512, 4, device="cuda")
    rc = lib.mbema_query_scan_static(_vp(x), _vp(rhos), None, None, None, _vp(out), 70, 512, 4, 0, 0, None)
    assert rc == 8 and b"fixed scratch" in lib.mbema_strerror(rc)
