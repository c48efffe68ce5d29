"""The C-ABI library builds, loads and exports every symbol include/mbema.h declares (no GPU needed)."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from mathbrain_b200 import build, _lib
    build.build()
    return _lib.load()


def test_header_symbols_exported(lib):
    hdr = open(os.path.join(ROOT, "include", "mbema.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    declared = set(re.findall(r"\b(mbema_[a-z0-9_]+)\s*\(", hdr))
    assert len(declared) >= 14
    for name in sorted(declared):
        assert hasattr(lib, name), name
    from mathbrain_b200 import _lib
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)


def test_version_and_strerror(lib):
    assert lib.mbema_version() == 200
    assert lib.mbema_strerror(0) == b"ok"
    assert b"workspace" in lib.mbema_strerror(4)


def test_argument_errors_before_launch(lib):
    # bad shapes / unsupported sizes are rejected on the host, nothing is launched (works without a GPU)
    assert lib.mbema_query_scan(None, None, None, None, None, None, 1, 0, 4, 0, 0, None, 0, None) == 2
    assert lib.mbema_query_scan(None, None, None, None, None, None, 1, 9000, 4, 0, 0, None, 0, None) == 3
    assert lib.mbema_query_scan(None, None, None, None, None, None, 1, 16, 4, 0, 0, None, 0, None) == 1
    assert lib.mbema_qgate_fwd(None, 0, None, 0, None, None, None, 1e-5, None, 0, None, None, 4, 2048, 1, None) == 3
    a = [None, 0, None, None, None, 0, None, None, None, None, None, None, None, None, None]
    assert lib.mbema_flash_fwd(*a, 1, 8, 128, 32, 64, 16, 100, 1, 0, None, 0, None) == 3      # hd != 64
    assert lib.mbema_flash_fwd(*a, 1, 8, 128, 64, 64, 16, 100, 1, 0, None, 0, None) == 1      # NULL pointers
    assert lib.mbema_query_scan_workspace_bytes(2, 128) >= 4 * 2 * 128 * 4


def test_operators_refuse_cpu_tensors():
    import mathbrain_b200 as mb
    with pytest.raises(mb._lib.MbemaError):
        mb.compute_query_ema_history(torch.zeros(1, 4, dtype=torch.long), torch.ones(2), 5)
    with pytest.raises(mb._lib.MbemaError):
        mb.precompute_boundaries(torch.zeros(1, 4, dtype=torch.long), torch.zeros(1, 16, dtype=torch.long),
                                 torch.ones(2), 64)


def test_product_does_not_import_oracle():
    pkg = os.path.join(ROOT, "mathbrain_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src, os.path.join(dirpath, f)


def test_synthetic_batch_format():
    from mathbrain_b200 import synth
    b = synth.make_chunk_batch(3, B=3, T=96, N=8, vocab=500, max_prefix=200, min_fill=10)
    x, u, pm = b["x"], b["unique_slots"], b["pad_mask"]
    assert x.shape == (3, 96) and u.shape[0] == 3 and u.shape[1] >= 16
    for i in range(3):
        fill = int(b["fill"][i])
        keys = u[i][pm[i]].tolist()
        assert len(set(keys)) == len(keys)
        assert set(x[i, :fill].tolist()) <= set(keys)
        assert (x[i, fill:] == 0).all()
        assert (b["c_base"][i][~pm[i]] == 0).all()
