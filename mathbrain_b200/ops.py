"""Python operators of the Per-Slot-EMA hot path, with the reference's names and signatures.

Every operator here runs hand-written sm_100a CUDA kernels from libmbema.so through its C ABI
(include/mbema.h).  There is no Triton, no dispatch between back ends and no CPU path: a tensor that is not
on a CUDA device, or a missing shared library, raises.

Reference operators mirrored (paths within the reference tree):
  compute_query_ema_history            mathbrain/triton_ema_query.py:120
  precompute_boundaries                mathbrain/triton_flash_ema.py:81
  _build_unique_index                  mathbrain/triton_flash_ema.py:475
  FlashEMAFunction                     mathbrain/triton_flash_ema.py:571
  FusedGatingFunction                  mathbrain/triton_fused_gating.py:122
  fused_apply_symmetric_query_gating   mathbrain/triton_fused_gating.py:179
  HAS_TRITON                           the flag mathbrain/model.py:78,162 tests before taking the GPU path
"""
from __future__ import annotations

import contextlib
import functools
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib

# mathbrain/model.py takes its GPU operator path when this name is truthy.
HAS_TRITON = True

_OPTIONS = {"inactive_mass": "full_V", "cbase_extra_decay": False, "mode": "auto", "fp32_backward": False,
            "_test_withhold_arrive": False}
_MODES = {"fp32": _lib.MODE_FP32, "tc_bf16": _lib.MODE_TC_BF16, "auto": None}


def set_options(inactive_mass: Optional[str] = None, cbase_extra_decay: Optional[bool] = None,
                mode: Optional[str] = None, fp32_backward: Optional[bool] = None):
    """Semantics and precision switches of the attention operator.

    inactive_mass      "full_V" (default): softmax over all V_total vocabulary slots, as the PyTorch reference
                       (mathbrain/flash_ema_attention.py:76-79); "listed_only": over the listed slots only, which
                       is what the reference's Triton kernel computes (mathbrain/triton_flash_ema.py:214-230).
    cbase_extra_decay  False (default): the slot state seen at chunk step 0 is exactly c_base
                       (mathbrain/data.py:128-140); True: rho * c_base, the Triton kernels' convention
                       (mathbrain/triton_flash_ema.py:48-50,185).
    mode               "auto" (default): the tensor-core kernels wherever the shape allows them (hd = 64, N in {64, 128},
                       an even number of heads, a slot list that fits shared memory), the fp32 kernels otherwise --
                       like the reference, which takes its fast path by itself (mathbrain/model.py:78);
                       "tc_bf16": tensor-core kernels (16-bit gate operands, fp32 accumulation; 2e-2 tolerance),
                       unsupported shapes raise; "fp32": fp32 arithmetic on the CUDA cores (1e-4 tolerance).
    fp32_backward      with mode "tc_bf16": keep the tensor-core forward but run the backward with the fp32 kernels.
    """
    if fp32_backward is not None:
        _OPTIONS["fp32_backward"] = bool(fp32_backward)
    if inactive_mass is not None:
        if inactive_mass not in ("full_V", "listed_only"):
            raise ValueError(inactive_mass)
        _OPTIONS["inactive_mass"] = inactive_mass
    if cbase_extra_decay is not None:
        _OPTIONS["cbase_extra_decay"] = bool(cbase_extra_decay)
    if mode is not None:
        if mode not in _MODES:
            raise ValueError(mode)
        _OPTIONS["mode"] = mode


def get_options():
    return dict(_OPTIONS)


@contextlib.contextmanager
def options(**kw):
    old = dict(_OPTIONS)
    set_options(**kw)
    try:
        yield
    finally:
        _OPTIONS.update(old)


# ---------------------------------------------------------------------------------------------
# helpers
# ---------------------------------------------------------------------------------------------
def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and t.device.type != "cuda":
            raise _lib.MbemaError("mathbrain_b200 operators need CUDA tensors (got %s); there is no CPU path"
                                  % t.device)


def _ptr(t):
    return None if t is None else t.data_ptr()


def _on_tensor_device(fn):
    """Run `fn` with the device of its CUDA tensor arguments current (kernels are launched on the current device's
    current stream while the buffers live where the tensors are); tensors on different devices are refused."""
    @functools.wraps(fn)
    def wrapper(*args, **kw):
        dev = None
        for a in list(args) + list(kw.values()):
            t = a.tile_state if isinstance(a, TileStates) else a
            if torch.is_tensor(t) and t.device.type == "cuda":
                if dev is None:
                    dev = t.device
                elif t.device != dev:
                    raise _lib.MbemaError("operands live on different devices (%s and %s)" % (dev, t.device))
        if dev is None or dev.index == torch.cuda.current_device():
            return fn(*args, **kw)
        with torch.cuda.device(dev):
            return fn(*args, **kw)
    return wrapper


def _dt(t):
    if t.dtype == torch.float32:
        return _lib.F32
    if t.dtype == torch.bfloat16:
        return _lib.BF16
    raise _lib.MbemaError("unsupported dtype %s (float32 or bfloat16 expected)" % t.dtype)


def _f32_or_bf16(t):
    return t if t.dtype in (torch.float32, torch.bfloat16) else t.float()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _workspace(nbytes, device):
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


class _Telemetry:
    """Optional bookkeeping for the benchmark: kernel-launch counts per entry point and CUDA-event pairs around
    selected entry points (recorded on the launching stream)."""

    # kernels launched by one call of each C entry point
    KERNELS = {"mbema_query_scan": 2, "mbema_tile_states": 4, "mbema_qgate_fwd": 1, "mbema_qgate_bwd": 2,
               "mbema_flash_fwd": 1, "mbema_flash_bwd": 2}

    def __init__(self):
        self.enabled = False
        self.launches = 0
        self.events = {}

    def reset(self):
        self.launches = 0
        self.events = {}

    def begin(self, name):
        if not self.enabled:
            return None
        self.launches += self.KERNELS[name]
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(torch.cuda.current_stream())
        return ev

    def end(self, name, ev):
        if ev is None:
            return
        ev1 = torch.cuda.Event(enable_timing=True)
        ev1.record(torch.cuda.current_stream())
        self.events.setdefault(name, []).append((ev, ev1))

    def elapsed_ms(self, name):
        """Per-call device times (ms) of an entry point; call after a synchronize."""
        return [a.elapsed_time(b) for a, b in self.events.get(name, [])]


telemetry = _Telemetry()

# Workspaces of the tensor-core entry points, one per (device, stream), kept for the life of the process.  Their first
# int32 is the kernels' status word: the kernels OR into it and nothing clears it until clear_status(), so a bounded
# wait that gave up in any call of a step is still visible when the step ends.
_tc_workspaces = {}


def _tc_workspace(nbytes, device):
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    ws = _tc_workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        new = torch.zeros(max(int(nbytes), 4096), dtype=torch.uint8, device=device)
        if ws is not None:
            new[:4].copy_(ws[:4])          # carry the status word over
        _tc_workspaces[key] = ws = new
    return ws


def device_status(device=None):
    """Status of the tensor-core kernels on `device` (default: the current one) since the last clear_status();
    synchronises.  0 = ok; otherwise bit 0 says that a bounded wait inside a kernel gave up (bits 8.. name the wait)
    and the results produced since then are invalid."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    st = 0
    for (d, _), ws in _tc_workspaces.items():
        if d == dev:
            st |= int(ws[:4].view(torch.int32).item())
    return st


def status_word(device=None):
    """The status of device_status() as a device tensor (int32 [1]), without synchronising: copy it to the host together
    with a step's results and test it there."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    words = [ws[:4].view(torch.int32) for (d, _), ws in _tc_workspaces.items() if d == dev]
    if not words:
        return torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", dev))
    out = words[0]
    for w in words[1:]:
        out = out | w
    return out


def check_status(device=None):
    """Raise if a tensor-core kernel reported a failed wait since the last clear_status() (synchronises)."""
    st = device_status(device)
    if st:
        raise _lib.MbemaError("a bounded wait inside a tensor-core kernel gave up (status 0x%x): results since the last "
                              "check are invalid" % st)


def clear_status(device=None):
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    for (d, _), ws in _tc_workspaces.items():
        if d == dev:
            ws[:4].zero_()


# The index workspace (token order, chain heads) of the last chunk that went through the scan or the snapshots, kept so
# that the second of the two calls the model makes on a chunk does not sort it again.  The key names the tensor's storage,
# its version counter (in-place writes bump it), its shape and the stream the workspace was filled on; the cache holds a
# reference to the tensor, so no other tensor can sit at that address while the entry is alive.
_index_cache = {"key": None, "ws": None, "x": None}     # "x" keeps the tensor alive: its address cannot be handed to another one


def _index_key(x):
    return (x.data_ptr(), x._version, tuple(x.shape), x.device.index, torch.cuda.current_stream(x.device).cuda_stream)


# ---------------------------------------------------------------------------------------------
# query-side scan
# ---------------------------------------------------------------------------------------------
@_on_tensor_device
def compute_query_ema_history(x, rhos, vocab_size, c_init=None, c_init_keys=None, doc_ids=None):
    """C_seq[b, t, :] = EMA state of token x[b, t] just before step t, float32 [B, L, N].

    Drop-in for mathbrain/triton_ema_query.py:120.  ``vocab_size`` is accepted for signature compatibility; no
    vocabulary-sized buffer is used.  When a key occurs more than once in ``c_init_keys`` (the collate function
    pads the list with token 0) the first entry wins.
    """
    _require_cuda(x, rhos, c_init, c_init_keys, doc_ids)
    lib = _lib.load()
    B, L = x.shape
    N = rhos.shape[0]
    x = x.long().contiguous()
    rhos = rhos.float().contiguous()
    K = 0
    if c_init is not None and c_init_keys is not None:
        c_init = c_init.float().contiguous()
        c_init_keys = c_init_keys.long().contiguous()
        K = c_init_keys.shape[1]
        if c_init.shape != (B, K, N):
            raise _lib.MbemaError("c_init must be [B, K, N] matching c_init_keys [B, K]")
    else:
        c_init = c_init_keys = None
    if doc_ids is not None:
        doc_ids = doc_ids.to(torch.int32).contiguous()
    C_seq = torch.empty(B, L, N, dtype=torch.float32, device=x.device)
    ws = _workspace(lib.mbema_query_scan_workspace_bytes(B, L), x.device)
    flags = 0
    _ev = telemetry.begin("mbema_query_scan")
    rc = lib.mbema_query_scan(_ptr(x), _ptr(rhos), _ptr(c_init), _ptr(c_init_keys), _ptr(doc_ids), _ptr(C_seq),
                              B, L, N, K, flags, _ptr(ws), ws.numel(), _stream())
    telemetry.end("mbema_query_scan", _ev)
    _lib.check(rc, "mbema_query_scan")
    # the token order of this chunk stays in `ws`: precompute_boundaries on the same x (mathbrain/model.py:157, :180) reuses it
    _index_cache["key"], _index_cache["ws"], _index_cache["x"] = _index_key(x), ws, x
    return C_seq


# ---------------------------------------------------------------------------------------------
# slot-state snapshots (the handle the model passes around as "C_bounds")
# ---------------------------------------------------------------------------------------------
@dataclass
class TileStates:
    """Opaque result of precompute_boundaries, consumed by FlashEMAFunction."""
    tile_state: torch.Tensor            # [B, nT, K, N] f32 view of a buffer that also holds a 16-bit copy behind it
    tok_state: torch.Tensor             # [B, T, N] f32
    kcount: torch.Tensor                # [2B] i32: valid-slot counts, then the sample order (heaviest first)
    seq_lens: Optional[torch.Tensor]    # [B] i32 or None
    unique: torch.Tensor                # [B, K] i64, the slot list the snapshots were built for
    shape: tuple                        # (B, T, K, N)


@_on_tensor_device
def precompute_boundaries(x, unique_tensor, rhos, Br, c_init=None, doc_ids=None, seq_lens=None):
    """Slot-state snapshots per time tile; drop-in for mathbrain/triton_flash_ema.py:81.

    ``Br`` (the reference's tile length) is accepted and ignored: the tile length is a property of the kernels
    (128 steps).  ``doc_ids`` must be None, as in every call the reference makes (mathbrain/model.py:180; the
    attention wrappers always run with has_doc_ids=False, mathbrain/triton_flash_ema.py:553-559).
    ``seq_lens`` (extension, int tensor [B]) marks the valid length of every row; later steps are skipped by the
    attention kernels.
    """
    if doc_ids is not None:
        raise NotImplementedError("precompute_boundaries: doc_ids is not supported (chunks are single-document)")
    _require_cuda(x, unique_tensor, rhos, c_init, seq_lens)
    lib = _lib.load()
    B, L = x.shape
    K = unique_tensor.shape[1]
    N = rhos.shape[0]
    x = x.long().contiguous()
    unique = unique_tensor.long().contiguous()
    rhos = rhos.float().contiguous()
    if c_init is not None:
        c_init = c_init.float().contiguous()
        if c_init.shape != (B, K, N):
            raise _lib.MbemaError("c_init must be [B, K, N] matching unique_tensor [B, K]")
    nT = (L + _lib.TILE_T - 1) // _lib.TILE_T
    n_el = B * nT * K * N
    tile_buf = torch.empty(n_el * 6 + 16, dtype=torch.uint8, device=x.device)   # fp32 block, then the 16-bit copy
    tile_state = tile_buf[: n_el * 4].view(torch.float32).view(B, nT, K, N)
    tok_state = torch.empty(B, L, N, dtype=torch.float32, device=x.device)
    kcount = torch.empty(2 * B, dtype=torch.int32, device=x.device)   # counts, then samples by decreasing count
    flags = _lib.FLAG_CBASE_EXTRA_DECAY if _OPTIONS["cbase_extra_decay"] else 0
    if _index_cache["key"] == _index_key(x) and _index_cache["ws"] is not None:
        ws = _index_cache["ws"]               # the sort of this very x, left by compute_query_ema_history
        flags |= _lib.FLAG_INDEX_READY
    else:
        ws = _workspace(lib.mbema_tile_states_workspace_bytes(B, L), x.device)
        _index_cache["key"], _index_cache["ws"], _index_cache["x"] = _index_key(x), ws, x
    _ev = telemetry.begin("mbema_tile_states")
    rc = lib.mbema_tile_states(_ptr(x), _ptr(unique), _ptr(rhos), _ptr(c_init), _ptr(tile_state), _ptr(tok_state),
                               _ptr(kcount), B, L, N, K, flags, _ptr(ws), ws.numel(), _stream())
    telemetry.end("mbema_tile_states", _ev)
    _lib.check(rc, "mbema_tile_states")
    if seq_lens is not None:
        seq_lens = seq_lens.to(torch.int32).contiguous()
    return TileStates(tile_state, tok_state, kcount, seq_lens, unique, (B, L, K, N))


def _build_unique_index(x, device=None):
    """Per-row sorted unique tokens packed to the front, -1 padding; K_max = max(count, 16).
    Drop-in for mathbrain/triton_flash_ema.py:475 (the fallback used when the data loader gives no slot list)."""
    _require_cuda(x)
    B, L = x.shape
    xs, _ = torch.sort(x, dim=1)
    first = torch.ones_like(xs, dtype=torch.bool)
    first[:, 1:] = xs[:, 1:] != xs[:, :-1]
    counts = first.sum(1)
    k_max = max(int(counts.max().item()), 16)
    rank = torch.cumsum(first.long(), 1) - 1
    out = torch.full((B, max(k_max, L)), -1, dtype=x.dtype, device=x.device)
    src = torch.where(first, xs, torch.full_like(xs, -1))
    idx = torch.where(first, rank, torch.full_like(rank, max(k_max, L) - 1))
    # non-first entries all write -1 into the last column, which is -1 unless the row has L distinct tokens,
    # in which case no non-first entry exists
    out.scatter_(1, idx, src)
    return out[:, :k_max].contiguous(), k_max


# ---------------------------------------------------------------------------------------------
# flash-EMA attention
# ---------------------------------------------------------------------------------------------
def _flash_mode(H, N, K):
    """Compute mode of an attention call under the current options."""
    m = _OPTIONS["mode"]
    if m == "auto":
        return _lib.MODE_TC_BF16 if _lib.load().mbema_flash_tc_supported(H, N, K) else _lib.MODE_FP32
    return _MODES[m]


def _flash_flags(use_silu):
    f = _lib.FLAG_SILU if use_silu else 0
    if _OPTIONS["inactive_mass"] == "listed_only":
        f |= _lib.FLAG_LISTED_ONLY
    if _OPTIONS["fp32_backward"]:
        f |= _lib.FLAG_FP32_BACKWARD
    if _OPTIONS["_test_withhold_arrive"]:      # test hook of the tensor-core forward (see include/mbema.h)
        f |= _lib.FLAG_TEST_WITHHOLD_ARRIVE
    return f


class FlashEMAFunction(torch.autograd.Function):
    """O = flash-EMA gated cross-attention; drop-in for mathbrain/triton_flash_ema.py:571.

    forward(Q[B,H,L,hd], x[B,L], E_k_active[B,K_max,D], E_v_active[B,K_max,D], W_pe[N,D], rhos[N], V_total,
            unique_tensor[B,K_max] (-1 = pad), K_max, C_bounds (from precompute_boundaries), use_silu, Br)
    returns O[B,H,L,hd] float32; backward returns (dQ, None, dE_k, dE_v, dW_pe, None x 7).
    """

    @staticmethod
    @_on_tensor_device
    def forward(ctx, Q, x, E_k_active, E_v_active, W_pe, rhos, V_total, unique_tensor, K_max, C_bounds,
                use_silu=True, Br=64):
        _require_cuda(Q, x, E_k_active, E_v_active, W_pe, rhos, unique_tensor)
        if not isinstance(C_bounds, TileStates):
            raise _lib.MbemaError("C_bounds must come from mathbrain_b200.precompute_boundaries")
        lib = _lib.load()
        B, H, L, hd = Q.shape
        D = H * hd
        N = rhos.shape[0]
        # the reference forces K_max >= 16 and then slices the slot list to K_max columns (mathbrain/model.py:169-171);
        # a list narrower than that arrives with its own width, which is what counts here
        K = min(int(K_max), unique_tensor.shape[1])
        if C_bounds.shape != (B, L, K, N):
            raise _lib.MbemaError("C_bounds was built for (B,L,K,N)=%s, operator called with %s"
                                  % (C_bounds.shape, (B, L, K, N)))
        Qc = _f32_or_bf16(Q).contiguous()
        Ek = _f32_or_bf16(E_k_active).contiguous()
        Ev = _f32_or_bf16(E_v_active).contiguous()
        if Ev.dtype != Ek.dtype:
            Ev = Ev.to(Ek.dtype)
        if Ek.shape != (B, K, D) or Ev.shape != (B, K, D):
            raise _lib.MbemaError("E_k_active / E_v_active must be [B, K_max, D]")
        W = W_pe.float().contiguous()
        if W.shape != (N, D):
            raise _lib.MbemaError("W_pe must be [N, D]")
        rh = rhos.float().contiguous()
        xx = x.long().contiguous()
        O = torch.empty(B, H, L, hd, dtype=torch.float32, device=Q.device)
        LSE = torch.empty(B, H, L, dtype=torch.float32, device=Q.device)
        mode = _flash_mode(H, N, K)
        flags = _flash_flags(use_silu)
        need = lib.mbema_flash_fwd_workspace_bytes(B, H, L, hd, N, K, mode)
        ws = _tc_workspace(need, Q.device) if mode == _lib.MODE_TC_BF16 else _workspace(need, Q.device)
        _ev = telemetry.begin("mbema_flash_fwd")
        rc = lib.mbema_flash_fwd(_ptr(Qc), _dt(Qc), _ptr(xx), _ptr(Ek), _ptr(Ev), _dt(Ek), _ptr(W), _ptr(rh),
                                 _ptr(C_bounds.unique), _ptr(C_bounds.tile_state), _ptr(C_bounds.tok_state),
                                 _ptr(C_bounds.kcount), _ptr(C_bounds.seq_lens), _ptr(O), _ptr(LSE),
                                 B, H, L, hd, N, K, int(V_total), flags, mode, _ptr(ws), ws.numel(), _stream())
        telemetry.end("mbema_flash_fwd", _ev)
        _lib.check(rc, "mbema_flash_fwd")
        ctx.save_for_backward(Qc, xx, Ek, Ev, W, rh, O, LSE)
        ctx.handle = C_bounds
        ctx.meta = (B, H, L, hd, N, K, int(V_total), flags, mode)
        ctx.in_dtypes = (Q.dtype, E_k_active.dtype, E_v_active.dtype, W_pe.dtype)
        return O

    @staticmethod
    @_on_tensor_device
    def backward(ctx, dO):
        lib = _lib.load()
        Qc, xx, Ek, Ev, W, rh, O, LSE = ctx.saved_tensors
        h = ctx.handle
        B, H, L, hd, N, K, V_total, flags, mode = ctx.meta
        if _OPTIONS["_test_withhold_arrive"]:      # test hook of the tensor-core backward, read at call time
            flags |= _lib.FLAG_TEST_WITHHOLD_ARRIVE
        D = H * hd
        dOc = _f32_or_bf16(dO).contiguous()
        dQ = torch.empty(B, H, L, hd, dtype=torch.float32, device=dO.device)
        dEk = torch.empty(B, K, D, dtype=torch.float32, device=dO.device)
        dEv = torch.empty(B, K, D, dtype=torch.float32, device=dO.device)
        dW = torch.empty(N, D, dtype=torch.float32, device=dO.device)
        need = lib.mbema_flash_bwd_workspace_bytes(B, H, L, hd, N, K, mode)
        ws = _tc_workspace(need, dO.device) if mode == _lib.MODE_TC_BF16 else _workspace(need, dO.device)
        _ev = telemetry.begin("mbema_flash_bwd")
        rc = lib.mbema_flash_bwd(_ptr(Qc), _dt(Qc), _ptr(xx), _ptr(Ek), _ptr(Ev), _dt(Ek), _ptr(W), _ptr(rh),
                                 _ptr(h.unique), _ptr(h.tile_state), _ptr(h.tok_state), _ptr(h.kcount),
                                 _ptr(h.seq_lens), _ptr(O), _ptr(LSE), _ptr(dOc), _dt(dOc), _ptr(dQ), _ptr(dEk),
                                 _ptr(dEv), _ptr(dW), B, H, L, hd, N, K, V_total, flags, mode, _ptr(ws), ws.numel(),
                                 _stream())
        telemetry.end("mbema_flash_bwd", _ev)
        _lib.check(rc, "mbema_flash_bwd")
        qd, kd, vd, wd = ctx.in_dtypes
        return (dQ.to(qd), None, dEk.to(kd), dEv.to(vd), dW.to(wd), None, None, None, None, None, None, None)


@_on_tensor_device
def slot_grad_scatter(dE_k, dE_v, unique_tensor, out):
    """out[token] += dE_k[b, k] + dE_v[b, k] for every listed slot (b, k) holding `token` (unique_tensor < 0: skipped).

    dE_k, dE_v [B, K, D] (float32 or bfloat16; dE_v may be None), unique_tensor [B, K] int64, out [V, D] float32,
    accumulated in place and returned.  This is the embedding-table side of the attention backward: what autograd's
    backward of `F.embedding(safe_unique, E_slots)` (mathbrain/model.py:63-64) computes, for one layer's K and V rows
    in one pass over them."""
    _require_cuda(dE_k, dE_v, unique_tensor, out)
    if out.dtype != torch.float32 or not out.is_contiguous():
        raise _lib.MbemaError("slot_grad_scatter: `out` must be a contiguous float32 [V, D] tensor")
    a = _f32_or_bf16(dE_k).contiguous()
    b = None if dE_v is None else dE_v.to(a.dtype).contiguous()
    ut = unique_tensor.long().contiguous()
    R, D = ut.numel(), a.shape[-1]
    if a.numel() != R * D or out.shape[1] != D:
        raise _lib.MbemaError("slot_grad_scatter: shapes do not match")
    rc = _lib.load().mbema_slot_grad_scatter(_ptr(a), _ptr(b), _dt(a), _ptr(ut), _ptr(out), R, D, out.shape[0], _stream())
    _lib.check(rc, "mbema_slot_grad_scatter")
    return out


class SlotLayerNormFunction(torch.autograd.Function):
    """memory_base[u] = LayerNorm(E_slots[tokens[u]]) for the DISTINCT tokens of a batch (rows for FlashEMARowsFunction
    after k_proj / v_proj): `F.embedding(safe_unique, E_slots)` + `ln_kv` of mathbrain/model.py:63-65, once per token
    instead of once per sample and slot.  The backward returns the dense [V, D] embedding gradient (LayerNorm backward
    fused with the scatter) and the LayerNorm parameter gradients."""

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda")
    def forward(ctx, E_slots, tokens, ln_w, ln_b, eps=1e-5, out_dtype=None):
        _require_cuda(E_slots, tokens, ln_w, ln_b)
        lib = _lib.load()
        with torch.cuda.device(E_slots.device):
            E = _f32_or_bf16(E_slots).contiguous()
            tok = tokens.long().contiguous()
            w, b = ln_w.float().contiguous(), ln_b.float().contiguous()
            U, (V, D) = tok.numel(), E.shape
            if out_dtype is None:
                out_dtype = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else E.dtype
            if out_dtype not in (torch.float32, torch.bfloat16):
                out_dtype = torch.float32
            out = torch.empty(U, D, dtype=out_dtype, device=E.device)
            mu = torch.empty(U, dtype=torch.float32, device=E.device)
            rstd = torch.empty(U, dtype=torch.float32, device=E.device)
            rc = lib.mbema_slot_ln_fwd(_ptr(E), _dt(E), _ptr(tok), _ptr(w), _ptr(b), float(eps), _ptr(out), _dt(out),
                                       _ptr(mu), _ptr(rstd), U, D, V, _stream())
            _lib.check(rc, "mbema_slot_ln_fwd")
        ctx.save_for_backward(E, tok, w, mu, rstd)
        ctx.in_dtypes = (E_slots.dtype, ln_w.dtype, ln_b.dtype)
        return out

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, dY):
        E, tok, w, mu, rstd = ctx.saved_tensors
        lib = _lib.load()
        with torch.cuda.device(E.device):
            dYc = _f32_or_bf16(dY).contiguous()
            U, (V, D) = tok.numel(), E.shape
            dE = torch.zeros(V, D, dtype=torch.float32, device=E.device)
            dw = torch.zeros(D, dtype=torch.float32, device=E.device)
            db = torch.zeros(D, dtype=torch.float32, device=E.device)
            rc = lib.mbema_slot_ln_bwd(_ptr(dYc), _dt(dYc), _ptr(E), _dt(E), _ptr(tok), _ptr(w), _ptr(mu), _ptr(rstd),
                                       _ptr(dE), _ptr(dw), _ptr(db), U, D, V, _stream())
            _lib.check(rc, "mbema_slot_ln_bwd")
        ed, wd, bd = ctx.in_dtypes
        return dE.to(ed), None, dw.to(wd), db.to(bd), None, None


def project_slot_rows(E_slots, tokens, ln_kv, k_proj, v_proj):
    """(E_k_rows, E_v_rows) [U, D]: `k_proj(ln_kv(E_slots[tokens]))`, `v_proj(...)` over the distinct tokens of a batch
    (`tokens` from shared_slot_rows), the operands of FlashEMARowsFunction.  Same values as the rows of the reference's
    per-sample `E_k_active / E_v_active` (mathbrain/model.py:63-68), each computed once; gradients reach `E_slots`,
    `ln_kv`, `k_proj` and `v_proj` through autograd.  The two projections are library GEMMs, as in the reference."""
    mem = SlotLayerNormFunction.apply(E_slots, tokens, ln_kv.weight, ln_kv.bias, ln_kv.eps)
    return k_proj(mem), v_proj(mem)


def shared_slot_rows(unique_tensor):
    """Rows for slot-embedding tables shared between samples: returns (tokens[U] int64, row_index[B,K] int32) with
    tokens the sorted distinct tokens listed anywhere in `unique_tensor` (entries < 0 are padding) and
    tokens[row_index[b,k]] == unique_tensor[b,k] at every listed slot (0 at padded ones, never read)."""
    _require_cuda(unique_tensor)
    valid = unique_tensor >= 0
    tokens, inverse = torch.unique(unique_tensor[valid], return_inverse=True)
    row_index = torch.zeros(unique_tensor.shape, dtype=torch.int32, device=unique_tensor.device)
    row_index[valid] = inverse.to(torch.int32)
    return tokens, row_index


class FlashEMARowsFunction(torch.autograd.Function):
    """FlashEMAFunction with slot-embedding rows shared between samples (an extension: the reference always
    materialises per-sample [B,K_max,D] tensors, mathbrain/model.py:63-68).

    forward(Q[B,H,L,hd], x[B,L], E_k_rows[U,D], E_v_rows[U,D], row_index[B,K_max] int32, W_pe[N,D], rhos[N], V_total,
            unique_tensor[B,K_max], K_max, C_bounds, use_silu)
    Slot (b,k) reads row row_index[b,k] (see shared_slot_rows); the gradients of E_k_rows / E_v_rows are the sums over
    all slots sharing a row.  backward returns (dQ, None, dE_k_rows, dE_v_rows, None, dW_pe, None x 6)."""

    @staticmethod
    @_on_tensor_device
    def forward(ctx, Q, x, E_k_rows, E_v_rows, row_index, W_pe, rhos, V_total, unique_tensor, K_max, C_bounds,
                use_silu=True):
        _require_cuda(Q, x, E_k_rows, E_v_rows, row_index, W_pe, rhos, unique_tensor)
        if not isinstance(C_bounds, TileStates):
            raise _lib.MbemaError("C_bounds must come from mathbrain_b200.precompute_boundaries")
        lib = _lib.load()
        B, H, L, hd = Q.shape
        D = H * hd
        N = rhos.shape[0]
        K = min(int(K_max), unique_tensor.shape[1])
        if C_bounds.shape != (B, L, K, N):
            raise _lib.MbemaError("C_bounds was built for (B,L,K,N)=%s, operator called with %s"
                                  % (C_bounds.shape, (B, L, K, N)))
        Qc = _f32_or_bf16(Q).contiguous()
        Ek = _f32_or_bf16(E_k_rows).contiguous()
        Ev = _f32_or_bf16(E_v_rows).to(Ek.dtype).contiguous()
        U = Ek.shape[0]
        if Ek.dim() != 2 or Ek.shape[1] != D or Ev.shape != Ek.shape or U < 1:
            raise _lib.MbemaError("E_k_rows / E_v_rows must be [U, D] with U >= 1")
        if tuple(row_index.shape) != (B, K):
            raise _lib.MbemaError("row_index must be [B, K_max]")
        ri = row_index.to(torch.int32).contiguous()
        W = W_pe.float().contiguous()
        if W.shape != (N, D):
            raise _lib.MbemaError("W_pe must be [N, D]")
        rh = rhos.float().contiguous()
        xx = x.long().contiguous()
        O = torch.empty(B, H, L, hd, dtype=torch.float32, device=Q.device)
        LSE = torch.empty(B, H, L, dtype=torch.float32, device=Q.device)
        mode = _flash_mode(H, N, K)
        flags = _flash_flags(use_silu)
        need = lib.mbema_flash_fwd_workspace_bytes(B, H, L, hd, N, K, mode)
        ws = _tc_workspace(need, Q.device) if mode == _lib.MODE_TC_BF16 else _workspace(need, Q.device)
        _ev = telemetry.begin("mbema_flash_fwd")
        rc = lib.mbema_flash_fwd_rows(_ptr(Qc), _dt(Qc), _ptr(xx), _ptr(Ek), _ptr(Ev), _dt(Ek), _ptr(ri), U, _ptr(W),
                                      _ptr(rh), _ptr(C_bounds.unique), _ptr(C_bounds.tile_state),
                                      _ptr(C_bounds.tok_state), _ptr(C_bounds.kcount), _ptr(C_bounds.seq_lens),
                                      _ptr(O), _ptr(LSE), B, H, L, hd, N, K, int(V_total), flags, mode, _ptr(ws),
                                      ws.numel(), _stream())
        telemetry.end("mbema_flash_fwd", _ev)
        _lib.check(rc, "mbema_flash_fwd_rows")
        ctx.save_for_backward(Qc, xx, Ek, Ev, ri, W, rh, O, LSE)
        ctx.handle = C_bounds
        ctx.meta = (B, H, L, hd, N, K, U, int(V_total), flags, mode)
        ctx.in_dtypes = (Q.dtype, E_k_rows.dtype, E_v_rows.dtype, W_pe.dtype)
        return O

    @staticmethod
    @_on_tensor_device
    def backward(ctx, dO):
        lib = _lib.load()
        Qc, xx, Ek, Ev, ri, W, rh, O, LSE = ctx.saved_tensors
        h = ctx.handle
        B, H, L, hd, N, K, U, V_total, flags, mode = ctx.meta
        D = H * hd
        dOc = _f32_or_bf16(dO).contiguous()
        dQ = torch.empty(B, H, L, hd, dtype=torch.float32, device=dO.device)
        dEk = torch.empty(U, D, dtype=torch.float32, device=dO.device)
        dEv = torch.empty(U, D, dtype=torch.float32, device=dO.device)
        dW = torch.empty(N, D, dtype=torch.float32, device=dO.device)
        need = lib.mbema_flash_bwd_workspace_bytes(B, H, L, hd, N, K, mode)
        ws = _tc_workspace(need, dO.device) if mode == _lib.MODE_TC_BF16 else _workspace(need, dO.device)
        _ev = telemetry.begin("mbema_flash_bwd")
        rc = lib.mbema_flash_bwd_rows(_ptr(Qc), _dt(Qc), _ptr(xx), _ptr(Ek), _ptr(Ev), _dt(Ek), _ptr(ri), U, _ptr(W),
                                      _ptr(rh), _ptr(h.unique), _ptr(h.tile_state), _ptr(h.tok_state), _ptr(h.kcount),
                                      _ptr(h.seq_lens), _ptr(O), _ptr(LSE), _ptr(dOc), _dt(dOc), _ptr(dQ), _ptr(dEk),
                                      _ptr(dEv), _ptr(dW), B, H, L, hd, N, K, V_total, flags, mode, _ptr(ws),
                                      ws.numel(), _stream())
        telemetry.end("mbema_flash_bwd", _ev)
        _lib.check(rc, "mbema_flash_bwd_rows")
        qd, kd, vd, wd = ctx.in_dtypes
        return (dQ.to(qd), None, dEk.to(kd), dEv.to(vd), None, dW.to(wd), None, None, None, None, None, None)


# ---------------------------------------------------------------------------------------------
# query gate + LayerNorm
# ---------------------------------------------------------------------------------------------
class FusedGatingFunction(torch.autograd.Function):
    """x_ln = LayerNorm(x_q * gate(p_pre + bias)) * ln_w + ln_b, eps = 1e-5, float32 output.
    Drop-in for mathbrain/triton_fused_gating.py:122; backward returns (dx_q, dp_pre, dbias, dln_w, dln_b, None)."""

    @staticmethod
    @_on_tensor_device
    def forward(ctx, x_q, p_pre, bias, ln_w, ln_b, use_silu=True):
        _require_cuda(x_q, p_pre, bias, ln_w, ln_b)
        lib = _lib.load()
        B, L, D = x_q.shape
        xq = _f32_or_bf16(x_q).contiguous()
        pp = _f32_or_bf16(p_pre).contiguous()
        bb = bias.float().contiguous()
        lw = ln_w.float().contiguous()
        lb = ln_b.float().contiguous()
        rows = B * L
        y = torch.empty(B, L, D, dtype=torch.float32, device=x_q.device)
        mu = torch.empty(rows, dtype=torch.float32, device=x_q.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x_q.device)
        flags = _lib.FLAG_SILU if use_silu else 0
        _ev = telemetry.begin("mbema_qgate_fwd")
        rc = lib.mbema_qgate_fwd(_ptr(xq), _dt(xq), _ptr(pp), _dt(pp), _ptr(bb), _ptr(lw), _ptr(lb), 1e-5, _ptr(y),
                                 _lib.F32, _ptr(mu), _ptr(rstd), rows, D, flags, _stream())
        telemetry.end("mbema_qgate_fwd", _ev)
        _lib.check(rc, "mbema_qgate_fwd")
        ctx.save_for_backward(xq, pp, bb, lw, mu, rstd)
        ctx.flags = flags
        ctx.in_dtypes = (x_q.dtype, p_pre.dtype, bias.dtype, ln_w.dtype, ln_b.dtype)
        return y

    @staticmethod
    @_on_tensor_device
    def backward(ctx, dy):
        lib = _lib.load()
        xq, pp, bb, lw, mu, rstd = ctx.saved_tensors
        B, L, D = xq.shape
        rows = B * L
        dyc = _f32_or_bf16(dy).contiguous()
        dev = dy.device
        dx = torch.empty(B, L, D, dtype=torch.float32, device=dev)
        dp = torch.empty(B, L, D, dtype=torch.float32, device=dev)
        dbias = torch.empty(D, dtype=torch.float32, device=dev)
        dlw = torch.empty(D, dtype=torch.float32, device=dev)
        dlb = torch.empty(D, dtype=torch.float32, device=dev)
        ws = _workspace(lib.mbema_qgate_bwd_workspace_bytes(rows, D), dev)
        _ev = telemetry.begin("mbema_qgate_bwd")
        rc = lib.mbema_qgate_bwd(_ptr(dyc), _dt(dyc), _ptr(xq), _dt(xq), _ptr(pp), _dt(pp), _ptr(bb), _ptr(lw),
                                 _ptr(mu), _ptr(rstd), _ptr(dx), _ptr(dp), _ptr(dbias), _ptr(dlw), _ptr(dlb),
                                 rows, D, ctx.flags, _ptr(ws), ws.numel(), _stream())
        telemetry.end("mbema_qgate_bwd", _ev)
        _lib.check(rc, "mbema_qgate_bwd")
        d0, d1, d2, d3, d4 = ctx.in_dtypes
        return dx.to(d0), dp.to(d1), dbias.to(d2), dlw.to(d3), dlb.to(d4), None


def fused_apply_symmetric_query_gating(x_q, C_seq, pe_proj, ln_q, q_proj, use_silu=True):
    """Q = q_proj(LN(x_q * gate(pe_proj(C_seq + 1)))); drop-in for mathbrain/triton_fused_gating.py:179.
    The two projections are library GEMMs, as in the reference; the "+1" enters as the bias W.sum(1)."""
    _require_cuda(x_q, C_seq)
    bias_offset = pe_proj.weight.sum(dim=1)
    p_pre = pe_proj(C_seq)
    q_ln = FusedGatingFunction.apply(x_q, p_pre, bias_offset, ln_q.weight, ln_q.bias, use_silu)
    return q_proj(q_ln)
