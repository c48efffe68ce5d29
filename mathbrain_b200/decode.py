"""Streaming decode: per-sequence slot state resident on the GPU, one new token per step.

    st = DecodeState(batch, vocab, rhos, capacity=4096, device="cuda")
    for t, tok in enumerate(stream):                 # tok: int64 [batch]
        O = st.attend(q, E_k, E_v, W_pe, t)          # [batch, H, 64] for every layer, BEFORE the update of step t
        C_q = st.update(tok, t)                      # query-side state of tok (for the query gate), then tok's slot += 1

The reference has no decode loop; this is one iteration of the loop body of its PyTorch attention
(mathbrain/flash_ema_attention.py:46-82) with the [V, N] state kept between steps.
"""
import torch

from . import _lib
from .ops import _dt, _ptr, _require_cuda, _stream, get_options


class DecodeState:
    def __init__(self, batch, vocab, rhos, capacity=4096, device="cuda"):
        _require_cuda(rhos)
        self.B, self.V, self.N, self.cap = int(batch), int(vocab), int(rhos.shape[0]), int(capacity)
        self.rhos = rhos.float().contiguous()
        dev = rhos.device if device is None else torch.device(device)
        self.state = torch.zeros(self.B, self.V, self.N, dtype=torch.float32, device=dev)
        self.last_t = torch.full((self.B, self.V), -1, dtype=torch.int32, device=dev)
        self.active = torch.zeros(self.B, self.cap, dtype=torch.int32, device=dev)
        self.n_active = torch.zeros(self.B, dtype=torch.int32, device=dev)
        self.overflow = torch.zeros(1, dtype=torch.int32, device=dev)
        self._ws = None
        self.t_dev = None        # device int32 step number (use_device_step): replaces the t_now arguments

    def use_device_step(self, t0=0):
        """Keep the step number in device memory from now on: attend / update ignore their t_now argument and
        advance() adds one, stream-ordered.  Nothing in a step then depends on a host value, so a whole step can be
        captured in a CUDA graph (torch.cuda.graph) and replayed; see capture_step."""
        self.t_dev = torch.tensor([int(t0)], dtype=torch.int32, device=self.state.device)
        return self.t_dev

    def advance(self):
        with torch.cuda.device(self.state.device):
            self._advance()

    def _advance(self):
        _lib.check(_lib.load().mbema_decode_advance(_ptr(self.t_dev), _stream()), "mbema_decode_advance")

    def capture_step(self, qs, E_ks, E_vs, W_pes, tok, use_silu=True, mode=None):
        """Capture one decode step (an attend per layer over the static tensors qs[l], E_ks[l], E_vs[l], W_pes[l],
        then the update with the static token tensor `tok`, then advance) in a CUDA graph.  Returns
        (graph, outputs, C_q): fill qs / tok in place, call graph.replay(), read outputs[l] and C_q.  Layers whose
        query depends on the previous layer's output need their own capture around this state's calls instead."""
        if self.t_dev is None:
            self.use_device_step(0)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):          # warm-up outside the capture: workspaces, kernel attributes
            rows = torch.arange(self.B, device=tok.device)
            tk = tok.long().clamp(0, self.V - 1)
            keep = (self.state[rows, tk].clone(), self.last_t[rows, tk].clone(), self.active.clone(),
                    self.n_active.clone(), self.t_dev.clone(), self.overflow.clone())
            for l in range(len(qs)):
                self.attend(qs[l], E_ks[l], E_vs[l], W_pes[l], 0, use_silu=use_silu, mode=mode)
            self.update(tok, 0)
            self.advance()
            self.state[rows, tk] = keep[0]            # undo the warm-up step: only the tokens' own rows were touched
            self.last_t[rows, tk] = keep[1]
            for dst, src in zip((self.active, self.n_active, self.t_dev, self.overflow), keep[2:]):
                dst.copy_(src)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            outs = [self.attend(qs[l], E_ks[l], E_vs[l], W_pes[l], 0, use_silu=use_silu, mode=mode) for l in range(len(qs))]
            C_q = self.update(tok, 0)
            self.advance()
        return graph, outs, C_q

    def attend(self, q, E_k, E_v, W_pe, t_now, V_total=None, use_silu=True, listed_only=False, mode=None):
        """O [B, H, 64] float32; see _attend.  Runs with the state's device current and refuses operands elsewhere."""
        for t in (q, E_k, E_v, W_pe):
            if t.device != self.state.device:
                raise _lib.MbemaError("decode: operand on %s, state on %s" % (t.device, self.state.device))
        with torch.cuda.device(self.state.device):
            return self._attend(q, E_k, E_v, W_pe, t_now, V_total, use_silu, listed_only, mode)

    def _attend(self, q, E_k, E_v, W_pe, t_now, V_total=None, use_silu=True, listed_only=False, mode=None):
        """O [B, H, 64] float32.  q [B, H, 64]; E_k, E_v [V, H*64] projected slot embeddings; W_pe [N, H*64].

        mode "fp32" (exact kernel) or "tc_bf16" (tensor cores; N = 64, H even); default: the package option `mode`,
        falling back to fp32 where the tensor-core kernel does not apply."""
        _require_cuda(q, E_k, E_v, W_pe)
        lib = _lib.load()
        B, H, hd = q.shape
        q = q.contiguous()
        E_k = E_k.contiguous()
        E_v = E_v.to(E_k.dtype).contiguous()
        W = W_pe.float().contiguous()
        O = torch.empty(B, H, hd, dtype=torch.float32, device=q.device)
        flags = (_lib.FLAG_SILU if use_silu else 0) | (_lib.FLAG_LISTED_ONLY if listed_only else 0)
        tc_ok = self.N == 64 and hd == 64 and H % 2 == 0
        if mode is None:
            mode = "tc_bf16" if (get_options()["mode"] in ("tc_bf16", "auto") and tc_ok) else "fp32"
        if mode == "tc_bf16":
            if E_k.dtype != torch.bfloat16:          # the kernel copies embedding rows as stored: keep bf16 tables to avoid this cast
                E_k, E_v = E_k.to(torch.bfloat16), E_v.to(torch.bfloat16)
            need = lib.mbema_decode_attend_tc_workspace_bytes(B, H, self.cap)
            if self._ws is None or self._ws.numel() < need:
                old = self._ws
                self._ws = torch.zeros(need, dtype=torch.uint8, device=q.device)   # its first int32 is the sticky status word
                if old is not None:
                    self._ws[:4].copy_(old[:4])
            rc = lib.mbema_decode_attend_tc(_ptr(q), _dt(q), _ptr(E_k), _ptr(E_v), _dt(E_k), _ptr(W), _ptr(self.rhos),
                                            _ptr(self.state), _ptr(self.last_t), _ptr(self.active),
                                            _ptr(self.n_active), _ptr(O), B, H, hd, self.V, self.N, self.cap,
                                            int(t_now), int(self.V if V_total is None else V_total), flags,
                                            _ptr(self.t_dev), _ptr(self._ws), self._ws.numel(), _stream())
            _lib.check(rc, "mbema_decode_attend_tc")
            return O
        if mode != "fp32":
            raise ValueError("mode must be 'fp32' or 'tc_bf16'")
        rc = lib.mbema_decode_attend(_ptr(q), _dt(q), _ptr(E_k), _ptr(E_v), _dt(E_k), _ptr(W), _ptr(self.rhos),
                                     _ptr(self.state), _ptr(self.last_t), _ptr(self.active), _ptr(self.n_active),
                                     _ptr(O), B, H, hd, self.V, self.N, self.cap, int(t_now),
                                     int(self.V if V_total is None else V_total), flags, _ptr(self.t_dev), _stream())
        _lib.check(rc, "mbema_decode_attend")
        return O

    def update(self, tok, t_now):
        """C_q [B, N]; see _update.  Runs with the state's device current and refuses a token tensor elsewhere."""
        if tok.device != self.state.device:
            raise _lib.MbemaError("decode: tokens on %s, state on %s" % (tok.device, self.state.device))
        with torch.cuda.device(self.state.device):
            return self._update(tok, t_now)

    def _update(self, tok, t_now):
        """Query-side state C_q [B, N] of the new tokens (before their update), then the slot update of step t_now."""
        _require_cuda(tok)
        lib = _lib.load()
        tok = tok.long().contiguous()
        C_q = torch.empty(self.B, self.N, dtype=torch.float32, device=tok.device)
        rc = lib.mbema_decode_update(_ptr(tok), _ptr(self.rhos), _ptr(self.state), _ptr(self.last_t), _ptr(self.active),
                                     _ptr(self.n_active), _ptr(C_q), _ptr(self.overflow), self.B, self.V, self.N,
                                     self.cap, int(t_now), _ptr(self.t_dev), _stream())
        _lib.check(rc, "mbema_decode_update")
        return C_q

    def device_status(self):
        """Status word of the tensor-core attend kernels since this state was created (synchronises): 0 = ok, else a
        bounded wait inside a kernel gave up and the outputs since then are invalid."""
        return 0 if self._ws is None else int(self._ws[:4].view(torch.int32).item())

    def check_overflow(self):
        """Synchronises; raises if an active list overflowed or a token was out of range."""
        code = int(self.overflow.item())
        if code:
            raise _lib.MbemaError("decode state: " + ("active-slot list full" if code == 1 else "token outside the vocabulary"))
