"""GPU-side construction of the wire format the operators consume (`unique_slots`, `pad_mask`, `c_base`) from
per-document slot state that stays resident on the GPU.

The reference builds these per chunk on the host: `WikiTextMMapDataset.__getitem__` (mathbrain/data.py:95-148) looks
the document's history up in Python loops and reads `states.bin`, and `dynamic_collate_fn` (mathbrain/data.py:211-235)
pads and stacks.  Here a `ChunkFeeder` holds, for B documents in flight, the state of every slot after its last update
and the step of that update (the layout of `DecodeState`), and for the next chunk of every document

    batch = feeder.next_batch(x, fill)        # x [B, T] int64 on the GPU, fill [B] valid lengths
    ...   C_seq = compute_query_ema_history(x, rhos, V, batch["c_base"], batch["unique_slots"]); the model step ...
    feeder.advance(x, fill, C_seq)            # the documents move on by `fill` tokens

builds `unique_slots` (the chunk's sorted distinct tokens first, then the sorted history-only tokens: the order of
mathbrain/data.py:104-124), `pad_mask` and `c_base` (state decayed to the chunk's first step, mathbrain/data.py:128-140)
with sorts, searches and scatters on the device and one gather kernel (`mbema_slot_state_gather`); the only host
synchronisation is the read of the widest slot list, which the reference's model does as well (mathbrain/model.py:169).
"""
import torch

from . import _lib
from .ops import _ptr, _require_cuda, _stream


class ChunkFeeder:
    def __init__(self, n_docs, vocab, rhos, capacity=8192, device="cuda"):
        _require_cuda(rhos)
        dev = torch.device(device) if device is not None else rhos.device
        self.B, self.V, self.N, self.cap = int(n_docs), int(vocab), int(rhos.shape[0]), int(capacity)
        self.rhos = rhos.float().contiguous().to(dev)
        self.state = torch.zeros(self.B, self.V, self.N, dtype=torch.float32, device=dev)   # value after the last update
        self.last_t = torch.full((self.B, self.V), -1, dtype=torch.int32, device=dev)        # step of that update
        self.seen = torch.zeros(self.B, self.cap, dtype=torch.int64, device=dev)             # tokens seen so far, per document
        self.n_seen = torch.zeros(self.B, dtype=torch.int64, device=dev)
        self.t0 = torch.zeros(self.B, dtype=torch.int32, device=dev)                         # step of the next chunk's first token

    def reset(self, docs):
        """Start new documents in the given rows (a tensor or list of row numbers)."""
        docs = torch.as_tensor(docs, dtype=torch.long, device=self.state.device)
        self.state[docs] = 0
        self.last_t[docs] = -1
        self.n_seen[docs] = 0
        self.t0[docs] = 0

    def _chunk_uniques(self, x, fill):
        """Sorted distinct tokens of every chunk, padded with V: ([B, T] int64, counts [B])."""
        B, T = x.shape
        pos = torch.arange(T, device=x.device).unsqueeze(0)
        xs = torch.where(pos < fill.unsqueeze(1), x, torch.full_like(x, self.V))
        xs, _ = torch.sort(xs, dim=1)
        first = torch.ones_like(xs, dtype=torch.bool)
        first[:, 1:] = xs[:, 1:] != xs[:, :-1]
        first &= xs < self.V
        rank = torch.cumsum(first, dim=1) - 1                                   # position among the distinct tokens
        out = torch.full_like(xs, self.V)
        rows = torch.arange(B, device=x.device).unsqueeze(1).expand(B, T)
        out[rows[first], rank[first]] = xs[first]
        return out, first.sum(1)

    def next_batch(self, x, fill):
        """Wire format of the next chunk of every document: dict(unique_slots [B, K] int64 (0-padded, as the collate
        function pads), pad_mask [B, K] bool, c_base [B, K, N] float32, K_max).  x [B, T] int64, fill [B] valid lengths."""
        _require_cuda(x, fill)
        if x.device != self.state.device:
            raise _lib.MbemaError("ChunkFeeder: chunk on %s, state on %s" % (x.device, self.state.device))
        with torch.cuda.device(self.state.device):
            return self._next_batch(x, fill)

    def _next_batch(self, x, fill):
        B, T = x.shape
        dev = x.device
        fill = fill.to(torch.long)
        cu, n_cu = self._chunk_uniques(x, fill)                                  # [B, T] sorted, V-padded
        # history-only tokens: seen before and not in the chunk, sorted
        idx = torch.arange(self.cap, device=dev).unsqueeze(0)
        seen = torch.where(idx < self.n_seen.unsqueeze(1), self.seen, torch.full_like(self.seen, self.V))
        where = torch.searchsorted(cu, seen).clamp_max(T - 1)
        in_chunk = torch.gather(cu, 1, where) == seen
        hist = torch.where(in_chunk, torch.full_like(seen, self.V), seen)
        hist, _ = torch.sort(hist, dim=1)
        n_hist = (hist < self.V).sum(1)
        counts = n_cu + n_hist
        K = max(16, int(counts.max()))                                           # the one host synchronisation
        unique = torch.zeros(B, K, dtype=torch.int64, device=dev)
        col = torch.arange(K, device=dev).unsqueeze(0)
        take_cu = col < n_cu.unsqueeze(1)
        take_h = (~take_cu) & (col < counts.unsqueeze(1))
        cu_w = cu[:, :K] if cu.shape[1] >= K else torch.nn.functional.pad(cu, (0, K - cu.shape[1]), value=self.V)
        unique = torch.where(take_cu, cu_w, unique)
        hcol = (col - n_cu.unsqueeze(1)).clamp(0, self.cap - 1)
        unique = torch.where(take_h, torch.gather(hist, 1, hcol), unique)
        pad_mask = col < counts.unsqueeze(1)
        slots = torch.where(pad_mask, unique, torch.full_like(unique, -1))
        c_base = torch.empty(B, K, self.N, dtype=torch.float32, device=dev)
        rc = _lib.load().mbema_slot_state_gather(_ptr(self.state), _ptr(self.last_t), _ptr(slots), _ptr(self.t0),
                                                 _ptr(self.rhos), _ptr(c_base), B, K, self.V, self.N, _stream())
        _lib.check(rc, "mbema_slot_state_gather")
        return dict(unique_slots=unique, pad_mask=pad_mask, c_base=c_base, K_max=K)

    def advance(self, x, fill, C_seq):
        """Move every document past its chunk: the state of each token of the chunk becomes the query-side state at its
        LAST occurrence plus one (C_seq from compute_query_ema_history on this chunk), stamped with that step; tokens seen
        for the first time join the document's list.  Raises if a list would overflow."""
        _require_cuda(x, fill, C_seq)
        B, T = x.shape
        dev = x.device
        fill = fill.to(torch.long)
        pos = torch.arange(T, device=dev).unsqueeze(0).expand(B, T)
        valid = pos < fill.unsqueeze(1)
        key = torch.where(valid, x * T + pos, torch.full_like(x, self.V * T))
        key, _ = torch.sort(key, dim=1)
        tok, t = key // T, key % T
        last = torch.ones_like(valid)
        last[:, :-1] = tok[:, :-1] != tok[:, 1:]
        last &= tok < self.V
        rows = torch.arange(B, device=dev).unsqueeze(1).expand(B, T)
        b_i, tok_i, t_i = rows[last], tok[last], t[last]
        new = self.last_t[b_i, tok_i] < 0
        # append the new tokens to their documents' lists (rank among the document's new tokens, in token order)
        newm = torch.zeros_like(valid)
        newm[last] = new
        rank = torch.cumsum(newm, dim=1) - 1
        dst = self.n_seen.unsqueeze(1) + rank
        if bool((dst[newm] >= self.cap).any()):
            raise _lib.MbemaError("ChunkFeeder: the list of seen tokens is full (capacity %d)" % self.cap)
        self.seen[rows[newm], dst[newm]] = tok[newm]
        self.n_seen += newm.sum(1)
        self.state[b_i, tok_i] = C_seq[b_i, t_i].float() + 1.0
        self.last_t[b_i, tok_i] = (self.t0.long()[b_i] + t_i).to(torch.int32)
        self.t0 += fill.to(torch.int32)
