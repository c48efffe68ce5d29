"""Corpus files and their streaming into the feeder.

On-disk format: the reference's `tokens.bin` (int32, all documents concatenated) and `doc_ids.bin` (int32, document of
every token) as written by `preprocess_corpus` (mathbrain/data.py:242-320), plus `doc_offsets.bin` (int64, first token
of every document and the total).  The reference's other two files are not needed: `states.bin` (N floats per corpus
token, 26 GB per 100 M tokens at N = 64, filled by a Python loop over every token) is replaced by per-document state
that stays resident on the GPU (feeder.ChunkFeeder), and `pos_dict.pkl` (positions of every token) by the feeder's list
of seen tokens.  A directory written by the reference can be read as it is (the offsets are derived from `doc_ids.bin`).
`export_states` reproduces `states.bin` with the scan kernels for tools that still want it.
"""
import os

import numpy as np
import torch

from .data import document_chunks


def write_corpus(documents, data_dir):
    """documents: iterable of token-id sequences.  Writes tokens.bin, doc_ids.bin, doc_offsets.bin."""
    os.makedirs(data_dir, exist_ok=True)
    docs = [np.asarray(d, dtype=np.int32) for d in documents]
    offsets = np.zeros(len(docs) + 1, dtype=np.int64)
    offsets[1:] = np.cumsum([len(d) for d in docs])
    tokens = np.concatenate(docs) if docs else np.zeros(0, np.int32)
    doc_ids = np.repeat(np.arange(len(docs), dtype=np.int32), [len(d) for d in docs])
    tokens.tofile(os.path.join(data_dir, "tokens.bin"))
    doc_ids.tofile(os.path.join(data_dir, "doc_ids.bin"))
    offsets.tofile(os.path.join(data_dir, "doc_offsets.bin"))
    return offsets


def read_corpus(data_dir):
    """(tokens int32 memmap, offsets int64 [n_docs + 1])."""
    tokens = np.memmap(os.path.join(data_dir, "tokens.bin"), dtype=np.int32, mode="r")
    off_path = os.path.join(data_dir, "doc_offsets.bin")
    if os.path.exists(off_path):
        offsets = np.fromfile(off_path, dtype=np.int64)
    else:   # a directory written by the reference: document boundaries are where doc_ids changes
        doc_ids = np.memmap(os.path.join(data_dir, "doc_ids.bin"), dtype=np.int32, mode="r")
        cuts = np.flatnonzero(np.diff(doc_ids)) + 1
        offsets = np.concatenate([[0], cuts, [len(doc_ids)]]).astype(np.int64)
    return tokens, offsets


class CorpusStream:
    """Documents streamed through `lanes` rows, one chunk per row and step, chunked by the reference's rule
    (data.document_chunks): a row keeps its document until the document ends, then takes the next one.

    Iterating yields dicts of CPU tensors (pinned where a GPU is present): x [lanes, T] int64 (token 0 beyond `fill`), y [lanes, T] int64 targets
    (-100 beyond `fill`: the value the loss ignores), fill [lanes] int32, new_doc [lanes] bool (the row starts a new
    document: reset its state first), active [lanes] bool (False once the corpus is exhausted: fill 0)."""

    def __init__(self, data_dir, block_size, lanes, ignore_index=-100):
        self.tokens, self.offsets = read_corpus(data_dir)
        self.T, self.lanes, self.ignore = int(block_size), int(lanes), int(ignore_index)
        self.n_docs = len(self.offsets) - 1

    def __iter__(self):
        T, B = self.T, self.lanes
        next_doc = 0
        cur = [None] * B            # per row: (chunk list of its document, index of the next chunk, document start)
        while True:
            x = torch.zeros(B, T, dtype=torch.int64)
            y = torch.full((B, T), self.ignore, dtype=torch.int64)
            if torch.cuda.is_available():                    # pinned: the copies to the device can be asynchronous
                x, y = x.pin_memory(), y.pin_memory()
            fill = torch.zeros(B, dtype=torch.int32)
            new_doc = torch.zeros(B, dtype=torch.bool)
            active = torch.zeros(B, dtype=torch.bool)
            for b in range(B):
                while cur[b] is None and next_doc < self.n_docs:
                    lo, hi = int(self.offsets[next_doc]), int(self.offsets[next_doc + 1])
                    chunks = document_chunks([hi - lo], T)
                    next_doc += 1
                    if chunks:
                        cur[b] = (chunks, 0, lo)
                        new_doc[b] = True
                if cur[b] is None:
                    continue
                chunks, i, lo = cur[b]
                _, cs, ce = chunks[i]
                seg = torch.from_numpy(np.asarray(self.tokens[lo + cs:lo + ce], dtype=np.int64))
                n = len(seg) - 1                             # the last token of the range is only a target
                x[b, :n] = seg[:-1]
                y[b, :n] = seg[1:]
                fill[b] = n
                active[b] = True
                cur[b] = (chunks, i + 1, lo) if i + 1 < len(chunks) else None
            if not bool(active.any()):
                return
            yield dict(x=x, y=y, fill=fill, new_doc=new_doc, active=active)


def export_states(data_dir, rhos, block_size=512, lanes=32, device="cuda", out_name="states.bin"):
    """Write the reference's `states.bin` ([tokens, N] float32: the state of every token's own slot right after its
    update, mathbrain/data.py:291-303) by streaming the corpus through the feeder and the scan kernel: documents run in
    `lanes` rows, `block_size` tokens per row and step, each continuing from its own resident state."""
    from .feeder import ChunkFeeder
    from .ops import compute_query_ema_history
    tokens, offsets = read_corpus(data_dir)
    N = int(rhos.shape[0])
    V = int(tokens.max()) + 1 if len(tokens) else 1
    states = np.memmap(os.path.join(data_dir, out_name), dtype=np.float32, mode="w+", shape=(len(tokens), N))
    rhos = rhos.to(device)
    # documents in lanes; every step scans [lanes, T] tokens, the document's own prefix state coming from the feeder
    T, B = int(block_size), int(lanes)
    feeder = ChunkFeeder(B, V, rhos, capacity=min(V, 1 << 16), device=device)
    next_doc, cur = 0, [None] * B
    n_docs = len(offsets) - 1
    while True:
        x = torch.zeros(B, T, dtype=torch.int64)
        fill = torch.zeros(B, dtype=torch.int32)
        where = [None] * B
        fresh = []
        for b in range(B):
            if cur[b] is None and next_doc < n_docs:
                cur[b] = (int(offsets[next_doc]), int(offsets[next_doc + 1]))
                next_doc += 1
                fresh.append(b)
            if cur[b] is None:
                continue
            lo, hi = cur[b]
            n = min(T, hi - lo)
            x[b, :n] = torch.from_numpy(np.asarray(tokens[lo:lo + n], dtype=np.int64))
            fill[b] = n
            where[b] = (lo, n)
            cur[b] = (lo + n, hi) if lo + n < hi else None
        if all(w is None for w in where):
            break
        if fresh:
            feeder.reset(fresh)
        xd, fd = x.to(device), fill.to(device)
        batch = feeder.next_batch(xd, fd)
        C_seq = compute_query_ema_history(xd, rhos, V, batch["c_base"], batch["unique_slots"])
        feeder.advance(xd, fd, C_seq)
        host = (C_seq + 1.0).cpu().numpy()
        for b, w in enumerate(where):
            if w is not None:
                states[w[0]:w[0] + w[1]] = host[b, :w[1]]
    states.flush()
    return states
