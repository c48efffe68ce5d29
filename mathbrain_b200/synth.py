"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

Everything is generated on the host with explicit generators; nothing here computes the operators themselves
(the slot state handed over as ``c_base`` is the closed-form sum over the prefix occurrences, which is how the
data pipeline defines it: mathbrain/data.py:128-140 of the reference).
"""
import math

import numpy as np
import torch

VOCAB = 50257


def make_rhos(n_scales, min_hl=1024.0, max_hl=4096.0):
    """rho_n = exp(-ln 2 / h_n), h log-spaced (mathbrain/model.py:128-130 of the reference)."""
    hl = torch.logspace(math.log10(min_hl), math.log10(max_hl), n_scales)
    return torch.exp(-torch.log(torch.tensor(2.0)) / hl)


class Zipf:
    """i.i.d. tokens with p(rank r) ~ r^-s, r = 1..V, token id = r - 1."""

    def __init__(self, vocab=VOCAB, s=1.1):
        p = np.arange(1, vocab + 1, dtype=np.float64) ** (-s)
        self.cdf = np.cumsum(p / p.sum())
        self.vocab = vocab

    def draw(self, rng, n):
        return np.minimum(np.searchsorted(self.cdf, rng.random(n)), self.vocab - 1).astype(np.int64)


def bursty_tokens(rng, zipf, n, p_repeat=0.2, window=64):
    """Zipf tokens where, with probability p_repeat, a token of the previous `window` positions is re-emitted."""
    base = zipf.draw(rng, n)
    rep = rng.random(n) < p_repeat
    back = rng.integers(1, window + 1, n)
    out = base.copy()
    for i in range(1, n):
        if rep[i]:
            out[i] = out[max(0, i - int(back[i]))]
    return out


def prefix_state(prefix, keys, rhos64):
    """State seen at the first chunk step by every key after `prefix` (closed form, float64 -> float32)."""
    P = len(prefix)
    out = np.zeros((len(keys), len(rhos64)), np.float64)
    if P == 0:
        return out.astype(np.float32)
    order = {int(k): i for i, k in enumerate(keys)}
    idx = np.array([order.get(int(t), -1) for t in prefix])
    dist = (P - np.arange(P)).astype(np.float64)
    w = rhos64[None, :] ** dist[:, None]
    ok = idx >= 0
    np.add.at(out, idx[ok], w[ok])
    return out.astype(np.float32)


def make_chunk_batch(seed, B, T, N, vocab=VOCAB, max_prefix=8192, min_fill=64, bursty=False, min_hl=1024.0,
                     max_hl=4096.0, full_fill=False):
    """One batch of single-document chunks in the wire format the model consumes.

    Per sample: a prefix of U{0..max_prefix} tokens (history of the same document) and a chunk filled with
    U{min_fill..T} tokens (positions beyond the fill hold token 0).  ``unique_slots`` lists the chunk's sorted
    unique tokens first, then the sorted history-only tokens (mathbrain/data.py:104-124); ``c_base`` is the state
    each listed slot shows at chunk step 0.  Returns CPU tensors.
    """
    rng = np.random.Generator(np.random.PCG64(seed))
    zipf = Zipf(vocab)
    rhos = make_rhos(N, min_hl, max_hl)
    rhos64 = rhos.double().numpy()
    xs, uniqs, cbs, fills = [], [], [], []
    for _ in range(B):
        P = int(rng.integers(0, max_prefix + 1)) if max_prefix > 0 else 0
        fill = T if full_fill else int(rng.integers(min_fill, T + 1))
        doc = bursty_tokens(rng, zipf, P + fill) if bursty else zipf.draw(rng, P + fill)
        prefix, chunk = doc[:P], doc[P:]
        cu = np.unique(chunk)
        hu = np.setdiff1d(np.unique(prefix), cu) if P else np.zeros(0, np.int64)
        keys = np.concatenate([cu, hu])
        xs.append(np.concatenate([chunk, np.zeros(T - fill, np.int64)]))
        uniqs.append(keys)
        cbs.append(prefix_state(prefix, keys, rhos64))
        fills.append(fill)
    K = max(16, max(len(u) for u in uniqs))
    x = torch.from_numpy(np.stack(xs))
    unique_slots = torch.zeros(B, K, dtype=torch.long)
    pad_mask = torch.zeros(B, K, dtype=torch.bool)
    c_base = torch.zeros(B, K, N)
    for b in range(B):
        k = len(uniqs[b])
        unique_slots[b, :k] = torch.from_numpy(uniqs[b])
        pad_mask[b, :k] = True
        c_base[b, :k] = torch.from_numpy(cbs[b])
    return dict(x=x, unique_slots=unique_slots, pad_mask=pad_mask, c_base=c_base, rhos=rhos,
                fill=torch.tensor(fills, dtype=torch.int32), K_max=K, vocab=vocab)


def make_document_batch(seed, n_samples, T, N, vocab=VOCAB, median_len=1500.0, sigma=1.0, min_hl=1024.0, max_hl=4096.0):
    """`n_samples` chunks of synthetic documents with lognormal lengths exp(N(ln median_len, sigma)), Zipf(1.1)
    tokens, chunked per document by the reference's rule (data.document_chunks; no chunk crosses a document, the last
    chunk of a document is short), every chunk carrying the slot state of its own document's prefix as c_base.
    Documents are drawn until their chunks number n_samples; same wire format as make_chunk_batch, plus `doc` and
    `prefix_len` per sample."""
    from .data import document_chunks
    rng = np.random.Generator(np.random.PCG64(seed))
    zipf = Zipf(vocab)
    rhos = make_rhos(N, min_hl, max_hl)
    rhos64 = rhos.double().numpy()
    xs, uniqs, cbs, fills, docs, prefixes = [], [], [], [], [], []
    d = 0
    while len(xs) < n_samples:
        n = int(math.exp(rng.normal(math.log(median_len), sigma)))
        doc = zipf.draw(rng, max(n, 0))
        for _, cs, ce in document_chunks([n], T):
            if len(xs) == n_samples:
                break
            chunk = doc[cs:ce - 1]                       # inputs; the last token of the range is only a target
            prefix = doc[:cs]
            cu = np.unique(chunk)
            hu = np.setdiff1d(np.unique(prefix), cu) if cs else np.zeros(0, np.int64)
            keys = np.concatenate([cu, hu])
            xs.append(np.concatenate([chunk, np.zeros(T - len(chunk), np.int64)]))
            uniqs.append(keys)
            cbs.append(prefix_state(prefix, keys, rhos64))
            fills.append(len(chunk))
            docs.append(d)
            prefixes.append(cs)
        d += 1
    K = max(16, max(len(u) for u in uniqs))
    B = n_samples
    unique_slots = torch.zeros(B, K, dtype=torch.long)
    pad_mask = torch.zeros(B, K, dtype=torch.bool)
    c_base = torch.zeros(B, K, N)
    for b in range(B):
        k = len(uniqs[b])
        unique_slots[b, :k] = torch.from_numpy(uniqs[b])
        pad_mask[b, :k] = True
        c_base[b, :k] = torch.from_numpy(cbs[b])
    return dict(x=torch.from_numpy(np.stack(xs)), unique_slots=unique_slots, pad_mask=pad_mask, c_base=c_base, rhos=rhos,
                fill=torch.tensor(fills, dtype=torch.int32), K_max=K, vocab=vocab,
                doc=torch.tensor(docs, dtype=torch.int64), prefix_len=torch.tensor(prefixes, dtype=torch.int64))


def select_samples(batch, idx):
    """The sub-batch of `make_chunk_batch` output holding samples `idx`, slot lists trimmed to the subset's longest."""
    idx = torch.as_tensor(idx, dtype=torch.long)
    K = max(16, int(batch["pad_mask"][idx].sum(1).max()))
    out = dict(batch)
    for k in ("x", "fill", "doc", "prefix_len"):
        if k in batch:
            out[k] = batch[k][idx].contiguous()
    for k in ("unique_slots", "pad_mask", "c_base"):
        out[k] = batch[k][idx][:, :K].contiguous()
    out["K_max"] = K
    return out


def make_layer_weights(seed, B, K, D, N, T, H, std=0.02, dtype=torch.float32):
    """Random operands of one attention layer: Q [B,H,T,hd], E_k/E_v [B,K,D], W_pe [N,D], dO like Q."""
    g = torch.Generator().manual_seed(seed)
    hd = D // H
    return dict(Q=(torch.randn(B, H, T, hd, generator=g) * std).to(dtype),
                E_k=(torch.randn(B, K, D, generator=g) * std).to(dtype),
                E_v=(torch.randn(B, K, D, generator=g) * std).to(dtype),
                W_pe=torch.randn(N, D, generator=g) * std,
                dO=(torch.randn(B, H, T, hd, generator=g) * std).to(dtype))
