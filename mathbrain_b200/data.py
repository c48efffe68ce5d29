"""Data-side helpers of the path: the reference's chunking rule for a corpus of documents."""


def document_chunks(doc_lengths, block_size):
    """Chunk list of a corpus of documents with the given token counts, by the reference's rule
    (mathbrain/data.py:74-82): documents shorter than 2 tokens are dropped, a document of n tokens gives
    max(1, ceil((n - 1) / block_size)) chunks, chunk c covers tokens [c * block_size, min(c * block_size +
    block_size + 1, n)) -- one token more than the block for the shifted target -- and chunks never cross a document.
    Returns a list of (document index, first token, end token)."""
    out = []
    for d, n in enumerate(doc_lengths):
        n = int(n)
        if n < 2:
            continue
        n_chunks = max(1, (n - 1 + block_size - 1) // block_size)
        for c in range(n_chunks):
            cs = c * block_size
            ce = min(cs + block_size + 1, n)
            if ce - cs >= 2:
                out.append((d, cs, ce))
    return out
