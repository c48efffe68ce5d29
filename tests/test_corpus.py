"""Corpus files and their streaming (CPU), and the states export against the reference's preprocessing loop (GPU)."""
import numpy as np
import pytest
import torch


def _documents(seed, n_docs, vocab, max_len):
    rng = np.random.Generator(np.random.PCG64(seed))
    return [rng.integers(0, vocab, int(rng.integers(0, max_len))).astype(np.int32) for _ in range(n_docs)]


def test_corpus_round_trip_and_reference_layout(tmp_path):
    from mathbrain_b200 import corpus
    docs = _documents(1, 9, 50, 40)
    corpus.write_corpus(docs, str(tmp_path))
    tokens, offsets = corpus.read_corpus(str(tmp_path))
    assert tokens.dtype == np.int32 and np.array_equal(np.asarray(tokens), np.concatenate(docs))
    assert offsets.tolist() == np.concatenate([[0], np.cumsum([len(d) for d in docs])]).tolist()
    # a directory as the reference writes it (no offsets file): boundaries come from doc_ids.bin; empty documents leave no trace there
    (tmp_path / "doc_offsets.bin").unlink()
    _, off2 = corpus.read_corpus(str(tmp_path))
    nonempty = [d for d in docs if len(d)]
    assert off2.tolist() == np.concatenate([[0], np.cumsum([len(d) for d in nonempty])]).tolist()


def test_stream_follows_the_chunk_rule(tmp_path):
    from mathbrain_b200 import corpus
    from mathbrain_b200.data import document_chunks
    docs = _documents(2, 12, 30, 70)
    corpus.write_corpus(docs, str(tmp_path))
    T, lanes = 16, 3
    seen = {}                                            # document start token -> list of (x, y) pieces, per lane order
    lane_doc = [None] * lanes
    order = []
    for step in corpus.CorpusStream(str(tmp_path), T, lanes):
        for b in range(lanes):
            if not step["active"][b]:
                assert int(step["fill"][b]) == 0
                continue
            if step["new_doc"][b]:
                lane_doc[b] = len(order)
                order.append([])
            n = int(step["fill"][b])
            assert n >= 1 and int(step["x"][b, n:].abs().sum()) == 0 and bool((step["y"][b, n:] == -100).all())
            order[lane_doc[b]].append((step["x"][b, :n].numpy().copy(), step["y"][b, :n].numpy().copy()))
    kept = [d for d in docs if len(d) >= 2]              # shorter documents give no chunk
    assert len(order) == len(kept)
    for pieces, d in zip(order, kept):
        chunks = document_chunks([len(d)], T)
        assert len(pieces) == len(chunks)
        for (px, py), (_, cs, ce) in zip(pieces, chunks):
            assert np.array_equal(px, d[cs:ce - 1]) and np.array_equal(py, d[cs + 1:ce])


@pytest.mark.gpu
def test_export_states_matches_the_preprocessing_loop(tmp_path):
    from mathbrain_b200 import corpus, synth
    docs = _documents(3, 7, 40, 90)
    corpus.write_corpus(docs, str(tmp_path))
    N = 8
    rhos = synth.make_rhos(N, 2.0, 50.0)
    states = corpus.export_states(str(tmp_path), rhos, block_size=32, lanes=3)
    # the reference's loop (mathbrain/data.py:277-303) restated: per document, state of the token's slot after its update
    r = rhos.double().numpy()
    want = []
    for d in docs:
        cur, last = {}, {}
        for t, v in enumerate(d.tolist()):
            cur[v] = cur[v] * r ** (t - last[v]) + 1.0 if v in cur else np.ones(N)
            last[v] = t
            want.append(cur[v].copy())
    want = np.stack(want) if want else np.zeros((0, N))
    assert states.shape == want.shape
    assert float(np.abs(np.asarray(states) - want).max() / np.abs(want).max()) < 1e-5
