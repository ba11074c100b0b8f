"""Token-file batches: a function of (seed, step) only, sharded over the data-parallel ranks, prefetched in the background."""
import numpy as np
import pytest
import torch

from cai_b200.utils.data import TokenBatches, open_tokens


@pytest.fixture()
def corpus(tmp_path):
    ids = (np.arange(50_000, dtype=np.uint32) * 7919 % 1000).astype(np.uint16)
    raw = tmp_path / "tokens.bin"
    ids.tofile(raw)
    npy = tmp_path / "tokens.npy"
    np.save(npy, ids.astype(np.uint32))
    return ids, raw, npy


def test_windows_are_next_token_pairs_of_the_file(corpus):
    ids, raw, _ = corpus
    src = TokenBatches(raw, vocab=1000, seq=64, rows_global=8, seed=3, prefetch=0)
    tok, tgt = src.make(5)
    assert tok.shape == tgt.shape == (8, 64) and tok.dtype == tgt.dtype == torch.int32
    assert torch.equal(tok[:, 1:], tgt[:, :-1])
    for row, off in zip(tok, src.offsets(5)):
        assert np.array_equal(row.numpy(), ids[off:off + 64].astype(np.int32))


def test_batch_depends_on_seed_and_step_only(corpus):
    _, raw, npy = corpus
    a = TokenBatches(raw, 1000, 32, 4, seed=11, prefetch=0)
    b = TokenBatches(npy, 1000, 32, 4, seed=11, prefetch=0)          # same ids, other container and width
    for s in (0, 1, 17):
        assert torch.equal(a.make(s)[0], b.make(s)[0])
    assert not torch.equal(a.make(0)[0], a.make(1)[0])
    assert not torch.equal(a.make(0)[0], TokenBatches(raw, 1000, 32, 4, seed=12, prefetch=0).make(0)[0])


def test_ranks_split_the_global_batch(corpus):
    _, raw, _ = corpus
    whole = TokenBatches(raw, 1000, 16, 8, seed=1, prefetch=0).make(9)
    parts = [TokenBatches(raw, 1000, 16, 8, seed=1, dp=4, dp_id=r, prefetch=0).make(9) for r in range(4)]
    assert torch.equal(torch.cat([p[0] for p in parts]), whole[0])
    assert torch.equal(torch.cat([p[1] for p in parts]), whole[1])
    with pytest.raises(ValueError):
        TokenBatches(raw, 1000, 16, 6, seed=1, dp=4)


def test_prefetch_serves_the_same_batches_and_restarts_on_a_jump(corpus):
    _, raw, _ = corpus
    src = TokenBatches(raw, 1000, 32, 4, seed=5, prefetch=2)
    ref = TokenBatches(raw, 1000, 32, 4, seed=5, prefetch=0)
    try:
        for s in (0, 1, 2, 3, 40, 41, 7):          # a resume lands on any step
            tok, tgt = src.get(s)
            want = ref.make(s)
            assert torch.equal(tok, want[0]) and torch.equal(tgt, want[1])
    finally:
        src.close()
    assert src._thread is None


def test_ids_outside_the_vocabulary_are_refused(corpus):
    _, raw, _ = corpus
    with pytest.raises(ValueError, match="vocabulary"):
        TokenBatches(raw, vocab=500, seq=32, rows_global=4, seed=0, prefetch=0).make(0)
    src = TokenBatches(raw, vocab=500, seq=32, rows_global=4, seed=0, prefetch=1)
    try:
        with pytest.raises(ValueError, match="vocabulary"):          # raised in the consumer, not lost in the thread
            src.get(0)
    finally:
        src.close()


def test_short_or_non_integer_files_are_refused(tmp_path):
    small = tmp_path / "small.bin"
    np.arange(10, dtype=np.uint16).tofile(small)
    with pytest.raises(ValueError, match="fewer"):
        TokenBatches(small, 1000, 32, 4, seed=0)
    bad = tmp_path / "bad.npy"
    np.save(bad, np.zeros(100, dtype=np.float32))
    with pytest.raises(ValueError, match="integers"):
        open_tokens(bad)


def test_byte_level_corpus_from_a_text_file(tmp_path):
    from cai_b200.utils.data import main
    text = tmp_path / "corpus.txt"
    text.write_bytes(bytes(range(256)) * 20)
    out = tmp_path / "corpus.bin"
    assert main([str(text), str(out)]) == 0
    ids = open_tokens(out)
    assert len(ids) == 256 * 20 and int(ids.max()) == 255
    tok, tgt = TokenBatches(out, vocab=256, seq=16, rows_global=2, seed=0, prefetch=0).make(0)
    assert torch.equal((tok[:, 1:]), tgt[:, :-1])
