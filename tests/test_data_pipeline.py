"""Tokenizers, datasets, the data-parallel sampler and the prefetching loader (CPU)."""

import numpy as np
import pytest
import torch

from bitscom_b200.data import (ByteTokenizer, DistributedBatchSampler, PackedTokenDataset,
                               PrefetchLoader, SyntheticTokens, TextLineDataset, build_loader,
                               load_tokenizer, tokenize_to_file)


def test_byte_tokenizer_round_trip_and_specials():
    tok = ByteTokenizer()
    ids = tok.encode("héllo\t世界")
    assert ids[0] == tok.bos_id and ids[-1] == tok.eos_id and min(ids[1:-1]) >= 3
    assert tok.decode(ids) == "héllo\t世界" and max(ids) < tok.vocab_size
    assert tok.encode("", add_bos=False, add_eos=False) == []
    assert isinstance(load_tokenizer("bytes"), ByteTokenizer)
    with pytest.raises(FileNotFoundError):
        load_tokenizer("/nonexistent/tokenizer.model")


def test_sentencepiece_tokenizer_keeps_id_zero_for_padding(tmp_path):
    spm = pytest.importorskip("sentencepiece")
    corpus = tmp_path / "corpus.txt"
    corpus.write_text("\n".join(f"the quick brown fox {i} jumps over the lazy dog" for i in range(200)))
    prefix = str(tmp_path / "sp")
    spm.SentencePieceTrainer.train(input=str(corpus), model_prefix=prefix, vocab_size=64,
                                   model_type="bpe", minloglevel=2)
    tok = load_tokenizer(prefix + ".model")
    ids = tok.encode("the quick brown fox")
    assert tok.pad_id == 0 and 0 not in ids and max(ids) < tok.vocab_size
    assert tok.decode(ids) == "the quick brown fox"


def test_text_line_dataset_pads_and_truncates(tmp_path):
    path = tmp_path / "docs.txt"
    path.write_text("short\n\n" + "x" * 100 + "\nlast line\n")
    ds = TextLineDataset(str(path), ByteTokenizer(), seq_length=16)
    assert len(ds) == 3
    a, b = ds[0], ds[1]
    assert a.shape == (16,) and a.dtype == torch.int64
    assert a[0] == 1 and a[6] == 2 and a[7:].eq(0).all()      # bos s h o r t eos pad...
    assert b.ne(0).all() and b[0] == 1                         # truncated, no padding


def test_packed_token_dataset_windows(tmp_path):
    path = str(tmp_path / "tokens.bin")
    np.arange(1000, dtype="<u2").tofile(path)
    ds = PackedTokenDataset(path, seq_length=64)
    assert len(ds) == 15
    assert ds[0].tolist() == list(range(64)) and ds[14][0].item() == 14 * 64
    with pytest.raises(IndexError):
        ds[15]
    npy = str(tmp_path / "tokens.npy")
    np.save(npy, np.arange(300, dtype=np.int32))
    assert len(PackedTokenDataset(npy, 100)) == 3
    text = tmp_path / "t.txt"
    text.write_text("ab\ncd\n")
    out = str(tmp_path / "t.u16")
    assert tokenize_to_file(str(text), ByteTokenizer(), out) == 8
    assert PackedTokenDataset(out, 4)[0].tolist() == [1, 100, 101, 2]


@pytest.mark.parametrize("drop_last", [True, False])
def test_sampler_partitions_the_epoch_across_ranks(drop_last):
    n, batch, dp = 103, 4, 3
    per_rank = []
    for r in range(dp):
        s = DistributedBatchSampler(n, batch, dp, r, shuffle=True, seed=5, drop_last=drop_last)
        s.set_epoch(2)
        per_rank.append([i for b in s for i in b])
        assert all(len(b) == batch for b in s)
    lens = {len(x) for x in per_rank}
    assert len(lens) == 1                                  # same number of batches everywhere
    flat = [i for x in per_rank for i in x]
    if drop_last:
        assert len(flat) == (n // (batch * dp)) * batch * dp and len(set(flat)) == len(flat)
    else:
        assert set(flat) == set(range(n)) and len(flat) == -(-n // (batch * dp)) * batch * dp
    again = DistributedBatchSampler(n, batch, dp, 0, shuffle=True, seed=5, drop_last=drop_last)
    again.set_epoch(2)
    assert [i for b in again for i in b] == per_rank[0]      # deterministic
    again.set_epoch(3)
    assert [i for b in again for i in b] != per_rank[0]      # reshuffled per epoch
    with pytest.raises(ValueError):
        DistributedBatchSampler(5, 4, 2, 0)


def test_prefetch_loader_yields_every_batch_once_and_recycles_buffers():
    ds = SyntheticTokens(vocab_size=1000, seq_length=32, num_items=96, seed=3)
    sampler = DistributedBatchSampler(len(ds), 6, dp_size=2, dp_rank=1, shuffle=False)
    loader = PrefetchLoader(ds, sampler, micro_batches=3, micro_batch_size=2, depth=3, pin=False)
    assert len(loader) == 8
    want = [torch.stack([ds[i] for i in idx]).view(3, 2, 32) for idx in sampler]
    seen = []
    prev = None
    for k, batch in enumerate(loader):
        assert batch.shape == (3, 2, 32)
        assert torch.equal(batch, want[k])
        if prev is not None:                       # the previous buffer is still intact
            assert torch.equal(prev[0], prev[1])
        prev = (batch, batch.clone())
        loader.mark_consumed()
        seen.append(batch.data_ptr())
    assert len(seen) == 8 and len(set(seen)) <= 3   # a ring of three host buffers
    assert [torch.equal(a, b) for a, b in zip(loader, want)] == [True] * 8   # second epoch


def test_prefetch_loader_surfaces_dataset_errors():
    class Broken(SyntheticTokens):
        def __getitem__(self, idx):
            if idx == 7:
                raise RuntimeError("bad record")
            return super().__getitem__(idx)

    ds = Broken(100, 8, num_items=16)
    loader = PrefetchLoader(ds, DistributedBatchSampler(16, 4, shuffle=False), 2, 2, pin=False)
    with pytest.raises(RuntimeError, match="bad record"):
        list(loader)


def test_build_loader_from_text_and_token_files(tmp_path):
    text = tmp_path / "docs.txt"
    text.write_text("\n".join(f"document number {i}" for i in range(40)))
    loader = build_loader(str(text), "bytes", seq_length=24, vocab_size=32000, micro_batches=2,
                          micro_batch_size=2, dp_size=2, dp_rank=0, seed=1)
    batches = list(loader)
    assert len(batches) == 5 and batches[0].shape == (2, 2, 24)
    with pytest.raises(ValueError):
        build_loader(str(text), "bytes", seq_length=24, vocab_size=100, micro_batches=1,
                     micro_batch_size=1)
    tokens = str(tmp_path / "tok.u16")
    tokenize_to_file(str(text), ByteTokenizer(), tokens)
    packed = build_loader(tokens, "bytes", seq_length=16, vocab_size=32000, micro_batches=1,
                          micro_batch_size=4, shuffle=False)
    first = next(iter(packed))
    assert first.shape == (1, 4, 16) and first[0, 0, 0].item() == 1
    synth = build_loader("synthetic", "bytes", seq_length=8, vocab_size=50, micro_batches=1,
                         micro_batch_size=2)
    assert next(iter(synth)).max().item() < 50
