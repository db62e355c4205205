"""Tokenizer, packed text dataset and data loaders on the checked-in assets (model: the reference's
tests/unit_tests/test_tokenizer.py, test_dataset_checkpointing.py)."""

import pytest
import torch

ASSETS = "tests/assets"


@pytest.fixture(scope="module")
def tok():
    from torchtitan_b200.components.tokenizer import HuggingFaceTokenizer

    return HuggingFaceTokenizer(tokenizer_path=f"{ASSETS}/tokenizer")


def test_tokenizer_round_trip_and_special_tokens(tok):
    text = "The quick brown fox jumps over the lazy dog."
    ids = tok.encode(text, add_bos=False, add_eos=False)
    assert ids and all(0 <= i < tok.get_vocab_size() for i in ids)
    assert tok.decode(ids).strip() == text
    with_special = tok.encode(text, add_bos=True, add_eos=True)
    assert len(with_special) >= len(ids)
    if tok.bos_id is not None:
        assert with_special[0] == tok.bos_id and ids[0] != tok.bos_id
    if tok.eos_id is not None:
        assert with_special[-1] == tok.eos_id
    vocab = tok.get_vocab()
    some = next(iter(vocab))
    assert tok.token_to_id(some) == vocab[some] and tok.id_to_token(vocab[some]) == some
    assert tok.vocab_size == tok.get_vocab_size() == len(vocab) or tok.vocab_size >= len(vocab)


def test_tokenizer_missing_path_raises():
    from torchtitan_b200.components.tokenizer import HuggingFaceTokenizer

    with pytest.raises(FileNotFoundError):
        HuggingFaceTokenizer(tokenizer_path=f"{ASSETS}/no_such_tokenizer")


def _dataset(tok, rank=0, world=1, seq=32, infinite=False):
    from torchtitan_b200.hf_datasets.text_datasets import HuggingFaceTextDataset

    return HuggingFaceTextDataset("c4_test", f"{ASSETS}/c4_test", tok, seq_len=seq, dp_rank=rank, dp_world_size=world,
                                  infinite=infinite)


def test_text_dataset_packs_documents_into_fixed_windows(tok):
    ds = _dataset(tok)
    it = iter(ds)
    rows = [next(it) for _ in range(5)]
    for inp, lab in rows:
        assert inp["input"].shape == (32,) and lab.shape == (32,) and inp["input"].dtype == torch.int64
        assert torch.equal(inp["input"][1:], lab[:-1])         # labels are the inputs shifted by one
    # consecutive windows continue the same token stream: the first label of a window is not re-fed as input later
    flat_first = torch.cat([r[0]["input"] for r in rows[:2]] + [rows[1][1][-1:]])
    assert flat_first.numel() == 65


def test_text_dataset_resumes_mid_stream(tok):
    ds = _dataset(tok)
    it = iter(ds)
    for _ in range(7):
        next(it)
    state = ds.state_dict()
    want = [next(it) for _ in range(4)]
    ds2 = _dataset(tok)
    ds2.load_state_dict(state)
    got = [x for _, x in zip(range(4), iter(ds2))]
    for (a, b), (c, d) in zip(want, got):
        assert torch.equal(a["input"], c["input"]) and torch.equal(b, d)


def test_text_dataset_shards_by_data_parallel_rank_and_reloops(tok):
    a = next(iter(_dataset(tok, rank=0, world=2)))
    b = next(iter(_dataset(tok, rank=1, world=2)))
    assert not torch.equal(a[0]["input"], b[0]["input"])
    finite = sum(1 for _ in _dataset(tok, seq=512))
    assert finite > 0
    inf = iter(_dataset(tok, seq=512, infinite=True))
    for _ in range(finite + 3):                                  # runs past the end by re-looping
        next(inf)
    with pytest.raises(ValueError):
        from torchtitan_b200.hf_datasets.text_datasets import HuggingFaceTextDataset

        HuggingFaceTextDataset("no_such_dataset", None, tok)


def test_parallel_aware_loader_batches_and_checkpoints_per_rank(tok):
    from torchtitan_b200.hf_datasets.text_datasets import HuggingFaceTextDataLoader

    def make(rank):
        return HuggingFaceTextDataLoader(HuggingFaceTextDataLoader.Config(dataset="c4_test", dataset_path=f"{ASSETS}/c4_test"),
                                         dp_world_size=2, dp_rank=rank, tokenizer=tok, seq_len=16, local_batch_size=3)

    dl = make(0)
    it = iter(dl)
    inp, lab = next(it)
    assert inp["input"].shape == (3, 16) and lab.shape == (3, 16)
    next(it)
    state = dl.state_dict()
    assert "dp_rank_0" in state and state["world_size"] == 2
    want = next(it)
    dl2 = make(0)
    dl2.load_state_dict(state)
    got = next(iter(dl2))
    assert torch.equal(want[0]["input"], got[0]["input"])
    other = make(1)
    other.load_state_dict(state)             # another rank's entry is ignored (with a warning), it starts from the beginning
    with pytest.raises(AssertionError):
        bad = dict(state)
        bad["world_size"] = 4
        make(0).load_state_dict(bad)
    # worker-only options are dropped when there are no workers; unknown loader options are rejected
    HuggingFaceTextDataLoader(HuggingFaceTextDataLoader.Config(dataset="c4_test", dataset_path=f"{ASSETS}/c4_test",
                                                               num_workers=0, persistent_workers=True, prefetch_factor=2),
                              dp_world_size=1, dp_rank=0, tokenizer=tok, seq_len=16, local_batch_size=1)
    from torchtitan_b200.components.dataloader import ParallelAwareDataloader

    with pytest.raises(ValueError, match="Invalid dataloader kwargs"):
        ParallelAwareDataloader(dl.dataset, dp_rank=0, dp_world_size=1, no_such_option=1)
    with pytest.raises(ValueError, match="'dataset' should not be passed"):
        ParallelAwareDataloader._validate_kwargs({"dataset": dl.dataset})


def test_synthetic_loader_is_seeded_per_rank_and_resumable():
    from torchtitan_b200.components.dataloader import SyntheticDataLoader

    def make(rank, **kw):
        return SyntheticDataLoader(SyntheticDataLoader.Config(seed=3, pin_memory=False, **kw), dp_world_size=2, dp_rank=rank,
                                   seq_len=8, local_batch_size=2, model_vocab_size=97)

    a, b = make(0), make(1)
    xa, la = next(iter(a))
    xb, _ = next(iter(b))
    assert xa["input"].shape == (2, 8) and int(xa["input"].max()) < 97
    assert torch.equal(xa["input"][:, 1:], la[:, :-1]) and not torch.equal(xa["input"], xb["input"])
    it = iter(a)
    next(it)
    state = a.state_dict()
    want = next(it)
    c = make(0)
    c.load_state_dict(state)
    assert torch.equal(next(iter(c))[0]["input"], want[0]["input"])
    assert len(list(make(0, num_batches=3))) == 3
