"""Data layer: datasets over token files, loaders (order, sharding over ranks, resume), collation, mixtures (CPU)."""

import numpy as np
import pytest
import torch

from olmo_core_b200.data import (
    DataCollator,
    DataMix,
    NumpyDataLoaderConfig,
    NumpyFSLDataLoader,
    NumpyFSLDatasetConfig,
    NumpyPackedFSLDatasetConfig,
    NumpyPaddedFSLDatasetConfig,
    NumpyVSLDatasetConfig,
    PaddingDirection,
    SourceMixtureConfig,
    SourceMixtureDatasetConfig,
    SourceMixtureList,
    TokenizerConfig,
    VSLCurriculumConfig,
    VSLCurriculumType,
)

EOS, PAD, VOCAB = 1, 0, 1000


def _tok():
    return TokenizerConfig(vocab_size=VOCAB, eos_token_id=EOS, pad_token_id=PAD)


def _write_tokens(path, n_docs, rng, lo=5, hi=200):
    docs = []
    for _ in range(n_docs):
        n = int(rng.integers(lo, hi))
        docs.append(np.concatenate([rng.integers(2, VOCAB, n - 1), [EOS]]))
    arr = np.concatenate(docs).astype(np.uint16)
    mm = np.memmap(path, mode="w+", dtype=np.uint16, shape=arr.shape)
    mm[:] = arr
    mm.flush()
    return arr, [len(d) for d in docs]


@pytest.fixture
def token_files(tmp_path):
    rng = np.random.default_rng(0)
    out = []
    for i in range(3):
        p = tmp_path / f"part-{i}.npy"
        arr, lens = _write_tokens(p, 60 + 10 * i, rng)
        out.append((str(p), arr, lens))
    return out


def test_collator_pads_left_and_right_and_validates_vocab():
    items = [{"input_ids": torch.tensor([5, 6, 7]), "label_mask": torch.tensor([True, True, False])},
             {"input_ids": torch.tensor([8]), "label_mask": torch.tensor([True])}]
    right = DataCollator(pad_token_id=0)(items)
    assert right["input_ids"].tolist() == [[5, 6, 7], [8, 0, 0]] and right["label_mask"].tolist() == [[True, True, False], [True, False, False]]
    left = DataCollator(pad_token_id=0, pad_direction=PaddingDirection.left)(items)
    assert left["input_ids"].tolist() == [[5, 6, 7], [0, 0, 8]]
    with pytest.raises(ValueError):
        DataCollator(pad_token_id=0, vocab_size=8)(items)


def test_fsl_dataset_windows_and_doc_lengths(token_files, tmp_path):
    cfg = NumpyFSLDatasetConfig(tokenizer=_tok(), paths=[p for p, _, _ in token_files], sequence_length=64,
                                generate_doc_lengths=True, work_dir=str(tmp_path / "work"))
    ds = cfg.build()
    ds.prepare()
    assert len(ds) == sum(len(a) // 64 for _, a, _ in token_files)
    first = token_files[0][1]
    item = ds[1]
    assert item["input_ids"].tolist() == first[64:128].tolist()
    assert int(item["doc_lens"].sum()) == 64
    # the second file starts right after the whole windows of the first
    n0 = len(first) // 64
    assert ds[n0]["input_ids"].tolist() == token_files[1][1][:64].tolist()
    assert ds[-1]["input_ids"].tolist() == ds[len(ds) - 1]["input_ids"].tolist()
    with pytest.raises(IndexError):
        ds[len(ds)]
    assert len(ds.fingerprint) == 64


def test_padded_and_packed_datasets(token_files, tmp_path):
    paths = [p for p, _, _ in token_files]
    padded = NumpyPaddedFSLDatasetConfig(tokenizer=_tok(), paths=paths, sequence_length=128, work_dir=str(tmp_path / "w")).build()
    padded.prepare()
    assert len(padded) == sum(len(l) for _, _, l in token_files)
    lens0 = token_files[0][2]
    it = padded[0]
    n = min(lens0[0], 128)
    assert it["input_ids"].shape == (128,) and int(it["label_mask"].sum()) == n
    assert it["input_ids"][:n].tolist() == token_files[0][1][:n].tolist() and (it["input_ids"][n:] == PAD).all()

    packed = NumpyPackedFSLDatasetConfig(tokenizer=_tok(), paths=paths, sequence_length=256, work_dir=str(tmp_path / "w"),
                                         generate_doc_lengths=True).build()
    packed.prepare()
    total_docs = sum(len(l) for _, _, l in token_files)
    assert len(packed) < total_docs
    seen_tokens = 0
    for i in range(len(packed)):
        it = packed[i]
        assert it["input_ids"].shape == (256,)
        k = int(it["label_mask"].sum())
        seen_tokens += k
        assert (it["input_ids"][k:] == PAD).all()
        assert it["input_ids"][k - 1] == EOS  # whole documents only
    assert seen_tokens == sum(min(l, 256) for _, _, lens in token_files for l in lens)


def _loader(ds, tmp_path, rank=0, world=1, gbs=8 * 64, seed=3, **kw):
    return NumpyFSLDataLoader(ds, collator=DataCollator(pad_token_id=PAD), global_batch_size=gbs, work_dir=tmp_path / "lw",
                              seed=seed, dp_world_size=world, dp_rank=rank, fs_local_rank=0, **kw)


def test_fsl_loader_order_is_independent_of_world_size_and_resumable(token_files, tmp_path):
    ds = NumpyFSLDatasetConfig(tokenizer=_tok(), paths=[p for p, _, _ in token_files], sequence_length=64,
                               work_dir=str(tmp_path / "work")).build()
    ds.prepare()
    single = _loader(ds, tmp_path)
    single.reshuffle(1)
    batches = list(single)
    assert len(batches) == single.total_batches == len(ds) // 8 and single.batches_processed == len(batches)
    assert single.tokens_processed == len(batches) * 8 * 64
    # every instance at most once
    all_idx = torch.cat([b["index"] for b in batches])
    assert len(set(all_idx.tolist())) == len(all_idx)
    # two ranks see the interleaved halves of the same global batches
    halves = []
    for r in range(2):
        l = _loader(ds, tmp_path, rank=r, world=2)
        l.reshuffle(1)
        halves.append(list(l))
    for b, h0, h1 in zip(batches, halves[0], halves[1]):
        assert torch.equal(b["input_ids"][0::2], h0["input_ids"]) and torch.equal(b["input_ids"][1::2], h1["input_ids"])
    # random access == iteration
    assert torch.equal(single[3]["input_ids"], batches[3]["input_ids"])
    # resume in the middle of the epoch
    a = _loader(ds, tmp_path)
    a.reshuffle(1)
    it = iter(a)
    for _ in range(4):
        next(it)
    state = a.state_dict()
    b = _loader(ds, tmp_path)
    b.load_state_dict(state)
    b.reshuffle(b.epoch)
    rest = list(b)
    assert len(rest) == len(batches) - 4 and torch.equal(rest[0]["input_ids"], batches[4]["input_ids"])
    # a new epoch has a new order
    single.reset()
    single.reshuffle(2)
    assert not torch.equal(next(iter(single))["index"], batches[0]["index"])


def test_loader_batch_size_change_keeps_position(token_files, tmp_path):
    ds = NumpyFSLDatasetConfig(tokenizer=_tok(), paths=[p for p, _, _ in token_files], sequence_length=64,
                               work_dir=str(tmp_path / "work")).build()
    ds.prepare()
    ref = _loader(ds, tmp_path)
    ref.reshuffle(1)
    small = list(ref)
    l = _loader(ds, tmp_path)
    l.reshuffle(1)
    it = iter(l)
    next(it), next(it)
    l.global_batch_size = 16 * 64
    assert l.batches_processed == 1
    big = next(it)
    assert torch.equal(big["input_ids"], torch.cat([small[2]["input_ids"], small[3]["input_ids"]]))
    with pytest.raises(RuntimeError):
        l.batches_processed = 3
        l.global_batch_size = 32 * 64


def test_vsl_dataset_and_loader(token_files, tmp_path):
    cfg = NumpyVSLDatasetConfig(tokenizer=_tok(), paths=[p for p, _, _ in token_files], max_sequence_length=128,
                                min_sequence_length=16, work_dir=str(tmp_path / "work"),
                                vsl_curriculum=VSLCurriculumConfig(name=VSLCurriculumType.grow_p2, num_cycles=2, balanced=False))
    ds = cfg.build()
    loader = NumpyDataLoaderConfig(global_batch_size=256, seed=0, work_dir=str(tmp_path / "work")).build(ds)
    loader.reshuffle(1)
    lengths = ds.get_instance_lengths()
    assert set(np.unique(lengths).tolist()) <= {16, 32, 64, 128}
    n = 0
    for batch in loader:
        n += 1
        assert batch["input_ids"].numel() == 256
        if n == 1:
            assert batch["input_ids"].shape[1] == 128  # the longest bucket comes first
    assert n == loader.total_batches > 0


def test_source_mixture_respects_ratios(token_files, tmp_path):
    paths = [p for p, _, _ in token_files]
    mix = SourceMixtureDatasetConfig(
        source_list=SourceMixtureList(sources=[
            SourceMixtureConfig(source_name="a", target_ratio=0.75, paths=paths[:2], max_repetition_ratio=2.0),
            SourceMixtureConfig(source_name="b", target_ratio=0.25, paths=paths[2:]),
        ]),
        requested_tokens=64 * 64, global_batch_size=8 * 64, quiet=True, render_tables=False)
    ds = NumpyFSLDatasetConfig.from_src_mix(mix, tokenizer=_tok(), sequence_length=64, work_dir=str(tmp_path / "work")).build()
    ds.prepare()
    assert len(ds) == 64
    per_source = [hi - lo for lo, hi in ds.offsets]
    assert abs(sum(per_source[:-1]) / 64 - 0.75) < 0.1


def test_data_mix_manifests():
    paths, labels = DataMix.v3_small_ppl_validation.build("s3://bucket", "allenai/dolma2-tokenizer")
    assert len(paths) == 11 and labels[0] == "c4_en-validation"
    assert paths[0] == "s3://bucket/eval-data/perplexity/v3_small_dolma2-tokenizer/c4_en/val/part-0-00000.npy"
    assert DataMix("dolma3-0925-6T-mix") is DataMix.OLMo_mix_0925
    with pytest.raises(FileNotFoundError):
        DataMix.dolma17.build("s3://bucket", "x")
