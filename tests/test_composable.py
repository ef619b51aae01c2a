"""Composable data API: token / document / instance sources, mixing arithmetic, loader order, sharding and resume."""

import numpy as np
import pytest
import torch

from olmo_core_b200.data import TokenizerConfig
from olmo_core_b200.data.composable import (
    ComposableDataLoaderConfig,
    ConcatAndChunkInstanceSource,
    InMemoryDocumentSource,
    InMemoryTokenSource,
    MixingInstanceSource,
    MixingTokenSource,
    NumpyDocumentSource,
    PackingInstanceSource,
    RandomInstanceSource,
    ShuffleStrategy,
    calculate_sample_sizes,
    render_source,
)
from olmo_core_b200.data.composable.utils import build_global_indices
from olmo_core_b200.exceptions import OLMoConfigurationError


def test_token_source_composition(tmp_path):
    a = InMemoryTokenSource(list(range(100)), work_dir=tmp_path, label="a")
    b = InMemoryTokenSource(list(range(100, 150)), work_dir=tmp_path, label="b")
    cat = a + b
    assert cat.num_tokens == 150
    np.testing.assert_array_equal(cat[95:105]["input_ids"], np.arange(95, 105))
    head, tail = cat.split(0.4)
    assert (head.num_tokens, tail.num_tokens) == (60, 90)
    np.testing.assert_array_equal(tail[0:3]["input_ids"], [60, 61, 62])
    up = a.resize(2.5, seed=None)  # two whole passes + the first half
    assert up.num_tokens == 250
    np.testing.assert_array_equal(up[198:203]["input_ids"], [98, 99, 0, 1, 2])
    assert a.sample(max_tokens=10, seed=3).fingerprint != a.sample(max_tokens=10, seed=4).fingerprint


def test_document_sampling_keeps_documents_whole(tmp_path):
    rng = np.random.default_rng(0)
    tokens = []
    for n in rng.integers(2, 9, size=40):
        tokens += list(rng.integers(5, 50, size=n - 1)) + [0]
    docs = InMemoryDocumentSource(tokens, eos_token_id=0, work_dir=tmp_path)
    offsets = list(docs.get_document_offsets())
    assert len(offsets) == 40 and offsets[0][0] == 0 and offsets[-1][1] == len(tokens)
    half = docs.sample_by_docs(factor=0.5, seed=1)
    assert half.num_tokens <= len(tokens) // 2
    ids = half[0:half.num_tokens]["input_ids"]
    ends = [e for _, e in half.get_document_offsets()]
    assert all(ids[e - 1] == 0 for e in ends) and (ids == 0).sum() == len(ends)  # every piece is one whole document


def test_sample_size_arithmetic():
    # sizes 100 and 1000 at 50/50 without repetition: the small source caps the mix at 200
    np.testing.assert_array_equal(calculate_sample_sizes([100, 1000], [0.5, 0.5], [1.0, 1.0]), [100, 100])
    # allowing the small source to repeat 4x lifts the cap
    np.testing.assert_array_equal(calculate_sample_sizes([100, 1000], [0.5, 0.5], [4.0, 1.0]), [400, 400])
    with pytest.raises(OLMoConfigurationError):
        calculate_sample_sizes([100, 1000], [0.5, 0.5], [1.0, 1.0], target_size=600)
    with pytest.warns(UserWarning):
        out = calculate_sample_sizes([100, 100], [1.0, 3.0], [1.0, 1.0])
    assert out.tolist() == [33, 100]  # 1:3 with the larger share capped by its source


def test_mixing_and_visualization(tmp_path):
    a = InMemoryTokenSource(list(range(100)), work_dir=tmp_path, label="a")
    b = InMemoryTokenSource(list(range(100, 400)), work_dir=tmp_path, label="b")
    mix = MixingTokenSource(MixingTokenSource.Spec(source=a, ratio=0.5), MixingTokenSource.Spec(source=b, ratio=0.5),
                            work_dir=tmp_path, seed=0)
    assert mix.num_tokens == 200
    ids = mix[0:200]["input_ids"]
    assert (ids < 100).sum() == 100
    inst = ConcatAndChunkInstanceSource(mix, sequence_length=10, work_dir=tmp_path)
    text = render_source(inst)
    assert "MixingTokenSource" in text and "[a]" in text and text.count("SamplingTokenSource") == 2
    ia = ConcatAndChunkInstanceSource(a, sequence_length=10, work_dir=tmp_path)
    ib = ConcatAndChunkInstanceSource(b, sequence_length=10, work_dir=tmp_path)
    imix = MixingInstanceSource(MixingInstanceSource.Spec(source=ia, ratio=0.25),
                                MixingInstanceSource.Spec(source=ib, ratio=0.75), work_dir=tmp_path, seed=0,
                                num_instances=20)
    assert len(imix) == 20 and len(imix.sampled_sources[0]) == 5


def test_packing_never_splits_or_overflows(tmp_path):
    rng = np.random.default_rng(1)
    tokens = []
    for n in rng.integers(2, 12, size=60):
        tokens += list(rng.integers(5, 50, size=n - 1)) + [0]
    docs = InMemoryDocumentSource(tokens, eos_token_id=0, work_dir=tmp_path)
    packed = PackingInstanceSource(docs, sequence_length=16, pad_token_id=1, work_dir=tmp_path)
    seen = 0
    for inst in packed:
        ids, mask = inst["input_ids"], inst["label_mask"]
        assert len(ids) == 16 and (ids[~mask] == 1).all()
        real = ids[mask]
        assert real[-1] == 0  # the last real token closes a document
        seen += mask.sum()
    assert seen == len(tokens)  # nothing dropped (no document is longer than an instance)
    assert len(packed) < 60


def test_numpy_document_source(tmp_path):
    tok = TokenizerConfig.gpt2()
    data = np.concatenate([np.arange(1, 8), [tok.eos_token_id], np.arange(10, 15), [tok.eos_token_id]]).astype(np.uint16)
    paths = []
    for i in range(2):
        p = tmp_path / f"part-{i}.npy"
        (data + 0).tofile(p)
        paths.append(str(p))
    (src,) = NumpyDocumentSource.Config(source_paths=[str(tmp_path / "part-*.npy")], tokenizer=tok,
                                        source_group_size=2).build(tmp_path / "work")
    assert src.num_tokens == 2 * len(data)
    np.testing.assert_array_equal(src[len(data) - 2:len(data) + 3]["input_ids"], [14, tok.eos_token_id, 1, 2, 3])
    assert list(src.get_document_offsets()) == [(0, 8), (8, 14), (14, 22), (22, 28)]
    # per-file views, a config-level token count, and the config algebra of every document source config
    cfg = NumpyDocumentSource.Config(source_paths=[str(tmp_path / "part-*.npy")], tokenizer=tok)
    assert cfg.get_num_tokens() == 2 * len(data) and src.source_sizes == (len(data), len(data))
    first, second = src.split_by_source()
    assert first.source_paths == (paths[0],) and second.num_tokens == len(data) and src.dtype == np.uint16
    np.testing.assert_array_equal(second[:3]["input_ids"], [1, 2, 3])
    (half,) = cfg.resize(0.5, seed=None).build(tmp_path / "work")
    assert half.num_tokens == len(data)
    a, b = cfg.split(0.25)
    (a_src,), (b_src,) = a.build(tmp_path / "work"), b.build(tmp_path / "work")
    assert a_src.num_tokens == 7 and a_src.num_tokens + b_src.num_tokens == 2 * len(data)
    (both,) = (cfg + cfg).build(tmp_path / "work")
    assert both.num_tokens == 4 * len(data) and len(list(both.get_document_offsets())) == 8


def test_global_indices_are_stable_across_sequence_lengths():
    a = build_global_indices(8, sequence_length=8, max_sequence_length=8, seed=5)
    b = build_global_indices(16, sequence_length=4, max_sequence_length=8, seed=5)
    np.testing.assert_array_equal(b.reshape(8, 2), np.stack([a * 2, a * 2 + 1], axis=1))


def _loader(source, work_dir, rank=0, world=1, **kwargs):
    cfg = ComposableDataLoaderConfig(seed=1, num_threads=1, display_source_visualization=False, **kwargs)
    loader = cfg.build(source, work_dir=work_dir, tokenizer=TokenizerConfig.gpt2(), global_batch_size=8 * 8)
    loader.dp_rank, loader.dp_world_size = rank, world
    return loader


def test_loader_shards_and_resumes(tmp_path):
    src = RandomInstanceSource(num_instances=64, sequence_length=8, vocab_size=100, work_dir=tmp_path, seed=3)
    whole = _loader(src, tmp_path)
    whole.reshuffle(1)
    batches = list(whole)
    assert len(batches) == 8 and all(b["input_ids"].shape == (8, 8) for b in batches)
    order = np.concatenate([b["index"].numpy() for b in batches])
    assert sorted(order.tolist()) == list(range(64)) and order.tolist() != list(range(64))
    # two ranks split every global batch between them
    parts = []
    for r in range(2):
        ld = _loader(src, tmp_path, rank=r, world=2)
        ld.reshuffle(1)
        parts.append(next(iter(ld))["index"].numpy())
    assert sorted(np.concatenate(parts).tolist()) == sorted(batches[0]["index"].tolist())
    # resume after three batches
    first = _loader(src, tmp_path)
    first.reshuffle(1)
    it = iter(first)
    for _ in range(3):
        next(it)
    state = first.state_dict()
    second = _loader(src, tmp_path)
    second.load_state_dict(state)
    second.reshuffle(state["epoch"])
    assert torch.equal(next(iter(second))["input_ids"], batches[3]["input_ids"])
    # a different source is refused
    other = RandomInstanceSource(num_instances=64, sequence_length=8, vocab_size=100, work_dir=tmp_path, seed=4)
    with pytest.raises(RuntimeError):
        _loader(other, tmp_path).load_state_dict(state)


def test_loader_intra_source_keeps_source_order(tmp_path):
    a = RandomInstanceSource(num_instances=16, sequence_length=8, vocab_size=100, work_dir=tmp_path, seed=1)
    b = RandomInstanceSource(num_instances=16, sequence_length=8, vocab_size=100, work_dir=tmp_path, seed=2)
    cfg = ComposableDataLoaderConfig(seed=1, num_threads=1, display_source_visualization=False,
                                     shuffle_strategy=ShuffleStrategy.intra_source)
    loader = cfg.build(a, b, work_dir=tmp_path, tokenizer=TokenizerConfig.gpt2(), global_batch_size=8 * 8)
    loader.reshuffle(1)
    order = np.concatenate([batch["index"].numpy() for batch in loader])
    assert (order[:16] < 16).all() and (order[16:] >= 16).all()


def test_numpy_document_source_long_documents_and_file_order(tmp_path):
    from olmo_core_b200.data.composable import LongDocStrategy, NumpyDocumentSourceConfigBase

    tok = TokenizerConfig.gpt2()
    eos = tok.eos_token_id
    data = np.concatenate([np.arange(1, 12), [eos], np.arange(20, 23), [eos], np.arange(30, 33)]).astype(np.uint16)
    for i in range(3):
        (data + i).astype(np.uint16).tofile(tmp_path / f"f-{i}.npy")
    pattern = [str(tmp_path / "f-*.npy")]
    assert issubclass(NumpyDocumentSource.Config, NumpyDocumentSourceConfigBase)

    # a 12-token document with a limit of 5: cut to its first 5 tokens, or into parts of 5, 5 and 2; the unterminated
    # tail of a file always counts as a document
    (trunc,) = NumpyDocumentSource.Config(source_paths=pattern, tokenizer=tok, source_group_size=-1, max_document_length=5,
                                          long_doc_strategy=LongDocStrategy.truncate).build(tmp_path / "w1")
    assert list(trunc.get_document_offsets())[:3] == [(0, 5), (12, 16), (16, 19)]
    (frag,) = NumpyDocumentSource.Config(source_paths=pattern, tokenizer=tok, source_group_size=-1, max_document_length=5,
                                         long_doc_strategy=LongDocStrategy.fragment).build(tmp_path / "w2")
    assert list(frag.get_document_offsets())[:5] == [(0, 5), (5, 10), (10, 12), (12, 16), (16, 19)]
    assert trunc.fingerprint != frag.fingerprint

    # the permutation seed reorders the files before they are grouped; the same seed gives the same order
    plain = NumpyDocumentSource.Config(source_paths=pattern, tokenizer=tok).build(tmp_path / "w3")
    assert [s.source_paths[0][-7:] for s in plain] == ["f-0.npy", "f-1.npy", "f-2.npy"]
    a = NumpyDocumentSource.Config(source_paths=pattern, tokenizer=tok, source_permutation_seed=3).build(tmp_path / "w4")
    b = NumpyDocumentSource.Config(source_paths=pattern, tokenizer=tok, source_permutation_seed=3).build(tmp_path / "w5")
    assert [s.source_paths for s in a] == [s.source_paths for s in b]
    assert sorted(s.source_paths[0] for s in a) == sorted(s.source_paths[0] for s in plain)
    with pytest.raises(Exception):
        NumpyDocumentSource.Config(source_paths=pattern, tokenizer=tok, source_group_size=0)


def test_sampling_keeps_max_sequence_length_units_together(tmp_path):
    a = InMemoryTokenSource(list(range(400)), work_dir=tmp_path)
    wide = ConcatAndChunkInstanceSource(a, sequence_length=5, max_sequence_length=20, work_dir=tmp_path)
    sample = wide.sample(max_instances=30, seed=2)
    assert len(sample) == 28 and sample.source_sample_sizes == (28,)
    firsts = [int(np.asarray(sample[i]["input_ids"])[0]) for i in range(len(sample))]
    for k in range(0, 28, 4):  # four neighbouring 5-token instances = one 20-token unit
        assert firsts[k] % 20 == 0 and firsts[k:k + 4] == [firsts[k] + 5 * j for j in range(4)]
    front, back = wide.split(0.25, seed=3)
    assert len(front) == 20 and len(back) == 60 and front.seed == 3
    seen = {int(np.asarray(s[i]["input_ids"])[0]) for s in (front, back) for i in range(len(s))}
    assert len(seen) == 80  # disjoint and complete
