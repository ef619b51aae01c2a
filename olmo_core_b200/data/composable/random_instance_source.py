"""Reproducible random instances for benchmarks and tests
(src/olmo_core/data/composable/random_instance_source.py)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np

from ...aliases import PathOrStr
from ..tokenizer import TokenizerConfig
from ..utils import get_rng
from .instance_source import Instance, InstanceSource, InstanceSourceConfig
from .token_source import _default_seed
from .utils import SEED_NOT_SET, resolve_seed

__all__ = ["RandomInstanceSource", "RandomInstanceSourceConfig"]


class RandomInstanceSource(InstanceSource):
    """
    Random token ids with random document boundaries, reproducible per index: for benchmarks and tests
    (src/olmo_core/data/composable/random_instance_source.py:44-196). Special tokens never appear inside a document;
    every ``max_sequence_length`` window ends with EOS (and starts with BOS when the tokenizer has one) and holds about
    ``max_sequence_length / avg_document_length`` documents.
    """

    DISPLAY_ICON = ""

    def __init__(self, *, tokenizer=None, sequence_length: int, avg_document_length: Optional[int] = None,
                 seed: Optional[int] = SEED_NOT_SET, num_instances: Optional[int] = None, num_tokens: Optional[int] = None,
                 max_sequence_length: Optional[int] = None, label: Optional[str] = None, work_dir: PathOrStr,
                 vocab_size: Optional[int] = None):
        if (num_tokens is None) == (num_instances is None):
            raise ValueError("Either num_tokens or num_instances must be set, but not both.")
        if num_tokens is None:
            num_tokens = num_instances * sequence_length  # type: ignore[operator]
        super().__init__(work_dir=work_dir, sequence_length=sequence_length, max_sequence_length=max_sequence_length,
                         label=label)
        if tokenizer is None:
            if vocab_size is None:
                raise ValueError("a tokenizer config (or 'vocab_size') is required")
            tokenizer = TokenizerConfig(vocab_size=vocab_size, eos_token_id=0, pad_token_id=1)
        self._tokenizer = tokenizer
        self._num_tokens = self.max_sequence_length * (num_tokens // self.max_sequence_length)
        self._avg_document_length = avg_document_length or self.max_sequence_length
        seed = resolve_seed(seed)
        assert seed is not None
        self._seed = seed

    @property
    def num_tokens(self) -> int:
        return self._num_tokens

    @property
    def seed(self) -> int:
        return self._seed

    @property
    def eos_token_id(self) -> int:
        return self._tokenizer.eos_token_id

    @property
    def bos_token_id(self) -> Optional[int]:
        return self._tokenizer.bos_token_id

    @property
    def pad_token_id(self) -> int:
        return self._tokenizer.pad_token_id

    @property
    def vocab_size(self) -> int:
        return self._tokenizer.vocab_size

    @property
    def avg_document_length(self) -> int:
        return self._avg_document_length

    @property
    def non_special_token(self) -> int:
        special = (self.eos_token_id, self.bos_token_id, self.pad_token_id)
        for token_id in range(self.vocab_size):
            if token_id not in special:
                return token_id
        raise RuntimeError("No non-special token found in the vocabulary.")

    @property
    def dtype(self):
        for dtype in (np.uint8, np.uint16, np.uint32):
            if np.iinfo(dtype).max >= self.vocab_size:
                return dtype
        return np.uint64

    def children(self):
        return []

    @property
    def fingerprint(self) -> str:
        return self._hash(self._num_tokens, self._seed, self.max_sequence_length, self.eos_token_id, self.bos_token_id,
                          self.pad_token_id, self.vocab_size)

    def __len__(self) -> int:
        return self._num_tokens // self.sequence_length

    def __getitem__(self, idx: int) -> Instance:
        idx = self.validate_index(idx)
        per_window = self.max_sequence_length // self.sequence_length
        window = idx // per_window
        rng = get_rng(self._seed + window)
        L = self.max_sequence_length
        tokens = rng.integers(0, self.vocab_size, L, dtype=self.dtype)
        filler = self.non_special_token
        for special in (self.eos_token_id, self.pad_token_id, self.bos_token_id):
            if special is not None:
                tokens[tokens == special] = filler
        num_docs = max(1, round(rng.integers(-3, 3) + L / self._avg_document_length))
        tokens[-1] = self.eos_token_id
        if self.bos_token_id is not None:
            tokens[0] = self.bos_token_id
        if num_docs > 1:
            margin = 1 if self.bos_token_id is None else 2
            ends = margin + rng.permutation(L - 2 * margin - 1)[: num_docs - 1]
            tokens[ends] = self.eos_token_id
            if self.bos_token_id is not None:
                tokens[ends + 1] = self.bos_token_id
        if per_window > 1:
            start = (idx % per_window) * self.sequence_length
            tokens = tokens[start: start + self.sequence_length]
        return {"input_ids": tokens}


@dataclass
class RandomInstanceSourceConfig(InstanceSourceConfig):
    tokenizer: TokenizerConfig
    sequence_length: int
    avg_document_length: int
    seed: Optional[int] = field(default_factory=_default_seed)
    num_instances: Optional[int] = None
    num_tokens: Optional[int] = None
    max_sequence_length: Optional[int] = None
    label: Optional[str] = None

    def build(self, work_dir: PathOrStr) -> RandomInstanceSource:
        return RandomInstanceSource(tokenizer=self.tokenizer, sequence_length=self.sequence_length,
                                    avg_document_length=self.avg_document_length, seed=self.seed,
                                    num_instances=self.num_instances, num_tokens=self.num_tokens,
                                    max_sequence_length=self.max_sequence_length, label=self.label, work_dir=work_dir)


RandomInstanceSource.Config = RandomInstanceSourceConfig  # type: ignore[attr-defined]
