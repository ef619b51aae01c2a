"""Tokenizer descriptions: vocabulary size and special token ids (src/olmo_core/data/tokenizer.py)."""

from __future__ import annotations

import json
from dataclasses import dataclass
from typing import List, Optional, Protocol

from ..config import Config, StrEnum

__all__ = ["TokenizerConfig", "TokenizerLike", "TokenizerName"]


class TokenizerLike(Protocol):
    eos_token_id: int

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]: ...


class TokenizerName(StrEnum):
    dolma2 = "allenai/dolma2-tokenizer"
    dolma2_sigdig = "allenai/dolma2-tokenizer-sigdig"
    gpt_neox_olmo_dolma_v1_5 = "allenai/gpt-neox-olmo-dolma-v1_5"
    gpt2 = "gpt2"


# name -> (vocab size, eos, pad, bos)
_KNOWN = {
    TokenizerName.dolma2: (100278, 100257, 100277, None),
    TokenizerName.dolma2_sigdig: (100278, 100257, 100277, 100257),
    TokenizerName.gpt_neox_olmo_dolma_v1_5: (50280, 50279, 1, None),
    TokenizerName.gpt2: (50257, 50256, 50256, 50256),
}


@dataclass
class TokenizerConfig(Config):
    vocab_size: int
    eos_token_id: int
    pad_token_id: int
    bos_token_id: Optional[int] = None
    identifier: Optional[str] = None
    """A path or Hugging Face identifier from which the concrete tokenizer can be loaded."""

    def padded_vocab_size(self, pad_multiple: int = 128) -> int:
        """Vocabulary size rounded up to a multiple of ``pad_multiple`` (embedding / LM-head GEMMs tile evenly)."""
        return pad_multiple * ((self.vocab_size + pad_multiple - 1) // pad_multiple)

    @classmethod
    def _known(cls, name: TokenizerName) -> "TokenizerConfig":
        vocab, eos, pad, bos = _KNOWN[name]
        return cls(vocab_size=vocab, eos_token_id=eos, pad_token_id=pad, bos_token_id=bos, identifier=name)

    @classmethod
    def dolma2(cls) -> "TokenizerConfig":
        return cls._known(TokenizerName.dolma2)

    @classmethod
    def dolma2_sigdig(cls) -> "TokenizerConfig":
        return cls._known(TokenizerName.dolma2_sigdig)

    @classmethod
    def gpt_neox_olmo_dolma_v1_5(cls) -> "TokenizerConfig":
        return cls._known(TokenizerName.gpt_neox_olmo_dolma_v1_5)

    @classmethod
    def gpt2(cls) -> "TokenizerConfig":
        return cls._known(TokenizerName.gpt2)

    @classmethod
    def from_hf(cls, identifier: str) -> "TokenizerConfig":
        """Read vocabulary size and special ids from a Hugging Face model's ``config.json`` (or ``tokenizer_config.json``)."""
        from ..io import read_text

        try:
            cfg = json.loads(read_text(f"hf://{identifier}/config.json"))
        except FileNotFoundError:
            cfg = json.loads(read_text(f"hf://{identifier}/tokenizer_config.json"))
        return cls(vocab_size=cfg["vocab_size"], eos_token_id=cfg["eos_token_id"],
                   pad_token_id=cfg.get("pad_token_id", cfg["eos_token_id"]), bos_token_id=cfg.get("bos_token_id"),
                   identifier=identifier)
