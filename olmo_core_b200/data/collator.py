"""
Batch collation for text data (output fields of src/olmo_core/data/collator.py:24-178).

Instances are dicts with ``input_ids`` and optional ``attention_mask``, ``attention_bias``, ``label_mask``,
``index``, ``instance_mask``, ``doc_lens`` and ``metadata`` (or bare token tensors). Sequences are padded to the
longest one of the batch, on the left or right. The batch is written into ONE pre-sized tensor per field instead of
padding and stacking per instance, so that a fixed-length batch is a single copy -- the loader pins that tensor for
the asynchronous host-to-device transfer.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Union

import torch

from ..config import StrEnum

__all__ = ["DataCollator", "PaddingDirection"]


class PaddingDirection(StrEnum):
    left = "left"
    right = "right"


def _as_tensor(x: Any) -> torch.Tensor:
    return x if isinstance(x, torch.Tensor) else torch.as_tensor(x)


@dataclass
class DataCollator:
    pad_token_id: int
    pad_direction: PaddingDirection = PaddingDirection.right
    label_ignore_index: int = -100
    vocab_size: Optional[int] = None
    """When set, token ids outside ``[0, vocab_size)`` raise here, with positions, rather than as a device fault later."""

    def _place(self, out: torch.Tensor, row: int, value: torch.Tensor, max_len: int) -> None:
        n = value.shape[-1]
        if self.pad_direction == PaddingDirection.left:
            out[row, ..., max_len - n:] = value
        else:
            out[row, ..., :n] = value

    def __call__(self, items: Union[Sequence[Dict[str, Any]], Sequence[torch.Tensor]]) -> Dict[str, Any]:
        assert items, "cannot collate an empty batch"
        dicts: List[Dict[str, Any]] = [x if isinstance(x, dict) else {"input_ids": x} for x in items]
        ids = [_as_tensor(d["input_ids"]) for d in dicts]
        B, max_len = len(ids), max(len(t) for t in ids)

        input_ids = torch.full((B, max_len), self.pad_token_id, dtype=torch.long)
        for i, t in enumerate(ids):
            self._place(input_ids, i, t.to(torch.long), max_len)
        if self.vocab_size is not None:
            bad = (input_ids < 0) | (input_ids >= self.vocab_size)
            if bad.any():
                raise ValueError(
                    f"Token IDs {input_ids[bad].unique().tolist()} outside valid range [0, {self.vocab_size}). "
                    f"Found at (batch_idx, pos): {bad.nonzero(as_tuple=False).tolist()[:10]}"
                )
        out: Dict[str, Any] = {"input_ids": input_ids}

        def has(key: str) -> bool:
            return dicts[0].get(key) is not None

        if has("attention_mask"):
            mask = torch.zeros((B, max_len), dtype=torch.float)
            for i, d in enumerate(dicts):
                self._place(mask, i, _as_tensor(d["attention_mask"]).to(torch.float), max_len)
            out["attention_mask"] = mask
        if has("attention_bias"):
            first = _as_tensor(dicts[0]["attention_bias"])
            fill = False if first.dtype == torch.bool else float("-inf")
            rows = []
            for d in dicts:
                b = _as_tensor(d["attention_bias"])
                while b.dim() < 3:
                    b = b.unsqueeze(0)
                n = b.shape[-1]
                full = torch.full(b.shape[:-2] + (max_len, max_len), fill, dtype=b.dtype)
                if self.pad_direction == PaddingDirection.left:
                    full[..., max_len - n:, max_len - n:] = b
                else:
                    full[..., :n, :n] = b
                rows.append(full)
            out["attention_bias"] = torch.stack(rows)
        if has("label_mask"):
            lm = torch.zeros((B, max_len), dtype=torch.bool)
            for i, d in enumerate(dicts):
                self._place(lm, i, _as_tensor(d["label_mask"]).to(torch.bool), max_len)
            out["label_mask"] = lm
        if has("index"):
            out["index"] = torch.stack([torch.as_tensor(d["index"]) for d in dicts])
        if has("instance_mask"):
            out["instance_mask"] = torch.stack([torch.as_tensor(d["instance_mask"]) for d in dicts])
        if has("doc_lens"):
            lens = [_as_tensor(d["doc_lens"]) for d in dicts]
            width = max(len(x) for x in lens)
            doc_lens = torch.zeros((B, width), dtype=lens[0].dtype)
            for i, x in enumerate(lens):
                doc_lens[i, : len(x)] = x
            out["doc_lens"] = doc_lens
            out["max_doc_lens"] = [int(x.max()) for x in lens]
        if has("metadata"):
            out["metadata"] = [d["metadata"] for d in dicts]
        return out
