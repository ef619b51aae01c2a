"""
Tokenise the "code fresh" evaluation corpus (one JSON row per source file, grouped by programming language) into the
flat ``uint32`` token files plus gzip'd ``start,end`` document tables that the numpy datasets read.
Function names and on-disk formats follow src/olmo_core/data/misc/code_fresh_export.py:14-174.

Every output file is written to a temporary name in the destination folder and renamed into place, so an interrupted
export never leaves a half-written file behind.
"""

from __future__ import annotations

import contextlib
import gzip
import json
import multiprocessing
import os
import tempfile
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Iterable, Iterator, List, Optional, Sequence, Tuple

import numpy as np

__all__ = [
    "CODE_FRESH_LANGUAGES",
    "ExportStats",
    "process_code_fresh_file_contents",
    "build_documents_and_stats",
    "flatten_documents",
    "write_memmap",
    "write_document_metadata",
    "write_stats",
    "get_export_dir_name",
    "default_num_procs",
]

CODE_FRESH_LANGUAGES: Tuple[str, ...] = tuple(
    """blade c clojure common_lisp cpp csharp css dart erlang fortran go haskell html java java_server_page javascript
    julia kotlin lua markdown mathematica matlab objective_c objective_cpp ocaml perl php powershell python
    restructuredtext ruby rust scala scheme swift systemverilog tcl tex typescript verilog vhdl vue""".split()
)


@dataclass
class ExportStats:
    language: str
    num_docs: int = 0
    total_tokens: int = 0
    max_doc_tokens_before_eos: int = 0
    max_doc_tokens_after_eos: int = 0
    num_skipped_empty: int = 0

    def add(self, doc: np.ndarray) -> None:
        self.num_docs += 1
        self.total_tokens += int(doc.size)
        self.max_doc_tokens_before_eos = max(self.max_doc_tokens_before_eos, int(doc.size) - 1)
        self.max_doc_tokens_after_eos = max(self.max_doc_tokens_after_eos, int(doc.size))


def process_code_fresh_file_contents(file_contents: str, tokenizer, *, max_doc_tokens_before_eos: int = 8191) -> Optional[np.ndarray]:
    """Token ids of one source file followed by EOS; ``None`` for files that are empty after stripping."""
    ids = tokenizer.encode(file_contents.strip(), add_special_tokens=False)
    if len(ids) == 0:
        return None
    if len(ids) > max_doc_tokens_before_eos:
        raise ValueError(f"a document has {len(ids)} tokens before EOS; the cap is {max_doc_tokens_before_eos}")
    out = np.empty(len(ids) + 1, dtype=np.uint32)
    out[:-1] = ids
    out[-1] = tokenizer.eos_token_id
    return out


def build_documents_and_stats(rows: Iterable[dict], tokenizer, *, language: str,
                              max_doc_tokens_before_eos: int = 8191) -> Tuple[List[np.ndarray], ExportStats]:
    stats = ExportStats(language=language)
    docs: List[np.ndarray] = []
    for row in rows:
        doc = process_code_fresh_file_contents(row["file_contents"], tokenizer,
                                               max_doc_tokens_before_eos=max_doc_tokens_before_eos)
        if doc is None:
            stats.num_skipped_empty += 1
        else:
            stats.add(doc)
            docs.append(doc)
    return docs, stats


def flatten_documents(docs: Sequence[np.ndarray]) -> Tuple[np.ndarray, List[Tuple[int, int]]]:
    """Concatenate the documents; also return their ``(start, end)`` token ranges."""
    ends = np.cumsum([len(d) for d in docs], dtype=np.int64)
    starts = np.concatenate([[0], ends[:-1]]) if len(docs) else ends
    tokens = np.concatenate(docs).astype(np.uint32, copy=False) if len(docs) else np.zeros(0, dtype=np.uint32)
    return tokens, [(int(s), int(e)) for s, e in zip(starts, ends)]


@contextlib.contextmanager
def _replace_when_done(path: Path) -> Iterator[Path]:
    path.parent.mkdir(parents=True, exist_ok=True)
    fd, tmp_name = tempfile.mkstemp(dir=path.parent, suffix=".tmp")
    os.close(fd)
    tmp = Path(tmp_name)
    try:
        yield tmp
        os.replace(tmp, path)
    finally:
        tmp.unlink(missing_ok=True)


def write_memmap(path: Path, arr: np.ndarray) -> None:
    with _replace_when_done(Path(path)) as tmp:
        if arr.size:
            out = np.memmap(tmp, mode="w+", dtype=arr.dtype, shape=arr.shape)
            out[:] = arr
            out.flush()
            del out


def write_document_metadata(path: Path, offsets: Sequence[Tuple[int, int]]) -> None:
    with _replace_when_done(Path(path)) as tmp:
        with gzip.open(tmp, "wt") as f:
            f.writelines(f"{start},{end}\n" for start, end in offsets)


def write_stats(path: Path, stats: ExportStats) -> None:
    with _replace_when_done(Path(path)) as tmp:
        tmp.write_text(json.dumps(asdict(stats), indent=2, sort_keys=True))


def get_export_dir_name(tokenizer_name: str) -> str:
    return "code_fresh_0825_1225_" + tokenizer_name.rsplit("/", 1)[-1]


def default_num_procs() -> int:
    return max(1, multiprocessing.cpu_count() - 1)
