"""
Batch and token-array helpers for the data layer (function names of src/olmo_core/data/utils.py:43-974).
"""

from __future__ import annotations

import gzip
import math
import os
from contextlib import contextmanager
from pathlib import Path
from typing import Any, Dict, Generator, Iterable, List, NamedTuple, Optional, Sequence, Tuple, TypeVar, Union

import numpy as np
import torch
import torch.nn.functional as F

from ..aliases import PathOrStr
from ..io import get_bytes_range, get_file_size, is_url, resource_path

T = TypeVar("T")

__all__ = [
    "split_batch",
    "melt_batch",
    "truncate_batch",
    "get_labels",
    "get_document_lengths",
    "get_cumulative_document_lengths",
    "iter_document_indices",
    "get_document_indices",
    "write_document_indices",
    "load_array_slice",
    "load_array_slice_into_tensor",
    "iter_batched",
    "memmap_to_write",
    "write_array_to_disk",
    "divide_into_buckets",
    "chunk_array",
    "get_rng",
    "bucket_documents",
    "segment_documents_into_instances",
    "get_doc_lengths_from_indices",
    "find_periodic_sequences",
    "RepetitionTuple",
    "chunked",
    "InstancePacker",
    "pack_documents_into_instances",
    "attention_mask_to_cache_leftpad",
    "iter_document_indices_with_max_sequence_length",
    "run_worker_func",
    "find_end_first_consecutive_true",
    "find_start_last_consecutive_true",
    "group_consecutive_values",
    "SegmentTreeNode",
    "SegmentTree",
]


# ----------------------------------------------------------------------------------------------
# batches
# ----------------------------------------------------------------------------------------------


def _per_instance_slices(batch_size: int, n: int) -> List[slice]:
    return [slice(i, min(i + n, batch_size)) for i in range(0, batch_size, n)]


def split_batch(batch: Dict[str, Any], num_microbatch_instances: int) -> List[Dict[str, Any]]:
    """Split a collated batch into micro-batches of at most ``num_microbatch_instances`` instances."""
    if num_microbatch_instances <= 0:
        raise RuntimeError("microbatch size is too small!")
    batch_size = batch["input_ids"].shape[0]
    if batch_size <= num_microbatch_instances:
        return [batch]
    out: List[Dict[str, Any]] = []
    for sl in _per_instance_slices(batch_size, num_microbatch_instances):
        mb: Dict[str, Any] = {}
        for key, value in batch.items():
            if isinstance(value, (torch.Tensor, list)):
                mb[key] = value[sl]
            else:
                raise RuntimeError(f"unexpected item in batch: '{key}={value}'")
        out.append(mb)
    return out


def _reshape_batch(batch: Dict[str, Any], target: int, melt: bool) -> Dict[str, Any]:
    bsz, cur = batch["input_ids"].shape
    if cur <= target:
        return batch
    if melt and cur % target != 0:
        raise RuntimeError("current sequence of batch must be a multiple of the target sequence length in order to 'melt' the batch")
    ratio = cur // target
    new: Dict[str, Any] = {}
    for key, value in batch.items():
        if isinstance(value, torch.Tensor):
            if value.shape == (bsz, cur):
                new[key] = value.reshape(-1, target) if melt else value[:, :target]
            elif value.shape in ((bsz,), (bsz, 1)):
                new[key] = value.repeat_interleave(ratio) if melt else value
            else:
                raise RuntimeError(f"unable to reshape '{key}' tensor in batch with shape '{value.shape}'")
        elif isinstance(value, list) and value:
            items: List[Any] = []
            for item in value:
                if isinstance(item, list):
                    if len(item) != cur:
                        raise RuntimeError(f"unexpected item length for '{key}' in batch")
                    if melt:
                        items.extend(item[i * target : (i + 1) * target] for i in range(ratio))
                    else:
                        items.append(item[:target])
                else:
                    items.extend([item] * (ratio if melt else 1))
            new[key] = items
        else:
            raise RuntimeError(f"unexpected item in batch: '{key}={value}'")
    return new


def melt_batch(batch: Dict[str, Any], target_sequence_length: int) -> Dict[str, Any]:
    """Shorten sequences to ``target_sequence_length`` and proportionally increase the number of instances."""
    return _reshape_batch(batch, target_sequence_length, melt=True)


def truncate_batch(batch: Dict[str, Any], target_sequence_length: int) -> Dict[str, Any]:
    """Cut every instance to ``target_sequence_length`` tokens."""
    return _reshape_batch(batch, target_sequence_length, melt=False)


def get_labels(batch: Dict[str, Any], label_ignore_index: int = -100) -> torch.Tensor:
    """Next-token labels: input ids shifted left, with masked / padded positions set to the ignore index."""
    labels = batch["input_ids"].clone()
    if (label_mask := batch.get("label_mask")) is not None:
        labels.masked_fill_(~label_mask, label_ignore_index)
    if (attention_mask := batch.get("attention_mask")) is not None:
        labels.masked_fill_(attention_mask == 0.0, label_ignore_index)
    if (instance_mask := batch.get("instance_mask")) is not None:
        labels.masked_fill_(~instance_mask.unsqueeze(-1), label_ignore_index)
    return F.pad(labels[..., 1:], (0, 1, 0, 0), value=label_ignore_index)


def attention_mask_to_cache_leftpad(attention_mask: torch.Tensor) -> torch.Tensor:
    """Number of left-padding positions per row of a ``[B, T]`` left-padded attention mask (int32)."""
    if attention_mask.ndim != 2:
        raise ValueError(f"expected 2-D attention_mask (batch, seq_len), got shape {attention_mask.shape}")
    valid = attention_mask if attention_mask.dtype == torch.bool else attention_mask != 0
    seen = valid.cummax(dim=1).values
    if bool((seen & ~valid).any()):
        raise ValueError("attention_mask must represent *prefix padding* (all padding tokens precede valid tokens)")
    return valid.int().argmax(dim=-1).int()


# ----------------------------------------------------------------------------------------------
# documents
# ----------------------------------------------------------------------------------------------


def get_document_lengths(input_ids: Union[torch.Tensor, np.ndarray], eos_token_id: int,
                         bos_token_id: Optional[int] = None) -> torch.Tensor:
    """Lengths of the documents inside a 1-D token sequence (documents end with EOS, the tail counts as one)."""
    if not isinstance(input_ids, torch.Tensor):
        input_ids = torch.tensor(input_ids.astype(np.int_), dtype=torch.long)
    n = input_ids.shape[0]
    if bos_token_id is None:
        ends = (input_ids == eos_token_id).nonzero(as_tuple=True)[0].to(torch.int32)
        tail = [] if n > 0 and input_ids[-1] == eos_token_id else [n - 1]
    else:
        ends = torch.logical_and(input_ids[:-1] == eos_token_id, input_ids[1:] == bos_token_id).nonzero(as_tuple=True)[0].to(torch.int32)
        tail = [n - 1]
    bounds = torch.cat([torch.tensor([-1], dtype=torch.int32), ends, torch.tensor(tail, dtype=torch.int32)])
    return bounds[1:] - bounds[:-1]


def get_cumulative_document_lengths(doc_lens: torch.Tensor) -> torch.Tensor:
    """``[0, l0, l0+l1, ...]`` (int32) over the non-zero entries of a (possibly padded, batched) length tensor."""
    nz = doc_lens.masked_select(doc_lens != 0)
    return torch.cat([torch.zeros(1, dtype=torch.int32, device=doc_lens.device), torch.cumsum(nz, 0, dtype=torch.int32)])


def _array_itemsize(dtype) -> int:
    return np.dtype(dtype).itemsize


def load_array_slice(path: PathOrStr, start_idx: int, end_idx: int, dtype) -> np.ndarray:
    """Items ``[start_idx, end_idx)`` of a flat binary array stored at a local path or URL."""
    item = _array_itemsize(dtype)
    if is_url(path):
        raw = get_bytes_range(path, start_idx * item, (end_idx - start_idx) * item)
        return np.frombuffer(raw, dtype=dtype)
    with open(path, "rb") as f:
        f.seek(start_idx * item)
        return np.frombuffer(f.read((end_idx - start_idx) * item), dtype=dtype)


def load_array_slice_into_tensor(path: PathOrStr, start_idx: int, end_idx: int, dtype) -> torch.Tensor:
    arr = load_array_slice(path, start_idx, end_idx, dtype)
    if arr.dtype in (np.uint8, np.uint16, np.uint32, np.uint64):
        arr = arr.astype(np.int64)
    return torch.from_numpy(np.ascontiguousarray(arr)).long() if arr.dtype != np.bool_ else torch.from_numpy(arr.copy())


def iter_document_indices(data_path: PathOrStr, local_cache: Optional[PathOrStr] = None,
                          use_array_if_local: Optional[bool] = None, eos_token_id: Optional[int] = None,
                          bos_token_id: Optional[int] = None, dtype=None) -> Generator[Tuple[int, int], None, None]:
    """
    ``(start, end)`` token offsets of every document in a token file (src/olmo_core/data/utils.py:170-250).

    A local file is scanned for end-of-sequence tokens when ``eos_token_id`` and ``dtype`` are given (with
    ``bos_token_id``, a document ends only where an EOS is followed by a BOS, or at an EOS that ends the file); otherwise
    the ``.csv.gz`` metadata file next to the data lists the documents. Tokens after the last end-of-sequence token belong
    to no document.
    """
    if use_array_if_local is None:
        use_array_if_local = eos_token_id is not None and dtype is not None and not is_url(data_path)
    if use_array_if_local and not is_url(data_path):
        if eos_token_id is None or dtype is None:
            raise ValueError("'eos_token_id' and 'dtype' are required to use the local array for finding document indices")
        n = get_file_size(data_path) // _array_itemsize(dtype)
        arr = load_array_slice(data_path, 0, n, dtype)
        if bos_token_id is None:
            ends = np.nonzero(arr == eos_token_id)[0] + 1
        else:
            ends = np.nonzero(np.logical_and(arr[:-1] == eos_token_id, arr[1:] == bos_token_id))[0] + 1
            if n > 0 and arr[-1] == eos_token_id:
                ends = np.append(ends, n)
        start = 0
        for end in ends.tolist():
            yield start, end
            start = end
        return
    meta = str(data_path).replace(".npy", ".csv.gz")
    try:
        meta_path = resource_path(os.path.dirname(meta), os.path.basename(meta), local_cache=local_cache)
    except FileNotFoundError as e:
        raise RuntimeError(
            f"Source metadata file '{os.path.basename(meta)}' is required to calculate document indices for '{data_path}'. "
            "If the source data file is local (on-disk) and 'eos_token_id' and 'dtype' are provided, then the document "
            "indices can be inferred from the source file."
        ) from e
    with gzip.open(meta_path, "rt") as f:
        for line in f:
            start, end, *_ = line.split(",")
            yield int(start), int(end)


def get_document_indices(data_path: PathOrStr, local_cache: Optional[PathOrStr] = None, **kwargs) -> List[Tuple[int, int]]:
    return list(iter_document_indices(data_path, local_cache=local_cache, **kwargs))


def write_document_indices(data_path: Path, *, dtype, eos_token_id: int) -> Path:
    """Scan a token file for EOS tokens and write ``<name>.csv.gz`` with one ``start,end`` row per document."""
    out = Path(str(data_path).replace(".npy", ".csv.gz"))
    with gzip.open(out, "wt") as f:
        for start, end in iter_document_indices(data_path, eos_token_id=eos_token_id, dtype=dtype, local_cache="/nonexistent"):
            f.write(f"{start},{end}\n")
    return out


def get_doc_lengths_from_indices(doc_indices: np.ndarray) -> np.ndarray:
    return doc_indices[1::2] - doc_indices[::2]


def iter_batched(iterable: Iterable[Dict[str, Any]], batch_num_tokens: int) -> Iterable[Tuple[Dict[str, Any], ...]]:
    """Group instances into tuples holding at most ``batch_num_tokens`` tokens each."""
    batch: List[Dict[str, Any]] = []
    tokens = 0
    for x in iterable:
        n = x["input_ids"].numel()
        if n > batch_num_tokens:
            raise RuntimeError(f"an instance has {n} tokens, more than the batch size of {batch_num_tokens}")
        if tokens + n > batch_num_tokens:
            yield tuple(batch)
            batch, tokens = [], 0
        batch.append(x)
        tokens += n
    if batch:
        yield tuple(batch)


@contextmanager
def memmap_to_write(path: Path, *, shape: Tuple[int, ...], dtype) -> Generator[np.ndarray, None, None]:
    """Write a ``.npy``-less raw memmap atomically: fill a temp file, then rename it into place."""
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_suffix(f".{os.getpid()}.tmp")
    mm = np.memmap(tmp, dtype=dtype, mode="w+", shape=shape)
    try:
        yield mm
    except BaseException:
        del mm
        tmp.unlink(missing_ok=True)
        raise
    mm.flush()
    del mm
    tmp.replace(path)


def write_array_to_disk(arr: np.ndarray, path: Path) -> None:
    with memmap_to_write(path, shape=arr.shape, dtype=arr.dtype) as mm:
        mm[:] = arr


def divide_into_buckets(n: int, b: int) -> List[int]:
    """Split ``n`` items into ``b`` buckets whose sizes differ by at most one."""
    q, r = divmod(n, b)
    return [q + 1] * r + [q] * (b - r)


def chunk_array(arr: np.ndarray, chunk_sizes: Sequence[int]) -> List[np.ndarray]:
    out, offset = [], 0
    for n in chunk_sizes:
        out.append(arr[offset : offset + n])
        offset += n
    return out


def get_rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed=seed))


def bucket_documents(path: PathOrStr, target: Path, *, buckets: Sequence[int], eos_token_id: int, dtype,
                     indices_dtype=np.uint32) -> Tuple[int, int]:
    """
    Cut documents into pieces whose lengths are powers of two from ``buckets`` (largest first) and write the
    ``(start, end)`` offsets of all pieces to ``target``. Returns (number of documents, number of pieces).
    """
    sizes = sorted(buckets, reverse=True)
    pieces: List[int] = []
    n_docs = 0
    for start, end in iter_document_indices(path, eos_token_id=eos_token_id, dtype=dtype):
        n_docs += 1
        pos = start
        while end - pos >= sizes[-1]:
            for s in sizes:
                if end - pos >= s:
                    pieces += [pos, pos + s]
                    pos += s
                    break
    arr = np.asarray(pieces, dtype=indices_dtype)
    write_array_to_disk(arr, target)
    return n_docs, len(pieces) // 2


def segment_documents_into_instances(path: PathOrStr, target: Path, *, max_sequence_length: int, eos_token_id: int, dtype,
                                     indices_dtype=np.uint32, bos_token_id: Optional[int] = None,
                                     sample: Optional[Tuple[int, int]] = None) -> Tuple[int, int]:
    """
    One instance per document, truncated to ``max_sequence_length``, written to ``target`` as flat
    ``start, end`` pairs. ``sample=(n, seed)`` draws ``n`` instances with replacement. Returns the number of
    documents and of instances written (src/olmo_core/data/utils.py:535-578).
    """
    idx: List[int] = []
    for start, end in iter_document_indices(path, eos_token_id=eos_token_id, bos_token_id=bos_token_id, dtype=dtype):
        idx += [start, start + min(end - start, max_sequence_length)]
    arr = np.asarray(idx, dtype=indices_dtype).reshape(-1, 2)
    n_docs = arr.shape[0]
    if sample is not None:
        n, seed = sample
        arr = get_rng(seed).choice(arr, size=n)
    if arr.size == 0:
        raise RuntimeError(f"Failed to produce any documents from '{path}'")
    write_array_to_disk(arr.reshape(-1), target)
    return n_docs, arr.shape[0]


# ----------------------------------------------------------------------------------------------
# repetition filter
# ----------------------------------------------------------------------------------------------


class RepetitionTuple(NamedTuple):
    start: int
    end: int
    period: int
    times: int


def find_periodic_sequences(arr: np.ndarray, max_period: int, min_period: int = 1,
                            mask_value: int = -1) -> Generator[RepetitionTuple, None, None]:
    """Yield maximal runs where ``arr[i] == arr[i + period]`` that repeat at least three times."""
    n = len(arr)
    for period in range(min_period, min(max_period, n // 3) + 1):
        same = np.concatenate([arr[:-period] == arr[period:], [False]])
        same &= np.concatenate([arr[:-period] != mask_value, [False]])
        edges = np.flatnonzero(np.diff(np.concatenate([[False], same, [False]]).astype(np.int8)))
        for start, stop in zip(edges[::2], edges[1::2]):
            length = (stop - start) + period
            times = length // period
            if times >= 3:
                yield RepetitionTuple(int(start), int(start + length), period, int(times))


def chunked(iterable: Iterable[T], n: int) -> Iterable[List[T]]:
    buf: List[T] = []
    for x in iterable:
        buf.append(x)
        if len(buf) == n:
            yield buf
            buf = []
    if buf:
        yield buf


# ----------------------------------------------------------------------------------------------
# packing
# ----------------------------------------------------------------------------------------------


class InstancePacker:
    """
    Best-fit-decreasing bin packing of documents into instances of ``max_sequence_length`` tokens. Free
    space per open instance is kept in a max segment tree so the tightest fitting instance is found in
    ``O(log n)``.
    """

    def __init__(self, max_sequence_length: int):
        self.max_sequence_length = max_sequence_length
        self.instances: List[List[int]] = []
        self._space: List[int] = []

    def reset(self) -> None:
        """Forget all instances."""
        self.instances = []
        self._space = []

    @property
    def instance_bins(self) -> List[List[int]]:
        return self.instances

    @property
    def total_tokens(self) -> int:
        """Tokens held by all instances (their capacity minus the free space left in them)."""
        return self.max_sequence_length * len(self.instances) - self.total_padding

    @property
    def total_padding(self) -> int:
        """Free tokens left over all instances (documents packed one by one with :meth:`pack_document`)."""
        return int(sum(self._space))

    def _best_fit(self, length: int) -> Optional[int]:
        best, best_space = None, None
        for i, s in enumerate(self._space):
            if s >= length and (best_space is None or s < best_space):
                best, best_space = i, s
        return best

    def _pack_document(self, document_id: int, document_length: int) -> int:
        return self.pack_document(document_id, document_length)

    def pack_document(self, document_id: int, document_length: int) -> int:
        if document_length > self.max_sequence_length:
            raise ValueError("document is longer than the maximum sequence length")
        i = self._best_fit(document_length)
        if i is None:
            self.instances.append([])
            self._space.append(self.max_sequence_length)
            i = len(self.instances) - 1
        self.instances[i].append(document_id)
        self._space[i] -= document_length
        return i

    def pack_documents(self, document_indices: np.ndarray) -> Tuple[List[List[int]], np.ndarray, int]:
        """
        ``document_indices``: ``[n, 2]`` (start, end). Returns ``(instances, sorted indices, total tokens)``: the documents
        are re-ordered longest first, the returned array holds them in that order and the instances refer to rows of
        it (``last_order`` keeps the permutation). Ties are resolved exactly as the reference does
        (src/olmo_core/data/utils.py:857-877: the same ``argsort`` call, and among instances with the same free space the
        one that reached it first), so a given file packs into the same instances in both implementations.
        """
        import bisect
        from collections import deque

        if self.instances:
            raise RuntimeError("call 'reset()' before packing another set of documents")
        lengths = document_indices[:, 1] - document_indices[:, 0]
        order = np.argsort(-1 * lengths.astype(np.int64))
        self.last_order = order
        document_indices = np.take(document_indices, order, axis=0)
        space_keys: List[int] = []  # distinct free sizes, ascending: best fit is a bisect
        by_space: Dict[int, Any] = {}
        total = 0
        for doc_id, n in enumerate((document_indices[:, 1] - document_indices[:, 0]).tolist()):
            n = int(n)
            if n > self.max_sequence_length:
                raise ValueError("document is longer than the maximum sequence length")
            total += n
            k = bisect.bisect_left(space_keys, n)
            if k < len(space_keys):
                space = space_keys[k]
                inst = by_space[space].popleft()
                if not by_space[space]:
                    del by_space[space]
                    space_keys.pop(k)
            else:
                self.instances.append([])
                inst = len(self.instances) - 1
                space = self.max_sequence_length
            self.instances[inst].append(doc_id)
            left = space - n
            if left > 0:
                if left not in by_space:
                    bisect.insort(space_keys, left)
                    by_space[left] = deque()
                by_space[left].append(inst)
        self._space = [0] * len(self.instances)
        for space, insts in by_space.items():
            for i in insts:
                self._space[i] = space
        return self.instances, document_indices, total


def pack_documents_into_instances(*paths: PathOrStr, max_sequence_length: int, eos_token_id: int, dtype,
                                  bos_token_id: Optional[int] = None, indices_dtype=np.uint64,
                                  long_doc_strategy="truncate") -> Tuple[List[List[int]], np.ndarray, int]:
    """
    Best-fit-decreasing packing of the documents of one or more token files (taken as one concatenated file) into
    instances of at most ``max_sequence_length`` tokens; longer documents are truncated or split. Returns the
    document ids of every instance, the ``(num_documents, 2)`` boundaries, and the number of tokens packed
    (src/olmo_core/data/utils.py:885-941).
    """
    if not paths:
        raise RuntimeError("At least one source path must be provided")
    docs: List[Tuple[int, int]] = []
    offset = 0
    for path in paths:
        for start, end in iter_document_indices_with_max_sequence_length(
                path, max_sequence_length, eos_token_id=eos_token_id, bos_token_id=bos_token_id, dtype=dtype,
                long_doc_strategy=long_doc_strategy):
            docs.append((offset + start, offset + end))
        offset += get_file_size(path) // _array_itemsize(dtype)
    arr = np.asarray(docs, dtype=indices_dtype).reshape(-1, 2)
    return InstancePacker(max_sequence_length).pack_documents(arr)


def iter_document_indices_with_max_sequence_length(
    data_path: PathOrStr, max_sequence_length: int, *, local_cache: Optional[PathOrStr] = None,
    use_array_if_local: Optional[bool] = None, eos_token_id: Optional[int] = None, bos_token_id: Optional[int] = None,
    dtype=None, long_doc_strategy="truncate",
) -> Generator[Tuple[int, int], None, None]:
    """
    :func:`iter_document_indices` with documents longer than ``max_sequence_length`` cut to their first part
    (``truncate``) or into consecutive parts (``fragment``) (src/olmo_core/data/utils.py:253-285).
    """
    from .types import LongDocStrategy

    strategy = LongDocStrategy(long_doc_strategy)
    kwargs = {} if use_array_if_local is None else {"use_array_if_local": use_array_if_local}
    for start, end in iter_document_indices(data_path, local_cache=local_cache, eos_token_id=eos_token_id,
                                            bos_token_id=bos_token_id, dtype=dtype, **kwargs):
        if end - start <= max_sequence_length:
            yield start, end
        elif strategy == LongDocStrategy.truncate:
            yield start, start + max_sequence_length
        elif strategy == LongDocStrategy.fragment:
            for s in range(start, end, max_sequence_length):
                yield s, min(end, s + max_sequence_length)
        else:
            raise NotImplementedError(strategy)


def run_worker_func(func, *args, **kwargs):
    """Entry point of data worker processes: runs ``func`` (remote-storage clients are created lazily per process here)."""
    return func(*args, **kwargs)


def find_end_first_consecutive_true(arr: np.ndarray) -> int:
    """End (exclusive) of the run of ``True`` that starts at position 0; 0 when the array starts with ``False``."""
    arr = np.asarray(arr, dtype=bool)
    if arr.size == 0 or not arr[0]:
        return 0
    false_at = np.flatnonzero(~arr)
    return int(false_at[0]) if false_at.size else int(arr.size)


def find_start_last_consecutive_true(arr: np.ndarray) -> int:
    """Start of the run of ``True`` that ends at the last position; -1 when the array ends with ``False``."""
    n = find_end_first_consecutive_true(np.asarray(arr)[::-1])
    return len(arr) - n if n > 0 else -1


def group_consecutive_values(arr: np.ndarray, stepsize: int = 1) -> List[np.ndarray]:
    """Split ``arr`` wherever the difference between neighbours is not ``stepsize``."""
    return np.split(arr, np.flatnonzero(np.diff(arr) != stepsize) + 1)


class SegmentTreeNode:
    """A node of :class:`SegmentTree`: ``weight`` is the largest weight among the leaves below it."""

    __slots__ = ("_tree", "_pos")

    def __init__(self, tree: "SegmentTree", pos: int):
        self._tree, self._pos = tree, pos

    @property
    def weight(self) -> int:
        return int(self._tree._w[self._pos])

    @property
    def is_root(self) -> bool:
        return self._pos == 1

    @property
    def is_leaf(self) -> bool:
        return self._pos >= self._tree.N

    @property
    def leaf_id(self) -> Optional[int]:
        return self._pos - self._tree.N if self.is_leaf else None

    @property
    def parent(self) -> Optional["SegmentTreeNode"]:
        return None if self.is_root else SegmentTreeNode(self._tree, self._pos >> 1)

    @property
    def children(self) -> Optional[Tuple["SegmentTreeNode", "SegmentTreeNode"]]:
        if self.is_leaf:
            return None
        return SegmentTreeNode(self._tree, 2 * self._pos), SegmentTreeNode(self._tree, 2 * self._pos + 1)

    def update(self, weight: Optional[int] = None) -> None:
        """Set a leaf's weight (or recompute an inner node) and refresh the maxima up to the root."""
        w, pos = self._tree._w, self._pos
        if weight is not None:
            assert self.is_leaf
            w[pos] = weight
            pos >>= 1
        while pos >= 1:
            w[pos] = max(w[2 * pos], w[2 * pos + 1])
            pos >>= 1


class SegmentTree:
    """
    Max segment tree over ``N`` leaves (``N`` a power of two), heap-ordered in one array. Used for best-fit packing
    (src/olmo_core/data/utils.py:745-803): leaf ``i`` carries weight ``i + 1`` while some open instance has exactly
    ``i + 1`` free tokens, and ``query(w)`` descends to the LEFTMOST leaf whose weight is at least ``w``, i.e. the
    tightest free space that still fits. The last leaf starts with weight ``N`` (a fresh instance always fits).
    """

    def __init__(self, N: int):
        assert N > 0 and N & (N - 1) == 0, "N should be a power of 2"
        self.N = N
        self._w = np.zeros(2 * N, dtype=np.int64)
        self.leaf_nodes = [SegmentTreeNode(self, N + i) for i in range(N)]
        self.root_node = SegmentTreeNode(self, 1)
        self.leaf_nodes[-1].update(N)

    def query(self, weight: int) -> SegmentTreeNode:
        pos = 1
        assert weight <= self._w[1]
        while pos < self.N:
            pos = 2 * pos if weight <= self._w[2 * pos] else 2 * pos + 1
        return SegmentTreeNode(self, pos)
