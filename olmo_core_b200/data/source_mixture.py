"""
Source mixtures: build a training set of a requested size from several sources with target token ratios, optional
up-sampling (``max_repetition_ratio``) and a cap on the share of a source that may be used (``max_source_fraction``)
(allocation rules of src/olmo_core/data/source_mixture.py).

The outcome is, per file, the number of tokens to take from its beginning -- consumed by
:class:`~olmo_core_b200.data.numpy_dataset.NumpyFSLDatasetMixture`.
"""

from __future__ import annotations

import logging
import math
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass
from itertools import chain
from typing import Any, Dict, List, Optional, Tuple

import numpy as np

from ..aliases import PathOrStr
from ..config import Config
from ..exceptions import OLMoConfigurationError
from ..io import file_exists, get_file_size, glob_directory
from .types import NumpyUIntTypes

log = logging.getLogger(__name__)

__all__ = ["SourceMixtureConfig", "SourceMixtureList", "SourceMixtureDataset", "SourceMixtureDatasetConfig",
           "SourceMixtureOutcome", "SourcePathTokens", "SourceTokenDetails"]


@dataclass
class SourceMixtureConfig(Config):
    source_name: str
    target_ratio: float
    """Share of the mixture's tokens that should come from this source."""
    paths: List[str]
    max_repetition_ratio: float = 1.0
    """How many times the source may be repeated (>= 1) to reach its share."""
    max_source_fraction: float = 1.0
    """Upper bound on the fraction of the source that may be used per repetition."""
    _resolved_paths: Optional[List[str]] = None

    def validate(self) -> None:
        if self.target_ratio and not 0 < self.target_ratio <= 1:
            raise OLMoConfigurationError("target_ratio must be > 0 and <= 1")
        if not 0 <= self.max_source_fraction <= 1 or (self.target_ratio and self.max_source_fraction == 0):
            raise OLMoConfigurationError("max_source_fraction must be in the range (0, 1]")
        if self.max_repetition_ratio < 1:
            raise OLMoConfigurationError("max_repetition_ratio must be >= 1")
        if not self.paths:
            raise OLMoConfigurationError("paths must not be empty")

    @property
    def resolved_paths(self) -> List[str]:
        """The paths with globs expanded (sorted) and existence checked; computed once."""
        if self._resolved_paths is None:
            out: List[str] = []
            for p in map(str, self.paths):
                if "*" in p:
                    matches = sorted(glob_directory(p))
                    if not matches:
                        raise FileNotFoundError(f"Glob pattern '{p}' did not match any files")
                    out.extend(matches)
                elif not file_exists(p):
                    raise FileNotFoundError(f"Path '{p}' does not exist")
                else:
                    out.append(p)
            self._resolved_paths = out
        return self._resolved_paths


@dataclass
class SourceMixtureList(Config):
    """The sources of a mixture; their target ratios must sum to one."""

    sources: List[SourceMixtureConfig]

    def validate(self) -> None:
        if not self.sources:
            raise OLMoConfigurationError("sources must not be empty")
        total = float(np.sum([s.target_ratio for s in self.sources]))
        if not np.allclose(total, 1.0):
            raise OLMoConfigurationError(f"target_ratios must sum to 1.0, got {total}")


@dataclass
class SourceTokenDetails:
    config: SourceMixtureConfig
    population: int
    num_selected: int

    def for_table(self, requested_tokens: int) -> Dict[str, str]:
        return {
            "source_name": self.config.source_name,
            "source_population": str(self.population),
            "num_selected": str(self.num_selected),
            "target_ratio": str(self.config.target_ratio),
            "max_repetion_ratio": str(self.config.max_repetition_ratio),
            "max_source_fraction": str(self.config.max_source_fraction),
            "observed_source_ratio": f"{self.num_selected / self.population:.4}",
            "observed_global_ratio": f"{self.num_selected / requested_tokens:.4}",
        }


@dataclass
class SourcePathTokens:
    path: str
    tokens: int
    max_tokens: int


@dataclass
class SourceMixtureOutcome:
    name: str
    path_tokens: List[SourcePathTokens]


@dataclass
class SourceMixtureDataset:
    """Result of :meth:`SourceMixtureDatasetConfig.build`: per source, per file, how many tokens to use."""

    sources: List[SourceMixtureOutcome]

    def _flat(self) -> List[SourcePathTokens]:
        return list(chain.from_iterable(s.path_tokens for s in self.sources))

    def to_index(self) -> Dict[Tuple[str, int], int]:
        """``{(path, position in to_paths()): tokens}`` -- a path can occur more than once when a source is repeated."""
        return {(str(item.path), i): item.tokens for i, item in enumerate(self._flat())}

    def to_paths(self) -> List[PathOrStr]:
        return [item.path for item in self._flat()]


@dataclass
class SourceMixtureDatasetConfig(Config):
    source_list: SourceMixtureList
    requested_tokens: int
    """Desired size in tokens; the result is rounded up to whole batches of whole instances."""
    global_batch_size: int
    processes: int = 1
    seed: int = 42
    render_tables: bool = True
    quiet: bool = False

    def validate(self) -> None:
        if self.requested_tokens <= 0:
            raise OLMoConfigurationError("requested_tokens must be > 0")
        self.source_list.validate()

    # -- counting ---------------------------------------------------------------------------------------
    @staticmethod
    def _bytes_to_tokens(num_bytes: int, npdtype: NumpyUIntTypes) -> int:
        return num_bytes // npdtype(0).itemsize

    def _count_tokens_for_file(self, path: PathOrStr, npdtype: NumpyUIntTypes) -> int:
        return self._bytes_to_tokens(get_file_size(path), npdtype)

    def _count_tokens_for_paths(self, paths: List[PathOrStr], source: Optional[str], npdtype: NumpyUIntTypes) -> int:
        del source
        with ThreadPoolExecutor(max_workers=max(self.processes, 1)) as pool:
            return sum(pool.map(lambda p: self._count_tokens_for_file(p, npdtype), paths))

    # -- allocation -------------------------------------------------------------------------------------
    def get_paths_and_tokens_for_source(self, source_config: SourceMixtureConfig, token_details: SourceTokenDetails,
                                        npdtype: NumpyUIntTypes) -> List[SourcePathTokens]:
        """
        Spread the source's share evenly over its files: each file contributes the same fraction of its tokens. A
        fraction above one means repetition: whole passes over all files, then one partial pass.
        """
        take = token_details.num_selected / token_details.population
        counts = {p: self._count_tokens_for_file(p, npdtype) for p in source_config.resolved_paths}
        passes: List[float] = []
        remaining = take
        while remaining > 0:
            passes.append(min(1.0, remaining))
            remaining -= passes[-1]
            if take <= 1:
                break
        return [SourcePathTokens(path=p, tokens=int(math.ceil(n * frac)), max_tokens=n)
                for frac in passes for p, n in counts.items()]

    def build(self, *, npdtype: NumpyUIntTypes, sequence_length: int) -> SourceMixtureDataset:
        self.validate()
        if self.global_batch_size % sequence_length != 0:
            raise OLMoConfigurationError("global_batch_size must be multiple of sequence_length")
        details: List[SourceTokenDetails] = []
        for src in self.source_list.sources:
            src.validate()
            population = self._count_tokens_for_paths(list(src.resolved_paths), src.source_name, npdtype)
            needed = int(self.requested_tokens * src.target_ratio)
            ceiling = int(population * src.max_source_fraction * src.max_repetition_ratio)
            if ceiling < needed:
                raise OLMoConfigurationError(
                    f"Insufficient tokens for source: {src.source_name} @ target global ratio: {src.target_ratio} :: "
                    f"{ceiling} < {needed}"
                )
            details.append(SourceTokenDetails(config=src, population=population, num_selected=needed))

        per_source = {d.config.source_name: self.get_paths_and_tokens_for_source(d.config, d, npdtype) for d in details}
        files = [f for items in per_source.values() for f in items]

        # Whole instances only. Start from floor(tokens / L) per file, then hand out the instances still missing to
        # reach the requested number of batches: first evenly, then by largest fractional remainder.
        L = sequence_length
        wanted = math.ceil(self.requested_tokens / self.global_batch_size) * (self.global_batch_size // L)
        cap = [f.max_tokens // L for f in files]
        have = [min(f.tokens // L, c) for f, c in zip(files, cap)]
        frac = [(f.tokens % L) / L if h < c else 0.0 for f, h, c in zip(files, have, cap)]
        missing = wanted - sum(have)
        room = [i for i in range(len(files)) if have[i] < cap[i]]
        if missing > 0 and room:
            share = missing // len(room)
            if share:
                for i in room:
                    have[i] += min(share, cap[i] - have[i])
            missing = wanted - sum(have)
            if missing > 0:
                ranked = sorted(((frac[i], i) for i in room if have[i] < cap[i]), reverse=True)
                for _, i in ranked[:missing]:
                    have[i] += 1
        for f, h in zip(files, have):
            f.tokens = h * L

        outcome = [SourceMixtureOutcome(name=name, path_tokens=items) for name, items in per_source.items()]
        total = sum(f.tokens for f in files)
        if self.render_tables and not self.quiet:
            self.render_mixture_outcome_tables(details)
        diff = total - self.requested_tokens
        log.info(f"Total tokens in mixture: {total} (requested: {self.requested_tokens}, diff: {diff:+} tokens, "
                 f"{100 * diff / self.requested_tokens:+.2f}%)")
        for name, items in per_source.items():
            got = sum(f.tokens for f in items) / max(total, 1)
            target = next(s.target_ratio for s in self.source_list.sources if s.source_name == name)
            log.info(f"{name}: {abs(got - target):.4f} difference from target ratio {target:.4f}")
        return SourceMixtureDataset(sources=outcome)

    def table_to_text(self, table) -> Any:
        """Plain-text form of a ``rich`` table, 250 columns wide, for log files
        (src/olmo_core/data/source_mixture.py:582-591)."""
        from rich.console import Console
        from rich.text import Text

        console = Console(width=250)
        with console.capture() as capture:
            table.width = 250
            console.print(table)
        return Text.from_ansi(capture.get())

    def render_mixture_outcome_tables(self, results: List[SourceTokenDetails]) -> None:
        rows = [r.for_table(self.requested_tokens) for r in results]
        headers = list(rows[0].keys())
        widths = [max(len(h), *(len(r[h]) for r in rows)) for h in headers]
        line = " | ".join(h.ljust(w) for h, w in zip(headers, widths))
        body = "\n".join(" | ".join(r[h].ljust(w) for h, w in zip(headers, widths)) for r in rows)
        population, selected = sum(r.population for r in results), sum(r.num_selected for r in results)
        log.info(f"Outcome by source\n{line}\n{'-' * len(line)}\n{body}")
        log.info(f"Global outcome: total_tokens={population:.2e} selected_tokens={selected:.2e} "
                 f"observed_global_ratio={selected / population:.4}")
