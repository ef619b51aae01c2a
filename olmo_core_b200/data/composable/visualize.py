"""Print a source tree (role of src/olmo_core/data/composable/visualize.py:1-92)."""

from __future__ import annotations

from typing import List

from .source_abc import SourceABC
from .utils import format_token_count

__all__ = ["visualize_source", "render_source"]


def _describe(node: SourceABC, icons: bool, count: int = 1) -> str:
    icon = f"{node.DISPLAY_ICON} " if icons and node.DISPLAY_ICON else ""
    name = f"{type(node).__name__}({node.fingerprint[:7]})" if count == 1 else f"{type(node).__name__} x {count}"
    label = f" [{node.label}]" if node.label else ""
    return f"{icon}{name}: {format_token_count(node.num_tokens)} tokens{label}"


def render_source(source: SourceABC, icons: bool = False) -> str:
    """The tree as text; runs of sibling leaves of one class and label are folded into ``Class x N``."""
    lines: List[str] = [_describe(source, icons)]

    def walk(node: SourceABC, prefix: str) -> None:
        groups: List[List[SourceABC]] = []
        for child in node.children():
            last = groups[-1][0] if groups else None
            if last is not None and child.is_leaf and last.is_leaf and type(child) is type(last) and child.label == last.label:
                groups[-1].append(child)
            else:
                groups.append([child])
        for i, group in enumerate(groups):
            tip, bar = ("└─ ", "   ") if i == len(groups) - 1 else ("├─ ", "│  ")
            if len(group) == 1:
                lines.append(prefix + tip + _describe(group[0], icons))
                walk(group[0], prefix + bar)
            else:
                total = sum(g.num_tokens for g in group)
                label = f" [{group[0].label}]" if group[0].label else ""
                lines.append(f"{prefix}{tip}{type(group[0]).__name__} x {len(group)}: {format_token_count(total)} tokens{label}")

    walk(source, "")
    return "\n".join(lines)


def visualize_source(source: SourceABC, icons: bool = False) -> None:
    print(render_source(source, icons=icons))
