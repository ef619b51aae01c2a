"""
Named data mixes: a mix is a manifest of ``label,relative/path/{TOKENIZER}/file.npy`` lines that resolves, for a
storage root and a tokenizer, to a list of token files and their labels
(names and resolution rules of src/olmo_core/data/mixes/__init__.py).

The two perplexity-validation mixes are regular (one file per domain) and are generated here. The multi-thousand-line
manifests of the pre-training mixes are data, not code, and are looked up at run time: in this directory, in every
directory of the ``OLMO_CORE_DATA_MIX_PATH`` environment variable (``:``-separated), and in the ``data/mixes`` folder of
an installed ``olmo_core`` distribution.
"""

from __future__ import annotations

import os
from abc import abstractmethod
from pathlib import Path
from typing import Iterable, List, Optional, Tuple

from ...config import StrEnum
from ..tokenizer import TokenizerName

__all__ = ["DataMixBase", "DataMix", "DATA_MIX_PATH_ENV_VAR"]

DATA_MIX_PATH_ENV_VAR = "OLMO_CORE_DATA_MIX_PATH"

_V3_SMALL_DOMAINS = ("c4_en", "dolma_books", "dolma_common-crawl", "dolma_pes2o", "dolma_reddit", "dolma_stack",
                     "dolma_wiki", "ice", "m2d2_s2orc", "pile", "wikitext_103")
_CODE_FRESH_LANGUAGES = (
    "blade", "c", "clojure", "common_lisp", "cpp", "csharp", "css", "dart", "erlang", "fortran", "go", "haskell", "html",
    "java", "java_server_page", "javascript", "julia", "kotlin", "lua", "markdown", "mathematica", "matlab",
    "objective_c", "objective_cpp", "ocaml", "perl", "php", "powershell", "python", "restructuredtext", "ruby", "rust",
    "scala", "scheme", "swift", "systemverilog", "tcl", "tex", "typescript", "verilog", "vhdl", "vue",
)


class DataMixBase(StrEnum):
    """Base of data-mix enumerations; subclass and implement :meth:`build` for private mixes."""

    @abstractmethod
    def build(self, base_dir: str, tokenizer: str) -> Tuple[List[str], List[str]]:
        """``(paths, labels)`` of the mix stored under ``base_dir`` (e.g. ``s3://ai2-llm``) for ``tokenizer``."""
        raise NotImplementedError


def _generated_manifest(name: str) -> Optional[List[str]]:
    if name == "v3-small-ppl-validation":
        return [f"{d}-validation,eval-data/perplexity/v3_small_{{TOKENIZER}}/{d}/val/part-0-00000.npy" for d in _V3_SMALL_DOMAINS]
    if name == "code-fresh-ppl-validation":
        return [f"code_fresh_{l}-validation,eval-data/perplexity/code_fresh_0825_1225_{{TOKENIZER}}/{l}/val/part-0-00000.npy"
                for l in _CODE_FRESH_LANGUAGES]
    return None


def _manifest_dirs() -> Iterable[Path]:
    yield Path(__file__).parent
    for d in os.environ.get(DATA_MIX_PATH_ENV_VAR, "").split(":"):
        if d:
            yield Path(d)
    try:
        from importlib import metadata

        for f in metadata.files("ai2-olmo-core") or []:
            if f.parent.name == "mixes" and f.suffix == ".txt":
                yield Path(f.locate()).parent
                break
    except Exception:
        return


def _manifest_lines(name: str) -> List[str]:
    generated = _generated_manifest(name)
    if generated is not None:
        return generated
    fname = f"{os.path.basename(name)}.txt"
    for d in _manifest_dirs():
        if (d / fname).is_file():
            return (d / fname).read_text().splitlines()
    raise FileNotFoundError(
        f"No manifest '{fname}' for data mix '{name}'. Put the manifest into a directory listed in ${DATA_MIX_PATH_ENV_VAR}."
    )


_OFFICIAL_DOLMA3 = {
    "OLMo-mix-0625-official", "OLMo-mix-0925-official", "OLMo-midtraining-mix-0625-100B",
    "OLMo-midtraining-mix-0925-ingredient1-100B", "OLMo-midtraining-mix-0925-ingredient2-100B",
    "OLMo-longmino-mix-0625", "OLMo-longmino-mix-0925",
}
_ALIASES = {
    "dolma3-0625-6T-mix": "OLMo-mix-0625",
    "dolma3-0925-6T-mix": "OLMo-mix-0925",
    "dolma3-0925-150B-mix": "OLMo-mix-0625-150Bsample",
}


class DataMix(DataMixBase):
    OLMoE_mix_0824 = "OLMoE-mix-0824"
    dolma17 = "dolma17"
    OLMo_mix_0625 = "OLMo-mix-0625"
    OLMo_mix_0625_150Bsample = "OLMo-mix-0625-150Bsample"
    OLMo_mix_0625_700Bsample = "OLMo-mix-0625-700Bsample"
    OLMo_mix_0625_official = "OLMo-mix-0625-official"
    OLMo_mix_0925 = "OLMo-mix-0925"
    OLMo_mix_0925_official = "OLMo-mix-0925-official"
    OLMo_midtraining_mix_0625_100B = "OLMo-midtraining-mix-0625-100B"
    OLMo_midtraining_mix_0925_ingredient1_100B = "OLMo-midtraining-mix-0925-ingredient1-100B"
    OLMo_midtraining_mix_0925_ingredient2_100B = "OLMo-midtraining-mix-0925-ingredient2-100B"
    OLMo_longmino_mix_0625 = "OLMo-longmino-mix-0625"
    OLMo_longmino_mix_0925 = "OLMo-longmino-mix-0925"
    v3_small_ppl_validation = "v3-small-ppl-validation"
    code_fresh_ppl_validation = "code-fresh-ppl-validation"

    @classmethod
    def _missing_(cls, value: object):
        target = _ALIASES.get(value) if isinstance(value, str) else None
        return next((m for m in cls if m.value == target), None) if target else None

    def _tokenizer_dir(self, tokenizer: str) -> str:
        """The directory name under which the mix stores files of ``tokenizer``."""
        name = str(self.value)
        if name == "v3-small-ppl-validation":
            return {TokenizerName.gpt_neox_olmo_dolma_v1_5: "gptneox20b", TokenizerName.dolma2: "dolma2-tokenizer"}.get(tokenizer, tokenizer)
        if name == "code-fresh-ppl-validation":
            return "dolma2-tokenizer" if tokenizer == TokenizerName.dolma2 else tokenizer
        if name == "OLMo-mix-0625":
            return "dolma2-tokenizer-sigdig" if tokenizer == TokenizerName.dolma2_sigdig else tokenizer
        if name in _OFFICIAL_DOLMA3:
            return "allenai/dolma3-tokenizer" if tokenizer == TokenizerName.dolma2 else tokenizer
        if tokenizer == TokenizerName.gpt_neox_olmo_dolma_v1_5:
            return "gpt-neox-olmo-dolma-v1_5"
        return tokenizer

    def build(self, base_dir: str, tokenizer: str) -> Tuple[List[str], List[str]]:
        base = base_dir if base_dir.endswith("/") else base_dir + "/"
        tok_dir = self._tokenizer_dir(tokenizer)
        paths: List[str] = []
        labels: List[str] = []
        for n, line in enumerate(_manifest_lines(str(self.value)), start=1):
            line = line.strip()
            if not line or line.startswith("#"):
                continue
            label, rel = line.split(",")
            if "{TOKENIZER}" not in rel:
                raise ValueError(f"line {n} in data mix '{self}' is invalid")
            paths.append(base + rel.replace("{TOKENIZER}", tok_dir))
            labels.append(label)
        return paths, labels
