"""
Named groups of downstream evaluation tasks (task ids of the ``olmo_eval`` in-loop suite; same groups as
src/olmo_core/eval/task_groups.py). The lists are generated from the task families below rather than spelled out.
"""

from typing import Dict, List

_MMLU = ("stem", "humanities", "social_sciences", "other")
_MINERVA = ("algebra", "counting_and_probability", "geometry", "intermediate_algebra", "number_theory", "prealgebra",
            "precalculus")
_MT_MBPP_ALL = ("bash", "c", "cpp", "csharp", "go", "haskell", "java", "javascript", "matlab", "php", "python", "r",
                "ruby", "rust", "scala", "swift", "typescript")
_MT_MBPP_CORE = ("rust", "java", "cpp")
_BASIC_SKILLS = ("arithmetic", "coding", "common_knowledge", "logical_reasoning", "pattern", "string_operations")


def _mmlu(kind: str, splits=("val", "test")) -> List[str]:
    return [f"mmlu_{cat}_{split}_{kind}" for split in splits for cat in _MMLU]


def _gen_bpb(mt_mbpp) -> List[str]:
    return (["gsm8k_gold_bpb_5shot"] + [f"minerva_math_{s}_gold_bpb_0shot" for s in _MINERVA]
            + ["codex_humaneval_gold_bpb_3shot", "codex_mbpp_gold_bpb_3shot"])


_BASIC = [f"basic_skills_{s}_rc_5shot" for s in _BASIC_SKILLS]
_MCQA_SANITY = ["copycolors_10way_fast"]

# Runs too small for the model to pick up the multiple-choice format: rank-choice (RC) formulations.
FULL_TASKS_SMALL_COMPUTE: List[str] = (
    ["arc_challenge_test_rc_5shot", "arc_easy_test_rc_5shot", "hellaswag_rc_5shot", "winogrande_val_rc_5shot",
     "csqa_val_rc_5shot", "piqa_val_rc_5shot", "socialiqa_val_rc_5shot"]
    + _mmlu("rc_5shot")
    + _gen_bpb(_MT_MBPP_ALL)
    + ["coqa_bpb_0shot", "drop_bpb_5shot", "jeopardy_bpb_5shot", "lambada_bpb_0shot", "naturalqs_bpb_5shot",
       "squad_bpb_5shot"]
    + [f"mt_mbpp_{lang}_gold_bpb_3shot" for lang in _MT_MBPP_ALL]
    + _MCQA_SANITY + _BASIC
    + ["lab_bench_dbqa_rc_3shot", "lab_bench_protocolqa_rc_3shot", "medmcqa_rc_5shot", "medqa_en_rc_5shot",
       "qasper_yesno_rc_5shot", "sciriff_yesno_rc_5shot"]
)

# Runs large enough for multiple choice (MC) to work.
FULL_TASKS_LARGE_COMPUTE: List[str] = (
    ["arc_challenge_test_mc_5shot_fast", "arc_easy_test_mc_5shot_fast", "hellaswag_rc_5shot", "csqa_val_mc_5shot_fast",
     "piqa_val_mc_5shot_fast", "socialiqa_val_mc_5shot_fast", "winogrande_val_rc_5shot"]
    + _mmlu("mc_5shot_fast")
    + _gen_bpb(_MT_MBPP_CORE)
    + [f"mt_mbpp_{lang}_gold_bpb_3shot" for lang in _MT_MBPP_CORE]
    + _MCQA_SANITY + _BASIC
)

FULL_TASKS: List[str] = sorted(set(FULL_TASKS_SMALL_COMPUTE) | set(FULL_TASKS_LARGE_COMPUTE))

# Roughly 2-3x cheaper than the full set.
FAST_TASKS: List[str] = (
    ["arc_challenge_test_bpb_5shot", "arc_challenge_test_mc_5shot_fast", "arc_easy_test_bpb_5shot",
     "arc_easy_test_mc_5shot_fast", "hellaswag_bpb_5shot"]
    + [f"mmlu_{cat}_test_{kind}" for cat in ("humanities", "other", "social_sciences", "stem")
       for kind in ("bpb_5shot", "mc_5shot_fast")]
    + _BASIC
    + ["codex_humaneval_gold_bpb_3shot", "codex_mbpp_gold_bpb_3shot", "minerva_math_500_gold_bpb_0shot"]
    + [f"mt_mbpp_{lang}_gold_bpb_3shot" for lang in ("cpp", "java", "rust")]
    + _MCQA_SANITY
)

TASK_GROUPS: Dict[str, List[str]] = {
    "full__small_compute": FULL_TASKS_SMALL_COMPUTE,
    "full__large_compute": FULL_TASKS_LARGE_COMPUTE,
    "full": FULL_TASKS,
    "fast": FAST_TASKS,
}
