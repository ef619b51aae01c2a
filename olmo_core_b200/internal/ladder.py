"""
Command line for model-ladder experiments (role of src/olmo_core/internal/ladder.py:33-739)::

    python ladder.py {dry-run|benchmark|launch-benchmark|run|launch|launch-all|status|metrics|metrics-all} [options]

A script calls :func:`main` with either ``configure_ladder(args) -> ModelLadder`` or just
``configure_model(args) -> ModelConfigurator`` (the rest of the ladder then follows the defaults: dolma2 tokenizer,
concat-and-chunk over the default pre-training mix, WSD-S / Chinchilla run recipe). ``run`` / ``benchmark`` execute on the
ranks of the current job (start them with torchrun); the ``launch*`` commands submit them to Beaker; ``--cluster local``
plans for this machine's GPUs.
"""

from __future__ import annotations

import argparse
import logging
import sys
from typing import Callable, List, Optional, Type

from .. import io
from ..data import DataMix, TokenizerConfig
from ..data.composable import (
    ComposableDataLoaderConfig,
    ConcatAndChunkInstanceSourceConfig,
    InstanceFilterConfig,
    NumpyDocumentSourceMixConfig,
)
from ..launch.beaker import BeakerLaunchConfig, OLMoCoreBeakerImage
from ..model_ladder import ModelConfigurator, ModelLadder, RunConfigurator, TransformerSize, WSDSChinchillaRunConfigurator
from ..utils import prepare_cli_environment
from .common import build_launch_config, get_gpu_type, get_root_dir

log = logging.getLogger(__name__)

__all__ = ["main", "parse_args", "get_default_ladder_factory", "configure_launcher"]

LadderFactory = Callable[[argparse.Namespace], ModelLadder]
_LAUNCHING = ("launch-benchmark", "launch", "launch-all")
_ALL_SIZES = ("launch-all", "metrics-all")


def get_default_ladder_factory(configure_model: Callable[[argparse.Namespace], ModelConfigurator],
                               configure_run: Optional[Callable[[argparse.Namespace], RunConfigurator]] = None
                               ) -> LadderFactory:
    def factory(args: argparse.Namespace) -> ModelLadder:
        tokenizer = TokenizerConfig.dolma2()
        root = get_root_dir(args.cluster)
        run = configure_run(args) if configure_run is not None else WSDSChinchillaRunConfigurator(
            chinchilla_multiple=args.chinchilla_multiple, lr_multiplier=args.lr_multiplier,
            stepped_schedule=args.stepped_schedule)
        sources = [ConcatAndChunkInstanceSourceConfig(
            sources=[NumpyDocumentSourceMixConfig(tokenizer=tokenizer, mix=DataMix.OLMo_mix_0925, mix_base_dir=root)],
            sequence_length=args.sequence_length)]
        return ModelLadder(
            name=args.name, project=args.project, dir=str(io.join_path(root, f"model-ladders/{args.name}")),
            sizes=[str(s) for s in TransformerSize], max_devices=args.max_gpus, device_type=get_gpu_type(args.cluster),
            model_configurator=configure_model(args), run_configurator=run, sequence_length=args.sequence_length,
            tokenizer=tokenizer, instance_sources=sources,
            data_loader=ComposableDataLoaderConfig(num_workers=8, instance_filter_config=InstanceFilterConfig()))

    return factory


def configure_launcher(args: argparse.Namespace, ladder: ModelLadder, cmd: str, size: Optional[str] = None
                       ) -> BeakerLaunchConfig:
    """Launch config for running ``cmd`` (``run`` or ``benchmark``) of one size with exactly the GPUs it plans for."""
    command = [sys.argv[0], cmd, *sys.argv[2:]]
    if size is not None:
        command += ["--size", str(size)]
    size = size or args.size
    gpus = ladder.get_num_devices(size)
    if gpus >= 8 and gpus % 8 != 0:
        raise ValueError(f"{gpus} GPUs do not fill whole 8-GPU nodes")
    launcher = build_launch_config(cmd=command, name=f"{args.name}-{size}", num_nodes=max(gpus // 8, 1),
                                   cluster=args.cluster, workspace=args.workspace, beaker_image=args.beaker_image,
                                   budget=args.budget, nccl_debug="VERSION")
    if gpus < 8:
        launcher.num_gpus = gpus
    launcher.priority = args.priority
    if args.preemptible is not None:
        launcher.preemptible = args.preemptible
    launcher.allow_dirty = args.allow_dirty
    return launcher


# -- sub-commands --------------------------------------------------------------------------------------------------
def dry_run(args: argparse.Namespace) -> None:
    prepare_cli_environment()
    ladder = args.configure_ladder(args)
    if args.show_model:
        log.info("Model config:\n%s", ladder.get_model_config(args.size))
    ladder.dry_run(args.size, show_plot=args.show_plot,
                   save_plot=io.join_path(args.output_dir, f"{ladder.name}/lr_schedule_{args.size}.png")
                   if args.save_plot else None)


def benchmark(args: argparse.Namespace) -> None:
    args.configure_ladder(args).run_benchmark(args.size)


def run(args: argparse.Namespace) -> None:
    args.configure_ladder(args).run(args.size)


def _submit(args: argparse.Namespace, ladder: ModelLadder, cmd: str, size: Optional[str] = None) -> None:
    launcher = configure_launcher(args, ladder, cmd, size=size)
    if args.dry_run:
        launcher.dry_run()
    else:
        launcher.launch(follow=args.follow, slack_notifications=args.slack_notifications)


def launch_benchmark(args: argparse.Namespace) -> None:
    prepare_cli_environment()
    _submit(args, args.configure_ladder(args), "benchmark")


def launch(args: argparse.Namespace) -> None:
    prepare_cli_environment()
    _submit(args, args.configure_ladder(args), "run")


def launch_all(args: argparse.Namespace) -> None:
    prepare_cli_environment()
    ladder = args.configure_ladder(args)
    args.follow = False
    for size in _selected_sizes(args, ladder):
        _submit(args, ladder, "run", size=size)


def _selected_sizes(args: argparse.Namespace, ladder: ModelLadder) -> List[str]:
    if getattr(args, "size", None):
        return [args.size]
    sizes = [args.size_enum(s) for s in ladder.sizes]
    if getattr(args, "max_size", None):
        sizes = [s for s in sizes if s <= args.size_enum(args.max_size)]
    return [str(s) for s in sizes]


def _alternative_dirs(args: argparse.Namespace, ladder_name: str) -> Optional[List[str]]:
    roots = getattr(args, "alternative_root", None)
    return [str(io.join_path(r, f"model-ladders/{ladder_name}")) for r in roots] if roots else None


def status(args: argparse.Namespace) -> None:
    """Per size: which planned (or, with ``--discover-all``, existing) checkpoints and metrics files are there."""
    prepare_cli_environment()
    ladder = args.configure_ladder(args)
    alt = _alternative_dirs(args, ladder.name)
    rows = []
    for size in _selected_sizes(args, ladder):
        expected = ladder.get_checkpoints(size, discover_all=False, alternative_dirs=alt)
        found = ladder.get_checkpoints(size, discover_all=True, alternative_dirs=alt) if args.discover_all else expected
        have = sum(c.exists for c in found)
        metrics = sum(c.metrics_path is not None for c in found)
        print(f"\n{size}: {have} of {len(expected)} checkpoint(s)")
        for c in found:
            print("  " + c.display().replace("\n", "\n  "))
        mark = "ok" if have >= len(expected) else ("partial" if have else "missing")
        rows.append((size, have, len(expected), metrics, len(expected) - 1, mark))
    print("\nsize      checkpoints   metrics   status")
    for size, have, want, m_have, m_want, mark in rows:
        print(f"{size:<9} {have:>4} / {want:<6} {m_have:>3} / {m_want:<5} {mark}")


def _write_metrics(args: argparse.Namespace, ladder: ModelLadder, sizes: List[str]) -> None:
    import pandas as pd

    frames = []
    for size in sizes:
        df = ladder.get_metrics(size, prefix=args.prefix, discover_all=args.discover_all,
                                alternative_dirs=_alternative_dirs(args, ladder.name))
        if df is None:
            log.warning("no metrics found for size %s", size)
        else:
            frames.append(df)
    if not frames:
        return
    table = pd.concat(frames, ignore_index=True)
    target = io.join_path(args.output_dir, f"{ladder.name}/metrics{'' if len(sizes) > 1 else '_' + sizes[0]}.{args.format}")
    import os

    os.makedirs(os.path.dirname(str(target)), exist_ok=True)
    if args.format == "csv":
        table.to_csv(target, index=False)
    else:
        table.to_json(target, orient="records", lines=True)
    print(f"wrote {len(table)} row(s) to {target}")


def metrics(args: argparse.Namespace) -> None:
    prepare_cli_environment()
    _write_metrics(args, args.configure_ladder(args), [args.size])


def metrics_all(args: argparse.Namespace) -> None:
    prepare_cli_environment()
    ladder = args.configure_ladder(args)
    _write_metrics(args, ladder, _selected_sizes(args, ladder))


_COMMANDS = {
    "dry-run": (dry_run, "Show the plan (batch size, devices, schedule) for one model size."),
    "benchmark": (benchmark, "Run a short benchmark of one size on the current job's ranks."),
    "launch-benchmark": (launch_benchmark, "Submit a benchmark of one size to Beaker."),
    "run": (run, "Train one size on the current job's ranks."),
    "launch": (launch, "Submit the run of one size to Beaker."),
    "launch-all": (launch_all, "Submit the runs of all sizes to Beaker."),
    "status": (status, "Show which checkpoints and metrics of the ladder exist."),
    "metrics": (metrics, "Collect the metrics of one size into a table."),
    "metrics-all": (metrics_all, "Collect the metrics of all sizes into a table."),
}


def parse_args(configure_ladder: LadderFactory, *, size_enum: Type[TransformerSize] = TransformerSize,
               add_additional_args: Optional[Callable[[str, argparse.ArgumentParser], None]] = None,
               argv: Optional[List[str]] = None) -> argparse.Namespace:
    first = list(size_enum)[0]
    base = argparse.ArgumentParser(
        sys.argv[0], usage=f"python {sys.argv[0]} [CMD] [OPTIONS...]", formatter_class=argparse.RawDescriptionHelpFormatter,
        description=(f"Launch and manage a ladder experiment.\n\nexamples:\n  python {sys.argv[0]} dry-run --help\n"
                     f"  python {sys.argv[0]} dry-run --size={first}"),
        epilog="The command (e.g. 'dry-run', 'launch') must be the first argument.")
    subs = base.add_subparsers(dest="cmd")
    for name, (func, help_text) in _COMMANDS.items():
        p = subs.add_parser(name, help=help_text, formatter_class=argparse.ArgumentDefaultsHelpFormatter)
        p.set_defaults(func=func, configure_ladder=configure_ladder, size_enum=size_enum)
        p.add_argument("--name", type=str, default="olmo3-ladder", help="Name of the ladder experiment.")
        p.add_argument("--project", type=str, default=None, help="Project name for experiment trackers.")
        p.add_argument("--sequence-length", type=int, default=8192)
        p.add_argument("--chinchilla-multiple", type=float, default=4.0)
        p.add_argument("--lr-multiplier", type=float, default=1.0)
        p.add_argument("--stepped-schedule", action="store_true", help="Scale each period's peak LR by 1/sqrt(multiple).")
        p.add_argument("--cluster", type=str, default="ai2/jupiter", help="Beaker cluster, or 'local'.")
        p.add_argument("--max-gpus", type=int, default=64)
        p.add_argument("--rank-mbz", type=int, default=None, help="Override the per-device micro-batch, in instances.")
        if name not in _ALL_SIZES:
            p.add_argument("--size", type=str, choices=[str(s) for s in size_enum], required=name != "status")
        if name in ("status", "launch-all", "metrics-all"):
            p.add_argument("--max-size", type=str, choices=[str(s) for s in size_enum], default=None)
        if name in _LAUNCHING:
            p.add_argument("--workspace", type=str, default="ai2/oe-t-ladder")
            p.add_argument("--budget", type=str, default="ai2/oe-other")
            p.add_argument("--beaker-image", type=str, default=str(OLMoCoreBeakerImage.stable))
            p.add_argument("--priority", choices=["low", "normal", "high", "urgent"], default="normal")
            p.add_argument("--preemptible", action=argparse.BooleanOptionalAction)
            p.add_argument("--allow-dirty", action="store_true")
            p.add_argument("--slack-notifications", action="store_true")
            p.add_argument("--dry-run", action="store_true", help="Print what would be submitted.")
            p.add_argument("--follow", action=argparse.BooleanOptionalAction, default=name != "launch-all")
        if name == "dry-run":
            p.add_argument("--show-plot", action="store_true")
            p.add_argument("--save-plot", action="store_true")
            p.add_argument("--show-model", action="store_true")
        if name in ("dry-run", "metrics", "metrics-all"):
            p.add_argument("--output-dir", type=str, default="./ladder-output")
        if name in ("status", "metrics", "metrics-all"):
            p.add_argument("--discover-all", action="store_true", help="Use every checkpoint found, not only the planned ones.")
            p.add_argument("--alternative-root", action="append", help="Additional root dir(s) to search.")
        if name in ("metrics", "metrics-all"):
            p.add_argument("--prefix", type=str, default=None, help="Only keep metrics whose name starts with this.")
            p.add_argument("--format", choices=["csv", "jsonl"], default="csv")
        if add_additional_args is not None:
            add_additional_args(name, p)
    args = base.parse_args(argv)
    if args.cmd is None:
        base.print_help()
        sys.exit(1)
    return args


def main(configure_ladder: Optional[LadderFactory] = None,
         configure_model: Optional[Callable[[argparse.Namespace], ModelConfigurator]] = None,
         configure_run: Optional[Callable[[argparse.Namespace], RunConfigurator]] = None,
         size_enum: Type[TransformerSize] = TransformerSize,
         add_additional_args: Optional[Callable[[str, argparse.ArgumentParser], None]] = None) -> None:
    if configure_ladder is None:
        if configure_model is None:
            raise ValueError("configure_model is required if configure_ladder is unspecified")
        configure_ladder = get_default_ladder_factory(configure_model, configure_run)
    elif configure_model is not None or configure_run is not None:
        raise ValueError("configure_model / configure_run are mutually exclusive with configure_ladder")
    args = parse_args(configure_ladder, size_enum=size_enum, add_additional_args=add_additional_args)
    args.func(args)
