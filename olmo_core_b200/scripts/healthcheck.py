"""
Node health checks to run on every node before a job starts (role of src/scripts/lambda/healthchecks.sh and
src/scripts/lambda/distributed_test.py in the reference): exit non-zero so that the scheduler fails the job fast.

``python -m olmo_core_b200.scripts.healthcheck [--expect-gpus 8] [--temp-warn 50] [--temp-fail 55] [--max-used-mib 1024]
[--collectives]``

* **GPU inventory**: the number of visible devices matches ``--expect-gpus``.
* **Temperature**: an idle GPU that is already hot points at a stuck workload or a cooling problem.
* **Idle**: no foreign compute process and (almost) no memory in use.
* **Clocks**: a throttle reason other than idle / power cap that is active while idle, or an SM clock ceiling below the
  hardware maximum (a leftover clock lock), is reported. The check only READS the state (``nvidia-smi --query-gpu``); it
  changes no setting of any GPU.
* **Collectives** (``--collectives``, under ``torchrun``): one all-reduce per rank pair pattern with a known answer, the
  peer-memory rendezvous and the bounded cross-GPU barrier kernel of this package.

``OLMO_SKIP_HEALTHCHECKS=1`` skips everything (exit 0).
"""

from __future__ import annotations

import argparse
import logging
import os
import shutil
import subprocess
import sys
from dataclasses import dataclass, field
from typing import Callable, List, Optional

log = logging.getLogger("healthcheck")

QUERY_FIELDS = ("index", "temperature.gpu", "memory.used", "clocks.max.sm", "clocks.applications.graphics",
                "clocks_event_reasons.hw_slowdown", "clocks_event_reasons.hw_thermal_slowdown",
                "clocks_event_reasons.sw_thermal_slowdown")


@dataclass
class Report:
    failures: List[str] = field(default_factory=list)
    warnings: List[str] = field(default_factory=list)

    def fail(self, msg: str) -> None:
        log.error(msg)
        self.failures.append(msg)

    def warn(self, msg: str) -> None:
        log.warning(msg)
        self.warnings.append(msg)

    @property
    def ok(self) -> bool:
        return not self.failures


def _run_smi(args: List[str]) -> str:
    exe = shutil.which("nvidia-smi")
    if exe is None:
        raise FileNotFoundError("nvidia-smi not found in PATH")
    return subprocess.run([exe, *args], capture_output=True, text=True, check=True, timeout=60).stdout


def check_gpus(report: Report, *, expect_gpus: Optional[int], temp_warn: int, temp_fail: int, max_used_mib: int,
               smi: Callable[[List[str]], str] = _run_smi) -> None:
    """Inventory, temperature, idleness and clock state of this node's GPUs, from two read-only nvidia-smi queries."""
    if temp_fail < temp_warn:
        raise ValueError(f"fail threshold ({temp_fail} C) below warn threshold ({temp_warn} C)")
    try:
        rows = [r for r in smi([f"--query-gpu={','.join(QUERY_FIELDS)}", "--format=csv,noheader,nounits"]).splitlines() if r.strip()]
    except Exception as e:
        report.fail(f"unable to query GPUs: {e}")
        return
    if expect_gpus is not None and len(rows) != expect_gpus:
        report.fail(f"expected {expect_gpus} GPUs on {os.uname().nodename}, nvidia-smi lists {len(rows)}")
    hottest = (-1, "?")
    for row in rows:
        cells = [c.strip() for c in row.split(",")]
        if len(cells) != len(QUERY_FIELDS):
            report.fail(f"could not parse nvidia-smi row: '{row}'")
            continue
        idx, temp, used, max_sm, app_clock, hw_slow, hw_therm, sw_therm = cells
        try:
            temp_c, used_mib = int(temp), int(used)
        except ValueError:
            report.fail(f"could not parse temperature / memory of GPU {idx}: '{temp}', '{used}'")
            continue
        hottest = max(hottest, (temp_c, idx))
        if temp_c >= temp_fail:
            report.fail(f"GPU {idx} is at {temp_c} C while idle (>= {temp_fail} C)")
        elif temp_c >= temp_warn:
            report.warn(f"GPU {idx} is at {temp_c} C while idle (>= {temp_warn} C)")
        if used_mib > max_used_mib:
            report.fail(f"GPU {idx} already has {used_mib} MiB in use (> {max_used_mib} MiB): not idle")
        for name, value in (("hw_slowdown", hw_slow), ("hw_thermal_slowdown", hw_therm), ("sw_thermal_slowdown", sw_therm)):
            if value.lower() == "active":
                report.fail(f"GPU {idx} reports {name} while idle")
        if app_clock.isdigit() and max_sm.isdigit() and int(app_clock) < int(max_sm) * 0.9:
            report.warn(f"GPU {idx}: application clock {app_clock} MHz is below its maximum {max_sm} MHz (clock lock left behind?)")
    if rows and hottest[0] >= 0:
        log.info(f"hottest GPU: {hottest[1]} at {hottest[0]} C (warn {temp_warn}, fail {temp_fail})")
    try:
        procs = [r for r in smi(["--query-compute-apps=pid,process_name,used_memory", "--format=csv,noheader,nounits"]).splitlines()
                 if r.strip()]
    except Exception as e:
        report.warn(f"unable to list compute processes: {e}")
        procs = []
    mine = str(os.getpid())
    foreign = [p for p in procs if p.split(",")[0].strip() != mine]
    if foreign:
        report.fail(f"{len(foreign)} compute process(es) already on this node's GPUs: {foreign[:4]}")


def check_collectives(report: Report) -> None:
    """All-reduce with a known answer over NCCL, then this package's peer-memory rendezvous and barrier kernel."""
    import torch
    import torch.distributed as dist

    from olmo_core_b200.distributed.utils import get_local_rank, get_rank, get_world_size

    started_here = False
    if not dist.is_initialized():
        if "RANK" not in os.environ:
            log.info("not under torchrun: skipping the collective checks")
            return
        torch.cuda.set_device(get_local_rank())
        dist.init_process_group("cpu:gloo,cuda:nccl")
        started_here = True
    rank, world = get_rank(), get_world_size()
    device = torch.device("cuda", torch.cuda.current_device())
    x = torch.full((1 << 20,), float(rank + 1), device=device)
    dist.all_reduce(x)
    want = world * (world + 1) / 2
    if not torch.all(x == want):
        report.fail(f"rank {rank}: all-reduce returned {x[0].item()}, expected {want}")
    if world > 1:
        try:
            from olmo_core_b200.ops import _lib
            from olmo_core_b200.parallel.symmetric import SymmetricBuffer, symmetric_memory_enabled

            if symmetric_memory_enabled(device):
                buf = SymmetricBuffer(1024, torch.float32, device)
                buf.barrier(timeout_ms=10_000)
                torch.cuda.synchronize()
                _lib.check_device_status(device)
                log.info(f"rank {rank}: peer-memory rendezvous and barrier ok ({buf})")
        except Exception as e:
            report.fail(f"rank {rank}: peer-memory check failed: {type(e).__name__}: {e}")
    dist.barrier()
    if started_here:
        dist.destroy_process_group()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--expect-gpus", type=int, default=None)
    ap.add_argument("--temp-warn", type=int, default=int(os.environ.get("OLMO_GPU_TEMP_WARN_C", 50)))
    ap.add_argument("--temp-fail", type=int, default=int(os.environ.get("OLMO_GPU_TEMP_FAIL_C", 55)))
    ap.add_argument("--max-used-mib", type=int, default=1024)
    ap.add_argument("--collectives", action="store_true")
    args = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO, format="[healthcheck] %(levelname)s %(message)s")
    if os.environ.get("OLMO_SKIP_HEALTHCHECKS", "0") == "1":
        log.info("SKIP (OLMO_SKIP_HEALTHCHECKS=1)")
        return 0
    report = Report()
    if os.environ.get("OLMO_SKIP_GPU_TEMP_CHECK", "0") == "1":
        args.temp_warn = args.temp_fail = 10_000
    if int(os.environ.get("LOCAL_RANK", "0")) == 0:
        check_gpus(report, expect_gpus=args.expect_gpus, temp_warn=args.temp_warn, temp_fail=args.temp_fail,
                   max_used_mib=args.max_used_mib)
    if args.collectives and report.ok:
        check_collectives(report)
    if not report.ok:
        log.error(f"{len(report.failures)} check(s) failed on {os.uname().nodename}")
        return 1
    log.info(f"all checks passed ({len(report.warnings)} warning(s))")
    return 0


if __name__ == "__main__":
    sys.exit(main())
