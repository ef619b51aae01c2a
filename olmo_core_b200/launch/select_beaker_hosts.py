"""
Pick Beaker hosts for a multi-node job so that every execution unit (a set of nodes that must share low-latency
networking, e.g. one pipeline stage) lands inside one physical block of the GCP cluster.
API of src/olmo_core/launch/select_beaker_hosts.py:19-325: :class:`HostMetadata`, :func:`get_hostname_constraints`
(pure, tested on CPU), and the Beaker / GCP lookups which need the ``beaker`` and ``google-cloud-compute`` clients.
"""

from __future__ import annotations

import argparse
import logging
from collections import defaultdict
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence, Set, Tuple

from ..exceptions import BeakerInsufficientResourcesError, OLMoEnvironmentError

log = logging.getLogger(__name__)

__all__ = ["HostMetadata", "get_hostname_constraints", "get_hosts_metadata_from_gcp", "get_occupied_beaker_hosts",
           "get_beaker_hostname_constraints", "main"]


@dataclass
class HostMetadata:
    block: str      #: hosts of one block see low network latency among themselves
    subblock: str   #: lower still inside a sub-block
    machine: str    #: physical machine


def get_hostname_constraints(hosts_metadata: Dict[str, HostMetadata], num_execution_units: int, num_hosts_per_task: int,
                             num_tasks: int, occupied_hosts: Optional[Set[str]] = None) -> List[List[str]]:
    """
    One host list per task. If a single block has more free hosts than the whole job needs, every task may use any
    host of that block (busy ones included: they may free up). Otherwise blocks are consumed from the emptiest down,
    each contributing a whole number of execution units.
    """
    total_hosts = num_hosts_per_task * num_tasks
    if num_hosts_per_task % num_execution_units != 0:
        raise ValueError("the number of execution units must divide the number of hosts of a task")
    unit = total_hosts // num_execution_units
    busy = occupied_hosts or set()

    members: Dict[str, List[str]] = defaultdict(list)
    free: Dict[str, List[str]] = defaultdict(list)
    for host, meta in hosts_metadata.items():
        members[meta.block].append(host)
        if host not in busy:
            free[meta.block].append(host)
    blocks = sorted(free, key=lambda blk: len(free[blk]), reverse=True)
    if not blocks:
        raise BeakerInsufficientResourcesError("no free hosts")
    if len(free[blocks[0]]) > total_hosts:
        return [list(members[blocks[0]]) for _ in range(num_tasks)]

    tasks: List[List[str]] = []
    cursor = 0
    for task in range(num_tasks):
        chosen: List[str] = []
        while len(chosen) < num_hosts_per_task and cursor < len(blocks):
            pool = free[blocks[cursor]]
            whole_units = len(pool) // unit * unit
            if whole_units == 0:
                cursor += 1
                continue
            take = min(num_hosts_per_task - len(chosen), whole_units)
            chosen += pool[:take]
            free[blocks[cursor]] = pool[take:]
        if len(chosen) < num_hosts_per_task:
            raise BeakerInsufficientResourcesError(
                f"task {task + 1} of {num_tasks}: found {len(chosen)} of {num_hosts_per_task} hosts with every "
                f"execution unit ({unit} hosts) inside one block"
            )
        tasks.append(chosen)
    return tasks


def get_hosts_metadata_from_gcp(zone: str, *, credentials_path: Optional[Path] = None) -> Dict[str, HostMetadata]:
    try:
        import google.auth
        from google.cloud.compute_v1 import InstancesClient
    except ImportError as e:
        raise OLMoEnvironmentError("host selection needs the 'google-cloud-compute' package") from e
    if credentials_path is not None:
        credentials, project = google.auth.load_credentials_from_file(str(credentials_path))
    else:
        credentials, project = google.auth.default()
    out: Dict[str, HostMetadata] = {}
    for page in InstancesClient(credentials=credentials).list(project=project, zone=zone).pages:
        for inst in page.items:
            if inst.status == "RUNNING":
                topo = inst.resource_status.physical_host_topology
                out[f"{inst.name}.reviz.ai2.in"] = HostMetadata(topo.block, topo.subblock, topo.host)
    return out


_PRIORITY_ORDER = ["low", "normal", "high", "urgent"]


def node_is_occupied(beaker, node, beaker_priority) -> Tuple[Any, bool]:
    """``(node, True)`` when the node runs a job that holds slots and that ``beaker_priority`` cannot preempt."""
    want = str(getattr(beaker_priority, "value", beaker_priority)).lower()
    want_rank = _PRIORITY_ORDER.index(want) if want in _PRIORITY_ORDER else 1
    for job in beaker.job.list(scheduled_on_node=node):
        details = getattr(job, "assignment_details", None)
        slots = getattr(getattr(details, "resource_assignment", None), "assigned_slots_count", 1)
        have = str(getattr(getattr(job, "priority", None), "value", getattr(job, "priority", None)) or "normal").lower()
        have_rank = _PRIORITY_ORDER.index(have) if have in _PRIORITY_ORDER else 1
        preemptible = bool(getattr(job, "preemptible", False)) and have_rank < want_rank
        if slots > 0 and not preemptible:
            return node, True
    return node, False


def get_occupied_beaker_hosts(hosts_metadata: Dict[str, HostMetadata], beaker_cluster: str, beaker_priority: str) -> Set[str]:
    """Hosts of the cluster that run a job this priority cannot preempt."""
    try:
        from beaker import Beaker
    except ImportError as e:
        raise OLMoEnvironmentError("host selection needs the 'beaker-py' package") from e
    ranks = ["low", "normal", "high", "urgent"]
    priority = str(beaker_priority).lower()
    beaker = Beaker.from_env()
    busy: Set[str] = set()
    for node in beaker.cluster.nodes(beaker_cluster):
        if node.hostname not in hosts_metadata:
            continue
        for job in beaker.job.list(node=node.id, finalized=False):
            job_priority = str(getattr(job, "priority", None) or "normal").lower()
            if ranks.index(job_priority if job_priority in ranks else "normal") >= ranks.index(priority):
                busy.add(node.hostname)
                break
    return busy


def get_beaker_hostname_constraints(num_nodes: int, num_execution_units: int, beaker_task_count: int, gcp_zone: str, *,
                                    beaker_cluster: str, beaker_priority: str = "urgent",
                                    gcp_credentials_path: Optional[Path] = None,
                                    hosts_metadata: Optional[Dict[str, HostMetadata]] = None) -> List[List[str]]:
    if num_nodes <= 0 or num_nodes % num_execution_units or num_nodes % beaker_task_count:
        raise ValueError("the node count must be a positive multiple of the execution units and of the task count")
    if str(beaker_priority) != "urgent":
        log.warning("host selection assumes it can preempt lower-priority jobs; it rarely works below 'urgent'")
    if hosts_metadata is None:
        hosts_metadata = get_hosts_metadata_from_gcp(gcp_zone, credentials_path=gcp_credentials_path)
    busy = get_occupied_beaker_hosts(hosts_metadata, beaker_cluster, str(beaker_priority))
    return get_hostname_constraints(hosts_metadata, num_execution_units, num_nodes // beaker_task_count,
                                    beaker_task_count, busy)


def main(argv: Optional[Sequence[str]] = None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("num_nodes", type=int)
    ap.add_argument("--num-execution-units", type=int, default=1)
    ap.add_argument("--task-count", type=int, default=1)
    ap.add_argument("--zone", default="us-central1-b")
    ap.add_argument("--cluster", default="ai2/augusta")
    ap.add_argument("--priority", default="urgent")
    ap.add_argument("--credentials", type=Path, default=None)
    args = ap.parse_args(argv)
    for hosts in get_beaker_hostname_constraints(args.num_nodes, args.num_execution_units, args.task_count, args.zone,
                                                 beaker_cluster=args.cluster, beaker_priority=args.priority,
                                                 gcp_credentials_path=args.credentials):
        print(",".join(hosts))


if __name__ == "__main__":
    main()
