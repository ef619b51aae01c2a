"""
Topology-aware node ranks on GCP: print the rank this node should use so that nodes sharing a block / sub-block /
machine are adjacent (which keeps ring and tree collectives on short paths) while rank 0 stays rank 0.
CLI of src/olmo_core/launch/reorder_ranks_in_gcp.py:9-108: ``python -m olmo_core_b200.launch.reorder_ranks_in_gcp
RANK WORLD_SIZE MASTER_ADDR``; the node ids travel through a ``TCPStore`` on rank 0.

The ordering itself is the pure function :func:`topology_order`, which tests exercise without any network.
"""

from __future__ import annotations

import argparse
import socket
import sys
from typing import List, Optional, Sequence, Tuple

__all__ = ["topology_order", "physical_host_id", "main"]

_METADATA_URL = "http://metadata.google.internal/computeMetadata/v1/instance/attributes/physical_host"


def _parts(host_id: str) -> Tuple[str, ...]:
    parts = tuple(host_id.strip("/").split("/"))
    if len(parts) < 3:
        raise ValueError(f"expected a host id of the form /block/subblock/machine, got {host_id!r}")
    return parts[:3]


def topology_order(host_ids: Sequence[str]) -> List[int]:
    """
    Old ranks in their new order. Rank 0 stays first; then come the ranks that share its machine, its sub-block, its
    block, and after them the remaining blocks, each grouped the same way; ties keep the lower old rank first.
    """
    if len(set(host_ids)) != len(host_ids):
        raise ValueError("host ids must be unique")
    parts = [_parts(h) for h in host_ids]
    first = parts[0]

    def key(rank: int):
        mine = parts[rank]
        away = tuple(mine[: i + 1] != first[: i + 1] for i in range(3))  # False sorts first: closest to rank 0
        return away + mine + (rank,)

    order = sorted(range(len(host_ids)), key=key)
    assert order[0] == 0
    return order


def physical_host_id(timeout: float = 5.0) -> Optional[str]:
    """This VM's ``/block/subblock/machine`` id from the metadata server; ``None`` outside of GCP."""
    import requests

    try:
        r = requests.get(_METADATA_URL, headers={"Metadata-Flavor": "Google"}, timeout=timeout)
    except requests.exceptions.RequestException:
        return None
    return r.text.strip() if r.status_code == 200 else None


def main(argv: Optional[Sequence[str]] = None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("rank", type=int)
    ap.add_argument("world_size", type=int)
    ap.add_argument("master_addr")
    ap.add_argument("--master_port", type=int, default=29501)
    ap.add_argument("--debug", action="store_true", help="use hostname-derived ids (for runs outside of GCP)")
    ap.add_argument("--verbose", action="store_true", help="rank 0 prints the whole mapping to stderr")
    args = ap.parse_args(argv)

    host_id = f"/dbg/dbg/{socket.gethostname()}_{args.rank}" if args.debug else physical_host_id()
    if host_id is None:  # not on GCP: keep the rank we were given
        print(args.rank)
        return

    import torch.distributed as dist

    store = dist.TCPStore(args.master_addr, args.master_port, args.world_size, is_master=args.rank == 0)
    store.set(f"host/{args.rank}", host_id)
    keys = [f"host/{i}" for i in range(args.world_size)]
    store.wait(keys)
    order = topology_order([store.get(k).decode() for k in keys])
    if args.verbose and args.rank == 0:
        for new, old in enumerate(order):
            print(f"rank {old} -> {new}", file=sys.stderr)
    print(order.index(args.rank))
    store.set(f"done/{args.rank}", "1")  # keep the store alive until everybody has read it
    store.wait([f"done/{i}" for i in range(args.world_size)])


if __name__ == "__main__":
    main()
