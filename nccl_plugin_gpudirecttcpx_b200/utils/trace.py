"""Reads the transport's exporter logs and says where requests and tasks spend their time.

The transport writes one line per queue transition when the telemetry switches are on
(`NCCL_GPUDIRECTTCPX_TELEMETRY_EXPORT_STATS_TO_FILE=1` plus the task / request level
switches), in the reference's format (reference: src/stats/stats_buffer.h:105-116,
src/stats/exporter.h:38-57):

    <T|R> <object address> <passive 0|1> <STATE> <nanoseconds since the epoch>

Objects are ring slots and are reused, so a life is the run of lines of one address from
its first state (POSTED for requests, ACTIVE for tasks) to FREE.  For every pair of
consecutive states this module reports how long objects sat in the first one.

    python -m nccl_plugin_gpudirecttcpx_b200.utils.trace /path/to/exporter_*.log
"""
from __future__ import annotations

import json
import statistics
import sys
from collections import defaultdict
from typing import Dict, Iterable, List, Tuple

FIRST_STATE = {"R": "POSTED", "T": "ACTIVE"}


def parse_lines(lines: Iterable[str]) -> List[Tuple[str, str, int, str, int]]:
    """(kind, address, passive, state, ns) per well-formed line; others are skipped."""
    out = []
    for line in lines:
        w = line.split()
        if len(w) != 5 or w[0] not in FIRST_STATE:
            continue
        try:
            out.append((w[0], w[1], int(w[2]), w[3], int(w[4])))
        except ValueError:
            continue
    return out


def dwell_times(events: List[Tuple[str, str, int, str, int]]) -> Dict[Tuple[str, str, str, str], List[int]]:
    """{(kind, side, state, next_state): [ns spent in `state` before `next_state`, ...]}.
    A life that does not begin with its first state (the log started in its middle, or
    lines were dropped when the bounded ring was full) is skipped until its next beginning."""
    last: Dict[Tuple[str, str], Tuple[str, int]] = {}
    out: Dict[Tuple[str, str, str, str], List[int]] = defaultdict(list)
    for kind, addr, passive, state, ns in sorted(events, key=lambda e: e[4]):
        key = (kind, addr)
        side = "recv" if passive else "send"
        if state == FIRST_STATE[kind]:
            last[key] = (state, ns)
            continue
        if key not in last:
            continue
        prev_state, prev_ns = last[key]
        out[(kind, side, prev_state, state)].append(ns - prev_ns)
        if state == "FREE":
            del last[key]
        else:
            last[key] = (state, ns)
    return out


def summarize(paths: Iterable[str]) -> List[dict]:
    # one file per comm: addresses mean something only inside their own file
    merged: Dict[Tuple[str, str, str, str], List[int]] = defaultdict(list)
    for p in paths:
        with open(p) as f:
            for key, ns in dwell_times(parse_lines(f)).items():
                merged[key].extend(ns)
    rows = []
    for (kind, side, a, b), ns in sorted(merged.items()):
        ns.sort()
        rows.append({
            "kind": "request" if kind == "R" else "task", "side": side, "from": a, "to": b, "count": len(ns),
            "mean_us": round(statistics.fmean(ns) / 1e3, 2), "p50_us": round(ns[len(ns) // 2] / 1e3, 2),
            "p99_us": round(ns[min(len(ns) - 1, int(len(ns) * 0.99))] / 1e3, 2), "max_us": round(ns[-1] / 1e3, 2),
        })
    return rows


def main(argv=None) -> int:
    paths = list(argv if argv is not None else sys.argv[1:])
    if not paths or paths[0] in ("-h", "--help"):
        print(__doc__)
        return 0 if paths else 2
    for row in summarize(paths):
        print(json.dumps(row))
    return 0


if __name__ == "__main__":
    sys.exit(main())
