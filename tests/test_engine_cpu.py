"""The collective engine without a GPU: gloo ranks, stand-in device, shared-memory peers.

The engine, the transport and the ring / hierarchy schedules are the product's C++
code; only the device is a stand-in (host memory, the kernels' CPU statement).  The
GPU counterparts of these cases are in test_engine.py and test_multigpu.py.
"""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

from conftest import free_port

ROOT = Path(__file__).resolve().parent.parent


def _run(nproc, gpus_per_node, timeout=420, **envkw):
    env = dict(os.environ)
    env.update({"TCPXB_TEST_GPUS_PER_NODE": str(gpus_per_node), "OMP_NUM_THREADS": "1", "TCPXB_FAKE_GPU": "1"})
    env.update({k: str(v) for k, v in envkw.items()})
    worker = str(ROOT / "tests" / "engine_cpu_worker.py")
    if nproc == 1:
        cmd = [sys.executable, worker]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
               "--master-addr", "127.0.0.1", "--master-port", str(free_port()), worker]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    rows = []
    for line in r.stdout.splitlines():
        for part in line.replace("}{", "}\n{").splitlines():
            if part.startswith('{"rank"'):
                rows.append(json.loads(part))
    return r, rows


@pytest.mark.parametrize("nproc,gpn", [(1, 1), (2, 1), (3, 1), (4, 2), (6, 2), (6, 3)])
def test_collectives_match_fp32_sums(nproc, gpn):
    """all_reduce (twice per size), all_gather, reduce_scatter in bf16 and fp32, plus send/recv
    around the ring: twin, two nodes, a three-node ring, and hierarchies of 2 x 2, 3 x 2, 2 x 3."""
    r, rows = _run(nproc, gpn)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert len(rows) == nproc and all(row["ok"] and row["device_status"][0] == 0 for row in rows)
    assert all(row["unpack_launches"] > 0 and row["fragments"] >= row["unpack_launches"] for row in rows)


@pytest.mark.parametrize("envkw", [dict(TCPXB_TEST_PLAIN=1), dict(TCPXB_TEST_REDUCE_IMPL=1),
                                   dict(NCCL_GPUDIRECTTCPX_RX_POOL_SCATTER=1, NCCL_GPUDIRECTTCPX_RX_POOL_BYTES=8 << 20),
                                   dict(TCPXB_TEST_WAKE_ON_EVENTS=1, TCPXB_TEST_IDLE_SLEEP_US=200),
                                   dict(TCPXB_TEST_IDLE_SLEEP_US=-1),
                                   dict(NCCL_GPUDIRECTTCPX_SOCKET_SNDBUF=65536, NCCL_GPUDIRECTTCPX_HELPER_NAP_US=0)])
def test_engine_variants(envkw):
    """The unfused baseline, the add-at-destination reduce, a small scattered page pool; the driving thread
    woken by events instead of napping, and spinning; bounded socket buffers with helpers that never nap."""
    r, rows = _run(4, 2, **envkw)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert len(rows) == 4 and all(row["ok"] for row in rows)


@pytest.mark.parametrize("nproc,gpn,asynchronous", [(2, 1, 0), (3, 1, 0), (4, 2, 0), (2, 1, 1), (4, 2, 1)])
def test_a_rank_that_leaves_is_an_error_for_the_others(nproc, gpn, asynchronous):
    """The last rank exits at a step boundary.  Its network neighbours get an error from the
    transport at once; its node-mates' bounded flag waits run out and set the device status.
    Nobody hangs, and the step before the exit was correct everywhere.  With the asynchronous
    call the error of the engine's own thread reaches the caller at `wait()`."""
    r, rows = _run(nproc, gpn, timeout=180, TCPXB_TEST_MODE="rank_leaves", TCPXB_TEST_ASYNC=asynchronous)
    assert len(rows) == nproc, r.stdout[-3000:] + r.stderr[-3000:]
    assert all(row["first_ok"] for row in rows)
    left = [row for row in rows if row["left"]]
    stayed = [row for row in rows if not row["left"]]
    assert len(left) == 1 and left[0]["rank"] == nproc - 1
    for row in stayed:
        assert row["outcome"] != "completed", row
        assert row["seconds"] < 30
    assert any(row["outcome"].startswith("error") for row in stayed)  # the ring neighbour saw the closed sockets
    if gpn > 1:
        mates = [row for row in stayed if row["rank"] // gpn == (nproc - 1) // gpn]
        assert mates and all(row["device_status"][0] == 3 for row in mates)  # TCPXB_ST_TIMEOUT
