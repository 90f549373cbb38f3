"""Multi-GPU tests: stock NCCL through the plugin, and the hierarchical engine.

Each case runs as child processes under torch.distributed.run with a hard time
limit, one rank per GPU.  Ranks leave only between steps, nothing here faults or
hangs a GPU on purpose.
"""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from conftest import free_port

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

ROOT = Path(__file__).resolve().parent.parent
NGPU = torch.cuda.device_count() if torch.cuda.is_available() else 0


def _run(worker, nproc, env_extra, timeout=150, port=None):
    port = port or free_port()
    env = dict(os.environ)
    env.update(env_extra)
    env.setdefault("TCPXB_TEST_DUMP_AFTER", str(timeout - 20))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(ROOT / "tests" / worker)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    rows = []
    for line in r.stdout.splitlines():
        for part in line.replace("}{", "}\n{").splitlines():
            if part.startswith('{"rank"'):
                rows.append(json.loads(part))
    return r, rows


@pytest.mark.parametrize("mode", ["host", "unpack"])
def test_nccl_collectives_through_the_plugin(mode):
    """all_reduce / all_gather / reduce_scatter of stock NCCL, every byte over the plugin."""
    from nccl_plugin_gpudirecttcpx_b200.parallel import plugin_env
    env = plugin_env(nics=2, nthreads=2, recv_mode=mode, rx_pool_mb=256)
    env["TCPXB_TEST_SIZES"] = "256,65536,1048576"
    env["TCPXB_TEST_BW_ELEMS"] = str(1 << 20)
    r, rows = _run("nccl_plugin_worker.py", 2, env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert len(rows) == 2 and all(row["ok"] for row in rows)


def test_nccl_socket_transport_gives_the_same_results():
    from nccl_plugin_gpudirecttcpx_b200.parallel import plugin_env
    env = plugin_env(nics=2, nthreads=2, builtin_socket=True)
    env["TCPXB_TEST_SIZES"] = "256,65536"
    env["TCPXB_TEST_BW_ELEMS"] = str(1 << 20)
    r, rows = _run("nccl_plugin_worker.py", 2, env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert len(rows) == 2 and all(row["ok"] for row in rows)


@pytest.mark.parametrize("world,G", [(2, 1), (4, 1), (4, 2), (8, 1), (8, 4)])
def test_nccl_plugin_agrees_with_the_socket_transport(world, G):
    """The same seeded collectives through stock NCCL twice: over this plugin and over NCCL's own
    socket transport, `world` ranks in nodes of G GPUs.  Each run is held to the fp32 oracle by the
    worker; here the two are also held to each other (all_gather bit for bit inside the worker,
    all_reduce samples within the rounding the differing channel layouts allow)."""
    if NGPU < world:
        pytest.skip(f"needs {world} GPUs")
    from nccl_plugin_gpudirecttcpx_b200.parallel import plugin_env
    results = {}
    for arm in ("plugin", "socket"):
        env = plugin_env(nics=2, nthreads=2, builtin_socket=(arm == "socket"), rx_pool_mb=256)
        if G > 1:  # nodes by host id: NVLink inside a node, the net transport between nodes
            env.pop("NCCL_P2P_DISABLE", None)
            env.pop("NCCL_SHM_DISABLE", None)
        env["TCPXB_TEST_GPUS_PER_NODE"] = str(G)
        env["TCPXB_TEST_SIZES"] = "256,65536,1048576"
        env["TCPXB_TEST_BW_ELEMS"] = str(1 << 20)
        r, rows = _run("nccl_plugin_worker.py", world, env, timeout=240)
        assert r.returncode == 0, arm + ": " + r.stdout[-2000:] + r.stderr[-3000:]
        assert len(rows) == world and all(row["ok"] for row in rows), arm
        results[arm] = {row["rank"]: row["samples"] for row in rows}
    for rank in range(world):
        for a, b in zip(results["plugin"][rank], results["socket"][rank]):
            for va, vb in zip(a, b):
                assert abs(va - vb) <= 0.05 * world * max(1.0, abs(vb)) * 2 ** -3, (rank, va, vb)


@pytest.mark.parametrize("world,G", [(2, 1), (4, 1), (4, 2), (8, 4)])
def test_engine_collectives(world, G):
    if NGPU < world:
        pytest.skip(f"needs {world} GPUs")
    r, rows = _run("engine_worker.py", world, {"TCPXB_TEST_GPUS_PER_NODE": str(G), "NCCL_NVLS_ENABLE": "0"}, timeout=200)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert len(rows) == world and all(row["ok"] for row in rows), rows


def test_engine_plain_mode_matches():
    r, rows = _run("engine_worker.py", 2, {"TCPXB_TEST_PLAIN": "1", "TCPXB_TEST_NUMELS": "4096,1048576"})
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert len(rows) == 2 and all(row["ok"] for row in rows)
