"""Hierarchical engine on one GPU: the rank is its own network peer (twin node), so every
byte goes isend -> pinned staging -> loopback sockets -> rx page pool -> fused unpack kernel."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def engine():
    from nccl_plugin_gpudirecttcpx_b200.parallel.engine import HierarchicalEngine, default_transport_env
    default_transport_env(nics=2, nthreads=2, nsocks_per_thread=1, pool_mb=256)
    e = HierarchicalEngine(gpus_per_node=1, request_bytes=1 << 20)
    yield e
    e.close()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("numel", [8, 4096, (1 << 20) + 8, 6 << 20])
def test_twin_all_reduce_doubles(engine, dtype, numel):
    x = torch.randn(numel, device="cuda", generator=torch.Generator("cuda").manual_seed(numel)).to(dtype)
    out = engine.all_reduce(x)
    torch.cuda.synchronize()
    want = (x.float() * 2).to(dtype)
    assert torch.equal(out, want)
    assert engine.device_status()[0] == 0


@pytest.mark.parametrize("numel", [1, 7, (1 << 20) + 3])
def test_twin_all_reduce_of_any_size(engine, numel):
    """Sizes below the 16-byte granularity of the native call are padded inside the binding."""
    x = torch.randn(numel, device="cuda", generator=torch.Generator("cuda").manual_seed(numel)).to(torch.bfloat16)
    out = engine.all_reduce(x)
    torch.cuda.synchronize()
    assert out.shape == x.shape and torch.equal(out, (x.float() * 2).to(torch.bfloat16))
    given = torch.empty_like(x)
    assert engine.all_reduce(x, given) is given
    torch.cuda.synchronize()
    assert torch.equal(given, out)


def test_twin_all_gather_and_reduce_scatter_of_any_size(engine):
    x = torch.randn(1001, device="cuda")  # 4004 bytes: no multiple of 16
    g = engine.all_gather(x)
    torch.cuda.synchronize()
    assert g.shape == (2002,) and torch.equal(g[:1001], x) and torch.equal(g[1001:], x)
    r = engine.reduce_scatter(x)
    torch.cuda.synchronize()
    assert r.shape == (1001,) and torch.equal(r, 2 * x)


def test_twin_all_gather_and_reduce_scatter(engine):
    x = torch.randn(3 << 18, device="cuda").to(torch.bfloat16)
    g = engine.all_gather(x)
    torch.cuda.synchronize()
    assert g.numel() == 2 * x.numel() and torch.equal(g[:x.numel()], x) and torch.equal(g[x.numel():], x)
    r = engine.reduce_scatter(x)
    torch.cuda.synchronize()
    assert torch.equal(r, (x.float() * 2).to(torch.bfloat16))


def test_twin_send_recv_and_stats(engine):
    import threading
    x = torch.randint(0, 255, (5 << 20,), dtype=torch.uint8, device="cuda")
    y = torch.zeros_like(x)
    before = engine.stats().bytes_received
    # the single rank is both ends: send and receive in one exchange via all_gather's path
    g = engine.all_gather(x)
    torch.cuda.synchronize()
    assert torch.equal(g[x.numel():], x)
    s = engine.stats()
    assert s.bytes_received - before == x.numel() and s.fragments > 0 and s.unpack_launches > 0


def test_plain_mode_matches_fused():
    from nccl_plugin_gpudirecttcpx_b200.parallel.engine import HierarchicalEngine
    e = HierarchicalEngine(gpus_per_node=1, request_bytes=1 << 20, plain_mode=True)
    try:
        x = torch.randn(3 << 20, device="cuda").to(torch.bfloat16)
        out = e.all_reduce(x)
        torch.cuda.synchronize()
        assert torch.equal(out, (x.float() * 2).to(torch.bfloat16))
    finally:
        e.close()


@pytest.mark.parametrize("pool", ["host", "device"])
def test_engine_with_pool_from_the_rx_buffer_manager_daemon(tmp_path, pool):
    """Same path, but the rx page pool comes from the rx buffer manager daemon over a UNIX socket:
    host memory as a memfd, or GPU memory the daemon allocated with the driver's virtual memory API,
    exported as a file descriptor and imported here (RX_POOL_MODE=device RX_BUF_MGR=daemon)."""
    import subprocess
    import sys
    from pathlib import Path
    from nccl_plugin_gpudirecttcpx_b200 import _build
    _build.build_host()
    prefix = tmp_path / "rxdm"
    cmd = [str(_build.OUT / "tcpxb_rxdm"), "--prefix", str(prefix), "--pool-mb", "64"]
    if pool == "device":
        cmd = [str(_build.OUT / "tcpxb_rxdm_gpu"), "--prefix", str(prefix), "--pool-mb", "64", "--device-pool"]
    daemon = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    try:
        assert daemon.stdout.readline().strip() == "ready"
        env = dict(os.environ, NCCL_GPUDIRECTTCPX_RX_BUF_MGR="daemon", NCCL_GPUDIRECTTCPX_UNIX_CLIENT_PREFIX=str(prefix),
                   NCCL_GPUDIRECTTCPX_REPORT_LIFECYCLE="1")
        r = subprocess.run([sys.executable, str(Path(__file__).parent / "rxdm_engine_worker.py")], env=env,
                           capture_output=True, text=True, timeout=120)
        assert r.returncode == 0 and "rxdm engine ok" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
    finally:
        daemon.terminate()
        try:
            daemon.wait(timeout=5)
        except subprocess.TimeoutExpired:
            daemon.kill()
    err = daemon.stderr.read()
    assert "pool for GPU" in err and f"of {pool} memory" in err
