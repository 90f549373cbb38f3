"""CPU tests of the C++ host core: unit tests, the ncclNet API loopback, sanitizer builds."""
import json
import os
import re
import subprocess
import sys
from pathlib import Path

import pytest

from nccl_plugin_gpudirecttcpx_b200 import _build

LIB = _build.OUT


@pytest.fixture(scope="module")
def host_lib():
    return _build.build_host()


def _env(**kw):
    env = dict(os.environ)
    env.update({
        "NCCL_GPUDIRECTTCPX_SOCKET_IFNAME": "lo",
        "NCCL_GPUDIRECTTCPX_VIRTUAL_NICS": "2",
        "NCCL_SOCKET_NTHREADS": "2",
        "NCCL_NSOCKS_PERTHREAD": "2",   # 4 sockets per comm
    })
    env.update({k: str(v) for k, v in kw.items()})
    if env.get("NCCL_GPUDIRECTTCPX_RECV_MODE") == "unpack" and "NCCL_PROTO" not in kw:
        # the settings unpack mode is documented with; without them the plugin falls back to host mode
        env.update({"NCCL_PROTO": "Simple", "NCCL_ALGO": "Ring"})
    return env


def _loopback(host_lib, args=(), exe="tcpxb_loopback", plugin=None, timeout=300, **envkw):
    cmd = [str(LIB / exe), "--plugin", str(plugin or host_lib)] + list(args)
    r = subprocess.run(cmd, env=_env(**envkw), capture_output=True, text=True, timeout=timeout)
    return r


def test_api_loopback_with_bounded_socket_buffers(host_lib):
    """SOCKET_SNDBUF / SOCKET_RCVBUF on the data sockets: byte-exact transfers go on, also with a value that
    is raised because it would stall a loopback stream."""
    for snd, rcv in (("262144", "0"), ("4096", "1048576")):
        r = _loopback(host_lib, ["--sizes", "1000,300000,8388608", "--inflight", "8", "--iters", "2"],
                      NCCL_GPUDIRECTTCPX_SOCKET_SNDBUF=snd, NCCL_GPUDIRECTTCPX_SOCKET_RCVBUF=rcv)
        assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
        assert "loopback PASSED" in r.stdout
        assert ("too small to keep a stream moving" in r.stdout + r.stderr) == (snd == "4096")


def test_unit_tests_binary(host_lib):
    r = subprocess.run([str(LIB / "tcpxb_unit_tests")], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "0 failure(s)" in r.stdout
    assert len(re.findall(r"^ok ", r.stdout, flags=re.M)) >= 16


def _parse(stdout):
    rows = [json.loads(l) for l in stdout.splitlines() if l.startswith('{"tool": "loopback",')]
    flows = [l.split() for l in stdout.splitlines() if l.startswith("FLOW ")]
    return rows, flows


def test_api_loopback_byte_exact_with_flow_stats(host_lib):
    """2 processes, host buffers, 4 sockets per comm on 2 loopback NICs, 8 in flight,
    1 KB / 64 KB / 4 MB / 64 MB, byte-exact, per-flow byte counters add up."""
    sizes = [1024, 65536, 4 << 20, 64 << 20]
    iters = 2
    r = _loopback(host_lib, ["--sizes", ",".join(map(str, sizes)), "--inflight", "8", "--iters", str(iters)])
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "loopback PASSED" in r.stdout
    rows, flows = _parse(r.stdout)
    assert [row["size"] for row in rows] == sizes and all(row["byte_exact"] for row in rows)
    assert all(row["comms"] == 2 and row["inflight"] == 8 for row in rows)
    total = sum(sizes) * 8 * iters  # per comm
    for side in ("send", "recv"):
        for comm in ("0", "1"):
            mine = [f for f in flows if f[1] == side and f[3] == comm]
            assert len(mine) == 4, "4 data sockets per comm"
            posted = sum(int(f[f.index("bytes_posted") + 1]) for f in mine)
            done = sum(int(f[f.index("bytes_done") + 1]) for f in mine)
            assert posted == total and done == total
            assert sum(1 for f in mine if int(f[f.index("bytes_done") + 1]) > 0) >= 2, "traffic is striped"
    assert len(re.findall(r"^per_flow_stats\[\d+:127\.0\.0\.[12]<\d+>->127\.0\.0\.[12]<\d+> (tx|rx)\] = ", r.stdout, flags=re.M)) == 16


@pytest.mark.parametrize("variant", [
    dict(args=["--v7"]),
    dict(args=["--random-sizes"]),                                   # receives posted larger than what arrives
    dict(args=["--random-sizes"], NCCL_INLINE_THRESHOLD=2048),
    dict(NCCL_GPUDIRECTTCPX_SCHED_ALG="KATY"),
    dict(NCCL_INLINE_THRESHOLD=2048),
    dict(NCCL_GPUDIRECTTCPX_RECV_SYNC=1),
    dict(NCCL_MIN_ZCOPY_SIZE=16384),
    dict(NCCL_DYNAMIC_CHUNK_SIZE=4096, NCCL_THREAD_SPIN_ENABLE=1),
    dict(NCCL_SOCKET_NTHREADS=1, NCCL_NSOCKS_PERTHREAD=1, NCCL_GPUDIRECTTCPX_FORCE_ACK=1),
    dict(NCCL_SOCKET_NTHREADS=8, NCCL_NSOCKS_PERTHREAD=1, NCCL_GPUDIRECTTCPX_SLOWNESS_SWITCH="ALL"),
    dict(NCCL_GPUDIRECTTCPX_CTRL_DEV="lo"),                          # control sockets on a named interface
    dict(NCCL_GPUDIRECTTCPX_TX_BINDINGS="lo#0:0-1;lo#1:0-1", NCCL_GPUDIRECTTCPX_RX_BINDINGS="lo#0:0-1;lo#1:0-1",
         NCCL_GPUDIRECTTCPX_WORKER_PIN_THREADS=1, NCCL_GPUDIRECTTCPX_REPORT_LIFECYCLE=1),
    dict(NCCL_GPUDIRECTTCPX_SPINWAIT_CONNECT=0),
    dict(args=["--comms-per-dev", "8", "--random-sizes"], NCCL_SOCKET_NTHREADS=2, NCCL_NSOCKS_PERTHREAD=1),  # 16 connections, as NCCL's channels
])
def test_api_loopback_variants(host_lib, variant):
    variant = dict(variant)
    args = variant.pop("args", []) + ["--sizes", "0,1,1000,2048,2049,300000,3000001", "--inflight", "8", "--iters", "2"]
    r = _loopback(host_lib, args, **variant)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "loopback PASSED" in r.stdout


def _has_v6_loopback():
    try:
        return any(l.split()[-1] == "lo" for l in open("/proc/net/if_inet6"))
    except OSError:
        return False


@pytest.mark.skipif(not _has_v6_loopback(), reason="no IPv6 loopback address on this machine")
def test_api_loopback_over_ipv6(host_lib):
    r = _loopback(host_lib, ["--sizes", "0,1000,300000,4194304", "--iters", "2"], NCCL_GPUDIRECTTCPX_SOCKET_FAMILY="AF_INET6",
                  NCCL_DEBUG="INFO")
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "loopback PASSED" in r.stdout
    assert "connected to ::1<" in r.stdout + r.stderr


@pytest.mark.skipif(len(os.sched_getaffinity(0)) < 2 or 0 not in os.sched_getaffinity(0) or 1 not in os.sched_getaffinity(0),
                    reason="needs cores 0 and 1")
def test_core_bindings_pin_the_helper_threads(host_lib):
    """TX/RX_BINDINGS restrict the helper threads to the listed cores; WORKER_PIN_THREADS gives each one core."""
    r = _loopback(host_lib, ["--sizes", "1000000", "--iters", "2", "--thread-times"], NCCL_GPUDIRECTTCPX_VIRTUAL_NICS=1,
                  NCCL_GPUDIRECTTCPX_TX_BINDINGS="lo:0-1", NCCL_GPUDIRECTTCPX_RX_BINDINGS="lo:1")
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    rows = [l.split() for l in r.stdout.splitlines() if l.startswith("THREAD ")]
    tx = [w for w in rows if w[2].startswith("tcpxb-tx")]
    rx = [w for w in rows if w[2].startswith("tcpxb-rx")]
    assert len(tx) == 2 and len(rx) == 2  # NCCL_SOCKET_NTHREADS=2 in this file's environment
    assert all(w[-1] == "0-1" for w in tx) and all(w[-1] == "1" for w in rx)
    r = _loopback(host_lib, ["--sizes", "1000000", "--iters", "2", "--thread-times"], NCCL_GPUDIRECTTCPX_VIRTUAL_NICS=1,
                  NCCL_GPUDIRECTTCPX_TX_BINDINGS="lo:0-1", NCCL_GPUDIRECTTCPX_WORKER_PIN_THREADS=1)
    assert r.returncode == 0
    tx = [l.split() for l in r.stdout.splitlines() if l.startswith("THREAD send tcpxb-tx")]
    assert sorted(w[-1] for w in tx) == ["0", "1"]


def _props(stdout):
    rows = []
    for l in stdout.splitlines():
        if l.startswith("PROPS "):
            w = l.split()[1:]
            rows.append(dict(zip(w[0::2], w[1::2])))
    return rows


@pytest.mark.parametrize("which", ["shared_device_allocation", "stream_counter", "memory_handles"])
def test_unit_tests_that_need_the_standin_device(host_lib, which):
    """Driver-API services (shareable allocation by file descriptor, dma-buf export, context guard, memory
    handles between processes) and the stream-ordered host counter, on the host-only library's stand-in device."""
    r = subprocess.run([str(LIB / "tcpxb_unit_tests"), which], capture_output=True, text=True, timeout=120,
                       env=dict(os.environ, TCPXB_FAKE_GPU="1"))
    assert r.returncode == 0, r.stdout + r.stderr
    assert f"ok {which}" in r.stdout and "skipped" not in r.stdout and "1 test(s), 0 failure(s)" in r.stdout


def test_device_properties_as_nccl_sees_them(host_lib):
    """Values of getProperties through both table versions (reference: src/net_tcpx.cc:705-744):
    host pointers only by default, 65536 comms, one receive per irecv, 10000 Mb/s when sysfs has no speed;
    CUDA pointers and the unpack device type (version 7) in unpack mode; regMrDmaBuf stays null."""
    r = _loopback(host_lib, ["--sizes", "1000", "--iters", "1"])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    p = _props(r.stdout)
    assert [d["name"] for d in p] == ["lo#0", "lo#1"] and [d["guid"] for d in p] == ["0", "1"]
    for d in p:
        assert d["ptr"] == "1" and d["maxComms"] == "65536" and d["maxRecvs"] == "1" and d["speed"] == "10000"
        assert d["devType"] == "0" and d["latency"] == "0.0" and d["port"] == "0" and d["regIsGlobal"] == "0"
    assert "TABLE regMrDmaBuf null" in r.stdout
    r = _loopback(host_lib, ["--v7", "--ptr", "cuda", "--sizes", "1000", "--iters", "1"], TCPXB_FAKE_GPU=1,
                  NCCL_GPUDIRECTTCPX_RECV_MODE="unpack", NCCL_GPUDIRECTTCPX_NIC_SPEED_MBPS=200000)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    for d in _props(r.stdout):
        assert d["ptr"] == "3" and d["devType"] == "1" and d["devVersion"] == "7" and d["speed"] == "200000"


@pytest.mark.parametrize("proto,algo", [("", ""), ("LL128", "Ring"), ("Simple", "Tree"), ("Simple", "")])
def test_unpack_mode_is_not_offered_without_simple_ring(host_lib, proto, algo):
    """Only NCCL's Simple-protocol ring primitives run the unpack consumer.  Asked for unpack mode under any
    other setting, the plugin warns once and behaves as in host mode (no unpack device type, host pointers),
    so that results stay correct (reference: src/net_tcpx.cc:739-740 always advertises the unpack type)."""
    r = _loopback(host_lib, ["--sizes", "1000,300000", "--iters", "1"], TCPXB_FAKE_GPU=1,
                  NCCL_GPUDIRECTTCPX_RECV_MODE="unpack", NCCL_PROTO=proto, NCCL_ALGO=algo)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    for d in _props(r.stdout):
        assert d["devType"] == "0" and d["ptr"] == "1"
    assert "needs NCCL_PROTO=Simple and NCCL_ALGO=Ring" in r.stdout + r.stderr


@pytest.mark.parametrize("threads,per,want", [(16, 3, "8 sockets, 8 threads"), (3, 4, "6 sockets, 3 threads"), (20, 3, "8 sockets, 4 threads"),
                                              (0, 0, "1 sockets, 1 threads"), (-2, -2, "4 sockets, 4 threads")])
def test_socket_and_thread_counts_are_clamped(host_lib, threads, per, want):
    """At most 8 sockets and 16 helper threads per connection (reference: src/macro.h:36-37); the automatic
    choice for an interface without a PCI device (loopback, veth) is 4 x 1."""
    r = _loopback(host_lib, ["--sizes", "300000", "--iters", "1"], NCCL_SOCKET_NTHREADS=threads, NCCL_NSOCKS_PERTHREAD=per,
                  NCCL_DEBUG="INFO", NCCL_GPUDIRECTTCPX_VIRTUAL_NICS=1)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert f"connected to 127.0.0.1<" in r.stdout + r.stderr and want in r.stdout + r.stderr


def test_plugin_disabled_by_env(host_lib):
    r = _loopback(host_lib, ["--sizes", "1024", "--iters", "1"], NCCL_GPUDIRECTTCPX_SOCKET_ENABLE=0)
    assert r.returncode != 0  # init fails so that NCCL would fall back


def test_telemetry_files(host_lib, tmp_path):
    r = _loopback(host_lib, ["--sizes", "65536,1000000", "--iters", "2"],
                  NCCL_GPUDIRECTTCPX_TELEMETRY_EXPORT_STATS_TO_FILE=1,
                  NCCL_GPUDIRECTTCPX_TELEMETRY_ENABLE_TASK_LEVEL_STATS=1,
                  NCCL_GPUDIRECTTCPX_TELEMETRY_ENABLE_REQUEST_LEVEL_STATS=1,
                  NCCL_GPUDIRECTTCPX_TELEMETRY_EXPORTER_PATH=str(tmp_path),
                  NCCL_GPUDIRECTTCPX_LOG_STATS_TO_STDOUT=1)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    logs = sorted(tmp_path.glob("exporter_[0-9]*_*.log"))
    stats = sorted(tmp_path.glob("exporter_stats_*_*.log"))
    assert len(logs) == 4 and len(stats) == 4  # 2 comms on each side
    text = logs[0].read_text().splitlines()
    assert text and all(re.match(r"^[TR] 0x[0-9a-f]+ [01] [A-Z]+ \d{19}$", l) for l in text)
    states = {l.split()[3] for l in text}
    assert {"ACTIVE", "COMPLETING", "INACTIVE", "POSTED", "TRANSMITTING"} <= states
    assert all(l.startswith("per_flow_stats[") for l in stats[0].read_text().splitlines())
    # the offline reader turns the lines into time spent per state; every life is whole
    from nccl_plugin_gpudirecttcpx_b200.utils.trace import summarize
    rows = summarize([str(p) for p in logs])
    steps = {(r["kind"], r["side"], r["from"], r["to"]): r for r in rows}
    for side in ("send", "recv"):
        for a, b in (("POSTED", "ACTIVE"), ("ACTIVE", "TRANSMITTING"), ("TRANSMITTING", "INACTIVE"), ("INACTIVE", "FREE")):
            assert steps[("request", side, a, b)]["count"] == 2 * 2 * 8 * 2  # sizes x iterations x in flight x comms
        for a, b in (("ACTIVE", "COMPLETING"), ("COMPLETING", "INACTIVE"), ("INACTIVE", "FREE")):
            assert steps[("task", side, a, b)]["count"] > 0
    assert len(rows) == 14 and all(r["p50_us"] <= r["p99_us"] <= r["max_us"] for r in rows)


@pytest.mark.parametrize("san", ["address", "thread", "undefined"])
def test_loopback_under_sanitizer(san):
    lib = _build.build_host(sanitize=san)
    env = {"ASAN_OPTIONS": "detect_leaks=1", "TSAN_OPTIONS": "halt_on_error=1 second_deadlock_stack=1"}
    r = _loopback(lib, ["--sizes", "0,1000,65536,2000000", "--inflight", "8", "--iters", "2"],
                  exe=f"tcpxb_loopback_{san}", timeout=600, **env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-6000:]
    assert "loopback PASSED" in r.stdout
    assert "WARNING: ThreadSanitizer" not in r.stderr and "ERROR: AddressSanitizer" not in r.stderr
    assert "runtime error:" not in r.stderr


STANDIN_VARIANTS = [
    # plugin-side unpack: staging ring on the sender, page pool + scatter list + host unpack on the receiver
    dict(NCCL_GPUDIRECTTCPX_CUDA_BUFFERS=1),
    dict(NCCL_GPUDIRECTTCPX_CUDA_BUFFERS=1, NCCL_GPUDIRECTTCPX_RX_POOL_SCATTER=1, NCCL_GPUDIRECTTCPX_RX_POOL_BYTES=32 << 20),
    dict(NCCL_GPUDIRECTTCPX_CUDA_BUFFERS=1, NCCL_GPUDIRECTTCPX_RX_POOL_MODE="device"),
    # consumer-side unpack: the tool plays NCCL's unpack kernel against the device handle
    dict(NCCL_GPUDIRECTTCPX_RECV_MODE="unpack"),
    dict(NCCL_GPUDIRECTTCPX_RECV_MODE="unpack", NCCL_GPUDIRECTTCPX_RX_POOL_SCATTER=1, NCCL_GPUDIRECTTCPX_RX_POOL_BYTES=32 << 20),
    dict(NCCL_GPUDIRECTTCPX_RECV_MODE="unpack", NCCL_GPUDIRECTTCPX_RX_POOL_MODE="device", args=["--v7"]),
    dict(NCCL_GPUDIRECTTCPX_RECV_MODE="unpack", args=["--random-sizes"]),
    dict(NCCL_GPUDIRECTTCPX_CUDA_BUFFERS=1, NCCL_INLINE_THRESHOLD=2048, args=["--random-sizes"]),
    # 16 connections share a 16 MiB pool: at most four of the largest messages fit at a time
    dict(NCCL_GPUDIRECTTCPX_RECV_MODE="unpack", NCCL_GPUDIRECTTCPX_RX_POOL_BYTES=16 << 20, NCCL_SOCKET_NTHREADS=2,
         NCCL_NSOCKS_PERTHREAD=1, args=["--comms-per-dev", "8", "--random-sizes"]),
    # two connections share a pool that holds exactly one of the largest messages: whoever gets the
    # pool's promise goes first, nobody waits while holding pages
    dict(NCCL_GPUDIRECTTCPX_RECV_MODE="unpack", NCCL_GPUDIRECTTCPX_RX_POOL_BYTES=8 << 20),
    dict(NCCL_GPUDIRECTTCPX_CUDA_BUFFERS=1, NCCL_GPUDIRECTTCPX_RX_POOL_BYTES=8 << 20, NCCL_GPUDIRECTTCPX_TX_STAGING_BYTES=8 << 20),
]


@pytest.mark.parametrize("variant", STANDIN_VARIANTS)
def test_device_pointer_paths_on_standin_device(host_lib, variant):
    """The paths that take CUDA pointers, run on the host-only build's stand-in device
    (device memory = host memory): staged sends, page pool, scatter lists, the unpack
    device-handle protocol {meta, bounce_buf, head} and irecvConsumed, byte-exact."""
    variant = dict(variant)
    args = variant.pop("args", []) + ["--ptr", "cuda", "--sizes", "0,1,1000,4097,300000,4194304,8388608", "--inflight", "8", "--iters", "2"]
    r = _loopback(host_lib, args, TCPXB_FAKE_GPU=1, **variant)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "loopback PASSED" in r.stdout
    rows, _ = _parse(r.stdout)
    assert len(rows) == 7 and all(row["byte_exact"] for row in rows)


def test_standin_device_oversize_receive_is_an_error(host_lib):
    """A device-memory receive that needs more page records than a scatter-list slot holds
    fails with an error from test(), and the tool ends instead of hanging."""
    r = _loopback(host_lib, ["--ptr", "cuda", "--sizes", str(16 << 20), "--inflight", "1", "--iters", "1"], timeout=120,
                  TCPXB_FAKE_GPU=1, NCCL_GPUDIRECTTCPX_CUDA_BUFFERS=1)
    assert r.returncode != 0
    assert "page records of a scatter-list slot" in r.stderr


def test_standin_device_pool_smaller_than_a_message_is_an_error(host_lib):
    r = _loopback(host_lib, ["--ptr", "cuda", "--sizes", str(4 << 20), "--inflight", "2", "--iters", "1"], timeout=120,
                  TCPXB_FAKE_GPU=1, NCCL_GPUDIRECTTCPX_RECV_MODE="unpack", NCCL_GPUDIRECTTCPX_RX_POOL_BYTES=1 << 20)
    assert r.returncode != 0
    assert "rx pages but the pool has" in r.stderr


def test_host_build_rejects_device_pointers_without_standin(host_lib):
    r = _loopback(host_lib, ["--ptr", "cuda", "--sizes", "1024", "--iters", "1"], timeout=120, NCCL_GPUDIRECTTCPX_CUDA_BUFFERS=1)
    assert r.returncode != 0
    assert "is not device memory" in r.stderr


@pytest.mark.parametrize("san", ["address", "thread"])
@pytest.mark.parametrize("mode", ["host", "unpack"])
def test_standin_device_under_sanitizer(san, mode):
    lib = _build.build_host(sanitize=san)
    env = {"ASAN_OPTIONS": "detect_leaks=1", "TSAN_OPTIONS": "halt_on_error=1 second_deadlock_stack=1", "TCPXB_FAKE_GPU": "1",
           "NCCL_GPUDIRECTTCPX_RX_POOL_SCATTER": "1", "NCCL_GPUDIRECTTCPX_RX_POOL_BYTES": str(64 << 20)}
    env.update({"NCCL_GPUDIRECTTCPX_RECV_MODE": "unpack"} if mode == "unpack" else {"NCCL_GPUDIRECTTCPX_CUDA_BUFFERS": "1"})
    r = _loopback(lib, ["--ptr", "cuda", "--sizes", "0,1000,65536,2000000", "--inflight", "8", "--iters", "2"],
                  exe=f"tcpxb_loopback_{san}", timeout=600, **env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-6000:]
    assert "loopback PASSED" in r.stdout
    assert "WARNING: ThreadSanitizer" not in r.stderr and "ERROR: AddressSanitizer" not in r.stderr
    assert "runtime error:" not in r.stderr


def test_fault_paths_surface_as_errors(host_lib):
    """Closed peer, socket shutdown in mid-message, forged control records, oversize message,
    full request ring, silent sender, a caller that polls only a younger request, and on the
    stand-in device a consumer that falls behind, frees slots out of order or holds the pool's
    pages: error codes, "try again" or back-pressure, never a hang."""
    r = subprocess.run([str(LIB / "tcpxb_fault_tests")], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "19 test(s), 0 failure(s)" in r.stdout


@pytest.mark.parametrize("san", ["address", "thread", "undefined"])
def test_unit_tests_under_sanitizer(san):
    _build.build_host(sanitize=san)
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1", TSAN_OPTIONS="halt_on_error=1 second_deadlock_stack=1")
    r = subprocess.run([str(LIB / f"tcpxb_unit_tests_{san}")], capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-6000:]
    assert "0 failure(s)" in r.stdout
    assert "WARNING: ThreadSanitizer" not in r.stderr and "ERROR: AddressSanitizer" not in r.stderr
    assert "runtime error:" not in r.stderr


@pytest.mark.parametrize("san", ["address", "thread", "undefined"])
def test_fault_paths_under_sanitizer(san):
    _build.build_host(sanitize=san)
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1", TSAN_OPTIONS="halt_on_error=1 second_deadlock_stack=1")
    r = subprocess.run([str(LIB / f"tcpxb_fault_tests_{san}")], capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-6000:]
    assert "0 failure(s)" in r.stdout
    assert "WARNING: ThreadSanitizer" not in r.stderr and "ERROR: AddressSanitizer" not in r.stderr
    assert "runtime error:" not in r.stderr


def test_rx_buffer_manager_daemon(host_lib, tmp_path):
    """The out-of-process rx buffer manager: pool fd over SCM_RIGHTS, flow rules, lifecycle registry."""
    prefix = tmp_path / "rxdm"
    daemon = subprocess.Popen([str(LIB / "tcpxb_rxdm"), "--prefix", str(prefix), "--pool-mb", "8"],
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    try:
        assert daemon.stdout.readline().strip() == "ready"
        env = dict(os.environ, TCPXB_TEST_RXDM_PREFIX=str(prefix))
        r = subprocess.run([str(LIB / "tcpxb_unit_tests"), "rxdm_daemon"], capture_output=True, text=True, timeout=60, env=env)
        assert r.returncode == 0, r.stdout + r.stderr
        assert "ok rxdm_daemon_roundtrip" in r.stdout and "skipped" not in r.stdout
    finally:
        daemon.terminate()
        try:
            daemon.wait(timeout=5)
        except subprocess.TimeoutExpired:
            daemon.kill()
    assert "application 4242 went away" in daemon.stderr.read()


@pytest.mark.parametrize("pool", ["host", "device"])
@pytest.mark.parametrize("mode", ["unpack", "host"])
def test_daemon_pool_carries_device_receives_on_standin_device(host_lib, tmp_path, mode, pool):
    """Receives into device memory land in the pool that the daemon owns and hands over as a file
    descriptor: a memfd of host memory, or (--device-pool) a shareable handle of device memory that
    the client imports and maps, with payload placed by the copy engine from a pinned mirror
    (reference: src/gpu/rx_pool.cu:62-124, src/gpu/common.cu:25-65)."""
    prefix = tmp_path / "rxdm"
    daemon = subprocess.Popen([str(LIB / "tcpxb_rxdm"), "--prefix", str(prefix), "--pool-mb", "32"] +
                              (["--device-pool"] if pool == "device" else []),
                              env=dict(os.environ, TCPXB_FAKE_GPU="1"),
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    try:
        assert daemon.stdout.readline().strip() == "ready"
        env = dict(TCPXB_FAKE_GPU=1, NCCL_GPUDIRECTTCPX_RX_BUF_MGR="daemon", NCCL_GPUDIRECTTCPX_UNIX_CLIENT_PREFIX=str(prefix))
        env.update({"NCCL_GPUDIRECTTCPX_RECV_MODE": "unpack"} if mode == "unpack" else {"NCCL_GPUDIRECTTCPX_CUDA_BUFFERS": 1})
        r = _loopback(host_lib, ["--ptr", "cuda", "--sizes", "0,1000,300000,4194304", "--inflight", "8", "--iters", "2"], **env)
        assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
        assert "loopback PASSED" in r.stdout
        # the daemon's own view afterwards: every rule withdrawn, every application gone, the pool still there
        q = subprocess.run([str(LIB / "tcpxb_rxdm"), "--status", "--prefix", str(prefix)], capture_output=True, text=True, timeout=20)
        assert q.returncode == 0, q.stderr
        st = json.loads(q.stdout)
        assert st["flow_rules"] == 0 and st["applications"] == 0 and st["pools"] == 1
    finally:
        daemon.terminate()
        try:
            daemon.wait(timeout=5)
        except subprocess.TimeoutExpired:
            daemon.kill()
    log = daemon.stderr.read()
    assert f"pool for GPU 0000:00:00.0: 32 MiB of {pool} memory" in log, log[-2000:]  # the pool came from the daemon


def test_daemon_pool_imported_by_memory_handle_on_standin_device(host_lib, tmp_path):
    """The reference's older import path (reference: src/gpu/rx_pool.cu:30-55): the daemon leaves a 64-byte
    memory handle in <prefix>/nvdma-<pci>, a plugin started with NCCL_TCPX_RXMEM_IMPORT_USE_GPU_PCI_CLIENT=0
    opens it and receives into that pool; flow rules and registration still go through the daemon's sockets."""
    prefix = tmp_path / "rxdm"
    daemon = subprocess.Popen([str(LIB / "tcpxb_rxdm"), "--prefix", str(prefix), "--pool-mb", "32", "--legacy-ipc-files"],
                              env=dict(os.environ, TCPXB_FAKE_GPU="1"), stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    try:
        assert daemon.stdout.readline().strip() == "ready", daemon.stderr.read()
        handle = prefix / "nvdma-0000:00:00.0"
        assert handle.stat().st_size == 64
        env = dict(TCPXB_FAKE_GPU=1, NCCL_GPUDIRECTTCPX_RX_BUF_MGR="daemon", NCCL_GPUDIRECTTCPX_UNIX_CLIENT_PREFIX=str(prefix),
                   NCCL_TCPX_RXMEM_IMPORT_USE_GPU_PCI_CLIENT=0, NCCL_GPUDIRECTTCPX_RECV_MODE="unpack", NCCL_DEBUG="INFO")
        r = _loopback(host_lib, ["--ptr", "cuda", "--sizes", "0,1000,300000,4194304", "--inflight", "8", "--iters", "2"], **env)
        assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
        assert "loopback PASSED" in r.stdout
        assert "32 MiB of device memory" in r.stdout + r.stderr  # the client's own log line about the imported pool
        q = subprocess.run([str(LIB / "tcpxb_rxdm"), "--status", "--prefix", str(prefix)], capture_output=True, text=True, timeout=20)
        st = json.loads(q.stdout)
        assert st["flow_rules"] == 0 and st["applications"] == 0 and st["pools"] == 0  # no descriptor was ever asked for
        # a handle file that is not a handle, and none at all
        handle.write_bytes(b"x" * 64)
        bad = _loopback(host_lib, ["--ptr", "cuda", "--sizes", "1000", "--iters", "1"], **env)
        assert bad.returncode != 0 and "opening the memory handle" in bad.stdout + bad.stderr
        handle.unlink()
        bad = _loopback(host_lib, ["--ptr", "cuda", "--sizes", "1000", "--iters", "1"], **env)
        assert bad.returncode != 0 and "no memory handle at" in bad.stdout + bad.stderr
    finally:
        daemon.terminate()
        try:
            daemon.wait(timeout=5)
        except subprocess.TimeoutExpired:
            daemon.kill()
    assert "handle in" in daemon.stderr.read()


def test_odd_gpus_without_rx_pool(host_lib):
    """NCCL_TCPX_RXMEM_IMPORT_SKIP_ODDS=1: device 0 keeps its pool, an odd device has none."""
    r = subprocess.run([str(LIB / "tcpxb_unit_tests"), "rx_pool_skip_odds"], capture_output=True, text=True, timeout=60,
                       env=dict(os.environ, TCPXB_FAKE_GPU="1"))
    assert r.returncode == 0 and "ok rx_pool_skip_odds" in r.stdout, r.stdout + r.stderr


@pytest.mark.parametrize("wire", ["native", "proto"])
@pytest.mark.parametrize("san", ["", "address"])
def test_rx_buffer_manager_daemon_survives_garbage(tmp_path, san, wire):
    """Random bytes, truncated frames and oversize lengths on every service socket: the daemon drops the
    connection and keeps serving."""
    import random
    import socket
    import struct
    prefix = tmp_path / "rxdm"
    if san:
        _build.build_host(sanitize=san)
    else:
        _build.build_host()
    daemon = subprocess.Popen([str(LIB / ("tcpxb_rxdm" + ("_" + san if san else ""))), "--prefix", str(prefix), "--pool-mb", "4",
                               "--wire", wire],
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True,
                              env=dict(os.environ, ASAN_OPTIONS="detect_leaks=0"))
    try:
        assert daemon.stdout.readline().strip() == "ready"
        rng = random.Random(7)
        per_gpu = ["get_gpu_fd", "get_gpu_metadata"] if wire == "native" else ["get_gpu_fd_host", "get_gpu_metadata_host"]
        services = ["rx_rule_manager", "rx_rule_uninstall", "rxdm_application_registry", "rxdm_status"] + per_gpu
        for name in services:
            for payload in (b"", b"\x00", struct.pack("!H", 65535) + b"x" * 100, struct.pack("!H", 8) + b"12345678",
                            bytes(rng.randrange(256) for _ in range(600)), struct.pack("!H", 300),
                            # well-framed protobuf with nested lengths that overrun, an endless varint, a huge field number
                            struct.pack("!H", 6) + bytes([0x12, 0x7f, 0x0a, 0x7f, 0x08, 0x01]),
                            struct.pack("!H", 12) + bytes([0x0a] + [0xff] * 11),
                            struct.pack("!H", 7) + bytes([0xf8, 0xff, 0xff, 0xff, 0x0f, 0x01, 0x00])):
                s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
                s.settimeout(2)
                s.connect(str(prefix / name))
                try:
                    s.sendall(payload)
                    s.shutdown(socket.SHUT_WR)
                    s.recv(4096)
                except OSError:
                    pass
                s.close()
        assert daemon.poll() is None, daemon.stderr.read()
        q = subprocess.run([str(LIB / "tcpxb_rxdm"), "--status", "--prefix", str(prefix)], capture_output=True, text=True, timeout=20)
        assert q.returncode == 0, q.stderr
        assert json.loads(q.stdout)["flow_rules"] == 0
        # and a well-formed registration afterwards, so that the keep-alive bookkeeping runs under the sanitizer too:
        # two applications register in one poll round, one leaves
        regs = []
        for _ in range(2):
            s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            s.settimeout(2)
            s.connect(str(prefix / "rxdm_application_registry"))
            if wire == "proto":
                body = bytes([0x32, 0x02, 0x08, 0x01])  # ApplicationRegisterRequest{register_client: true}
            else:
                body = struct.pack("<IHHii", 0x4d445852, 5, 0, 1, 4242).ljust(144, b"\0")
            s.sendall(struct.pack("!H", len(body)) + body)
            regs.append(s)
        for s in regs:
            assert len(s.recv(4096)) > 2
        q = subprocess.run([str(LIB / "tcpxb_rxdm"), "--status", "--prefix", str(prefix)], capture_output=True, text=True, timeout=20)
        assert json.loads(q.stdout)["applications"] == 2
        regs[0].close()
        for _ in range(50):
            q = subprocess.run([str(LIB / "tcpxb_rxdm"), "--status", "--prefix", str(prefix)], capture_output=True, text=True, timeout=20)
            if json.loads(q.stdout)["applications"] == 1:
                break
        assert json.loads(q.stdout)["applications"] == 1
        regs[1].close()
    finally:
        daemon.terminate()
        try:
            daemon.wait(timeout=5)
        except subprocess.TimeoutExpired:
            daemon.kill()
    assert "ERROR: AddressSanitizer" not in daemon.stderr.read()
