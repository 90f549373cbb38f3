"""CPU tests of the Python helpers: flag listing, NCCL environment builder, clocks sampler."""
import os

from nccl_plugin_gpudirecttcpx_b200 import _build


def test_flag_docs_cover_the_reference_surface():
    _build.build_host()
    from nccl_plugin_gpudirecttcpx_b200.utils.flags import flag_docs
    names = {r[0] for r in flag_docs()}
    for env in ("NCCL_GPUDIRECTTCPX_SOCKET_ENABLE", "NCCL_MIN_ZCOPY_SIZE", "NCCL_NSOCKS_PERTHREAD", "NCCL_SOCKET_NTHREADS",
                "NCCL_INLINE_THRESHOLD", "NCCL_DYNAMIC_CHUNK_SIZE", "NCCL_THREAD_SPIN_ENABLE", "NCCL_USE_DMA_BUF",
                "NCCL_GPUDIRECTTCPX_CONNECTION_RETRY", "NCCL_GPUDIRECTTCPX_RECV_SYNC", "NCCL_GPUDIRECTTCPX_FORCE_ACK",
                "NCCL_GPUDIRECTTCPX_TX_COMPLETION_NANOSLEEP", "NCCL_GPUDIRECTTCPX_TIMEOUT_THRESHOLD_NS",
                "NCCL_GPUDIRECTTCPX_TIMEOUT_FREQUENCY_NS", "NCCL_GPUDIRECTTCPX_SPINWAIT_CONNECT",
                "NCCL_GPUDIRECTTCPX_LOG_STATS_TO_STDOUT", "NCCL_GPUDIRECTTCPX_TELEMETRY_ENABLE_TASK_LEVEL_STATS",
                "NCCL_GPUDIRECTTCPX_TELEMETRY_EXPORTER_PATH", "NCCL_GPUDIRECTTCPX_REPORT_LIFECYCLE",
                "NCCL_GPUDIRECTTCPX_CUDA_USE_PRIMARY_CTX", "NCCL_GPUDIRECTTCPX_NIC_N_RXQS",
                "NCCL_GPUDIRECTTCPX_FLOW_STEERING_STRATEGY", "NCCL_GPUDIRECTTCPX_PROGRAM_FLOW_STEERING_WAIT_MICROS",
                "NCCL_TCPX_RXMEM_IMPORT_USE_GPU_PCI_CLIENT", "NCCL_GPUDIRECTTCPX_SOCKET_IFNAME",
                "NCCL_GPUDIRECTTCPX_SOCKET_FAMILY", "NCCL_GPUDIRECTTCPX_CTRL_DEV", "NCCL_GPUDIRECTTCPX_PORT_MAPPING",
                "NCCL_GPUDIRECTTCPX_TX_BINDINGS", "NCCL_GPUDIRECTTCPX_RX_IRQ_BINDINGS", "NCCL_GPUDIRECTTCPX_WORKER_PIN_THREADS",
                "NCCL_GPUDIRECTTCPX_SCHED_ALG", "NCCL_GPUDIRECTTCPX_SLOWNESS_SWITCH", "NCCL_GPUDIRECTTCPX_UNIX_CLIENT_PREFIX",
                "NET_COMM_ID", "NCCL_GPUDIRECTTCPX_RECV_MODE", "NCCL_GPUDIRECTTCPX_VIRTUAL_NICS"):
        assert env in names, env
    by_name = {r[0]: r for r in flag_docs()}
    assert by_name["NCCL_DYNAMIC_CHUNK_SIZE"][2] == "131072"   # the documented default, not 0
    assert by_name["NCCL_GPUDIRECTTCPX_TIMEOUT_THRESHOLD_NS"][2] == "10000000000"


def test_plugin_env_variants(monkeypatch):
    from nccl_plugin_gpudirecttcpx_b200.parallel import plugin_env
    from nccl_plugin_gpudirecttcpx_b200.utils import native
    monkeypatch.setattr(native, "load", lambda name, build=True: None)
    base = plugin_env(nics=3, nthreads=2, nsocks_per_thread=2, chunk_bytes=65536)
    assert base["NCCL_GPUDIRECTTCPX_VIRTUAL_NICS"] == "3" and base["NCCL_SOCKET_NTHREADS"] == "2"
    assert base["NCCL_NSOCKS_PERTHREAD"] == "2" and base["NCCL_DYNAMIC_CHUNK_SIZE"] == "65536"
    assert base["NCCL_NET_PLUGIN"].endswith("libnccl-net.so") and base["NCCL_P2P_DISABLE"] == "1"
    assert "NCCL_NET_GDR_LEVEL" not in base and "NCCL_GPUDIRECTTCPX_CUDA_BUFFERS" not in base  # host buffers by default
    unpack = plugin_env(recv_mode="unpack")
    assert unpack["NCCL_PROTO"] == "Simple" and unpack["NCCL_ALGO"] == "Ring" and unpack["NCCL_NET_GDR_READ"] == "0"
    assert unpack["NCCL_GPUDIRECTTCPX_RECV_MODE"] == "unpack"
    sock = plugin_env(builtin_socket=True, nthreads=2)
    assert sock["NCCL_NET"] == "Socket" and sock["NCCL_NET_PLUGIN"] == "none" and sock["NCCL_SOCKET_NTHREADS"] == "2"
    assert not any(k.startswith("NCCL_GPUDIRECTTCPX_") for k in sock)


def test_socket_settings_follow_the_cores_per_rank(monkeypatch):
    import importlib
    pe = importlib.import_module("nccl_plugin_gpudirecttcpx_b200.parallel.plugin_env")  # the package re-exports the function
    assert pe.socket_settings_for(32, 8) == {"nthreads": 2, "chunk_bytes": 128 * 1024}   # 4 cores per rank
    assert pe.socket_settings_for(24, 4) == {"nthreads": 4, "chunk_bytes": 512 * 1024}   # 6 cores per rank
    assert pe.socket_settings_for(2, 8)["nthreads"] == 2
    monkeypatch.setattr(os, "sched_getaffinity", lambda pid: set(range(32)))
    monkeypatch.setenv("LOCAL_WORLD_SIZE", "8")
    env = pe.plugin_env(nthreads=0, chunk_bytes=0, builtin_socket=True)
    assert env["NCCL_SOCKET_NTHREADS"] == "2" and env["NCCL_DYNAMIC_CHUNK_SIZE"] == str(128 * 1024)
    env = pe.plugin_env(nthreads=3, chunk_bytes=0, builtin_socket=True)
    assert env["NCCL_SOCKET_NTHREADS"] == "3" and env["NCCL_DYNAMIC_CHUNK_SIZE"] == str(128 * 1024)
    # four cores per rank: four NCCL channels, for the plugin and for the baseline alike; the caller's own setting wins
    monkeypatch.delenv("NCCL_MAX_NCHANNELS", raising=False)
    assert env["NCCL_MAX_NCHANNELS"] == "4" and env["NCCL_MIN_NCHANNELS"] == "4"
    monkeypatch.setattr(native_mod(), "load", lambda name, build=True: None)
    plug = pe.plugin_env(nthreads=2)
    assert plug["NCCL_MAX_NCHANNELS"] == "4" and plug["NCCL_GPUDIRECTTCPX_SOCKET_SNDBUF"] == str(256 * 1024)
    assert pe.plugin_env(nthreads=2, sndbuf=0, max_channels=0).get("NCCL_MAX_NCHANNELS") is None
    monkeypatch.setenv("LOCAL_WORLD_SIZE", "2")  # sixteen cores per rank: NCCL's own choice, the kernel's buffer tuning
    roomy = pe.plugin_env(nthreads=2)
    assert "NCCL_MAX_NCHANNELS" not in roomy and roomy["NCCL_GPUDIRECTTCPX_SOCKET_SNDBUF"] == "0"
    assert pe.loopback_sndbuf(4) == 256 * 1024 and pe.loopback_sndbuf(8) == 256 * 1024 and pe.loopback_sndbuf(16) == 0
    monkeypatch.setenv("LOCAL_WORLD_SIZE", "8")
    monkeypatch.setenv("NCCL_MAX_NCHANNELS", "12")
    assert "NCCL_MAX_NCHANNELS" not in pe.plugin_env(nthreads=2)


def native_mod():
    from nccl_plugin_gpudirecttcpx_b200.utils import native
    return native


def test_clock_sampler_without_nvidia_smi(monkeypatch):
    import shutil
    from nccl_plugin_gpudirecttcpx_b200.utils import clocks
    monkeypatch.setattr(shutil, "which", lambda name: None)
    s = clocks.ClockSampler(0).start()
    summary = s.stop()
    assert summary["samples"] == 0 and summary["reasons"] == [] and summary["sm_mhz"] is None
    # and the parser on canned lines
    s.samples = [["0", "1965", "1965", "700.1", "Not Active", "Not Active", "Not Active", "Active"],
                 ["0", "1800", "1965", "990.0", "Not Active", "Not Active", "Not Active", "Not Active"]]
    out = s.summary()
    assert out["sm_mhz"] == 1882.5 and out["sm_max_mhz"] == 1965 and out["reasons"] == ["sw_power_cap"]


def test_environment_doc_matches_the_flag_registry():
    """docs/environment.md carries the table the native registry generates."""
    from pathlib import Path
    from nccl_plugin_gpudirecttcpx_b200.utils.flags import markdown_table
    text = (Path(__file__).resolve().parent.parent / "docs" / "environment.md").read_text()
    table = text.split("<!-- table:begin -->\n")[1].split("<!-- table:end -->")[0]
    assert table == markdown_table()


def test_clock_sampler_against_a_fake_nvidia_smi(tmp_path, monkeypatch):
    """The sampler only ever runs a read-only query, and digests what the tool prints."""
    import os
    import stat
    import time
    from nccl_plugin_gpudirecttcpx_b200.utils import clocks
    fake = tmp_path / "nvidia-smi"
    fake.write_text(
        "#!/bin/sh\n"
        f"echo \"$@\" > {tmp_path}/argv\n"
        "i=0\n"
        "while true; do\n"
        "  if [ $i -lt 2 ]; then echo '3, 1965, 1965, 640.00, Not Active, Not Active, Not Active, Not Active';\n"
        "  else echo '3, 1410, 1965, 999.10, Not Active, Not Active, Not Active, Active'; fi\n"
        "  i=$((i+1)); sleep 0.05\n"
        "done\n")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", f"{tmp_path}:{os.environ['PATH']}")
    s = clocks.ClockSampler(3, period_ms=50).start()
    time.sleep(0.5)
    out = s.stop()
    argv = (tmp_path / "argv").read_text().split()
    assert "--id=3" in argv and any(a.startswith("--query-gpu=") for a in argv) and "-lms" in argv
    assert not any(a in ("-lgc", "-rgc", "-ac", "-rac", "-pm", "-pl", "-r", "--gpu-reset", "-c", "-e", "-mig") for a in argv)
    assert out["samples"] >= 4 and out["sm_max_mhz"] == 1965 and out["sm_mhz"] == 1410 and out["reasons"] == ["sw_power_cap"]


def test_bench_rails_and_threads_follow_the_cores():
    import sys
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    import bench
    assert bench.rails_and_threads(16, 1) == (4, 2)     # the one-GPU box
    assert bench.rails_and_threads(24, 2) == (4, 1)
    assert bench.rails_and_threads(32, 4) == (4, 1)
    assert bench.rails_and_threads(32, 8) == (4, 1)     # 4 cores per rank: helpers sleep when idle, 4 rails still win
    assert bench.rails_and_threads(2, 8) == (1, 1)
    assert bench.rails_and_threads(32, 8, nics=2) == (2, 1) and bench.rails_and_threads(32, 8, nthreads=3) == (4, 3)
