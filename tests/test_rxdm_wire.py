"""The receive-datapath manager protocol in the reference's wire format (RXDM_WIRE=proto).

The hand-written codec in csrc/core/rxdm_proto.cc is checked against the protobuf library
itself: the schema below restates the reference's messages (reference:
src/rx_buf_mgr_client/proto/unix_socket_proto.proto:17-70, unix_socket_message.proto) as a
descriptor built at run time, a client made of that library talks to this repository's daemon,
and this repository's client talks to a daemon made of that library.
"""
import json
import os
import socket
import struct
import subprocess
import threading
from pathlib import Path

import pytest

from nccl_plugin_gpudirecttcpx_b200 import _build

LIB = Path(_build.OUT)


@pytest.fixture(scope="module")
def host_lib():
    _build.build_host()
    return LIB / "libtcpxb_host.so"


@pytest.fixture(scope="module")
def pb():
    """Message classes for UnixSocketProto and its parts, from a descriptor built here."""
    from google.protobuf import descriptor_pb2, descriptor_pool, message_factory

    F = descriptor_pb2.FieldDescriptorProto
    f = descriptor_pb2.FileDescriptorProto(name="rxdm_wire_test.proto", package="rxdm_wire_test", syntax="proto2")

    def msg(name, fields, oneof=None):
        m = f.message_type.add(name=name)
        if oneof:
            m.oneof_decl.add(name=oneof)
        for fname, number, ftype, extra in fields:
            fd = m.field.add(name=fname, number=number, type=ftype, label=extra.get("label", F.LABEL_OPTIONAL))
            if "type_name" in extra:
                fd.type_name = ".rxdm_wire_test." + extra["type_name"]
            if oneof and extra.get("in_oneof", True):
                fd.oneof_index = 0
        return m

    msg("SocketAddress", [("ip_address", 1, F.TYPE_STRING, {}), ("port", 2, F.TYPE_INT32, {})])
    msg("FlowSteerNtupleProto", [("flow_type", 1, F.TYPE_INT32, {}),
                                 ("src", 2, F.TYPE_MESSAGE, {"type_name": "SocketAddress"}),
                                 ("dst", 3, F.TYPE_MESSAGE, {"type_name": "SocketAddress"})])
    msg("FlowSteerRuleRequest", [("flow_steer_ntuple", 1, F.TYPE_MESSAGE, {"type_name": "FlowSteerNtupleProto"}),
                                 ("queue_id", 2, F.TYPE_INT32, {}), ("gpu_pci_addr", 3, F.TYPE_STRING, {})])
    msg("QueueIdQuery", [("gpu_pci_addr", 1, F.TYPE_STRING, {})])
    msg("QueueIdResponse", [("queue_ids", 1, F.TYPE_INT32, {"label": F.LABEL_REPEATED})])
    msg("ApplicationRegisterRequest", [("register_client", 1, F.TYPE_BOOL, {})])
    msg("UnixSocketProto", [("raw_bytes", 1, F.TYPE_BYTES, {}),
                            ("flow_steer_rule_request", 2, F.TYPE_MESSAGE, {"type_name": "FlowSteerRuleRequest"}),
                            ("queue_id_query", 3, F.TYPE_MESSAGE, {"type_name": "QueueIdQuery"}),
                            ("queue_id_response", 4, F.TYPE_MESSAGE, {"type_name": "QueueIdResponse"}),
                            ("application_register_request", 6, F.TYPE_MESSAGE, {"type_name": "ApplicationRegisterRequest"})],
        oneof="payload")
    pool = descriptor_pool.DescriptorPool()
    pool.Add(f)
    return {d.name: message_factory.GetMessageClass(pool.FindMessageTypeByName("rxdm_wire_test." + d.name)) for d in f.message_type}


def frame(body: bytes) -> bytes:
    return struct.pack("!H", len(body)) + body


def read_exact(s, n):
    buf = b""
    while len(buf) < n:
        chunk = s.recv(n - len(buf))
        if not chunk:
            raise EOFError
        buf += chunk
    return buf


def read_frame(s) -> bytes:
    (n,) = struct.unpack("!H", read_exact(s, 2))
    return read_exact(s, n) if n else b""


def call(prefix, service, body: bytes):
    """One request on a fresh connection; the connection comes back open for the reply."""
    s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    s.settimeout(5)
    s.connect(str(prefix / service))
    s.sendall(frame(body))
    return s


def start_daemon(prefix, *extra, env=None):
    d = subprocess.Popen([str(LIB / "tcpxb_rxdm"), "--prefix", str(prefix), "--wire", "proto", *extra],
                         stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env)
    assert d.stdout.readline().strip() == "ready", d.stderr.read()
    return d


def stop_daemon(d):
    d.terminate()
    try:
        d.wait(timeout=5)
    except subprocess.TimeoutExpired:
        d.kill()
    return d.stderr.read()


def daemon_status(prefix):
    q = subprocess.run([str(LIB / "tcpxb_rxdm"), "--status", "--prefix", str(prefix)], capture_output=True, text=True, timeout=20)
    assert q.returncode == 0, q.stderr
    return json.loads(q.stdout)


def test_codec_bytes_match_the_protobuf_library(host_lib, pb):
    """The golden bytes of the C++ unit test are what the protobuf library produces for the same messages."""
    P = pb["UnixSocketProto"]
    rule = P()
    r = rule.flow_steer_rule_request
    r.flow_steer_ntuple.flow_type = 1
    r.flow_steer_ntuple.src.ip_address, r.flow_steer_ntuple.src.port = "10.0.0.1", 5000
    r.flow_steer_ntuple.dst.ip_address, r.flow_steer_ntuple.dst.port = "10.0.0.2", 6000
    r.queue_id = 3
    r.gpu_pci_addr = "0000:1b:00.0"
    assert rule.SerializeToString().hex() == ("1232" "0a20" "0801" "120d" "0a08" "31302e302e302e31" "108827" "1a0d" "0a08" "31302e302e302e32"
                                              "10f02e" "1003" "1a0c" "303030303a31623a30302e30")
    assert P(raw_bytes=b"Ok.").SerializeToString().hex() == "0a034f6b2e"
    reg = P()
    reg.application_register_request.register_client = True
    assert reg.SerializeToString().hex() == "32020801"
    q = P()
    q.queue_id_query.gpu_pci_addr = "0000:1b:00.0"
    assert q.SerializeToString().hex() == "1a0e0a0c303030303a31623a30302e30"
    resp = P()
    resp.queue_id_response.queue_ids.extend([8, 9, 300])
    assert resp.SerializeToString().hex() == "2207080808090" "8ac02"
    neg = P()
    neg.flow_steer_rule_request.queue_id = -1
    assert neg.SerializeToString().hex() == "120b10ffffffffffffffffff01"
    r = subprocess.run([str(LIB / "tcpxb_unit_tests"), "rxdm_proto_wire_bytes"], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "ok rxdm_proto_wire_bytes" in r.stdout, r.stdout + r.stderr


def test_protobuf_library_client_against_the_daemon(host_lib, pb, tmp_path):
    """A client that knows only the reference's protocol (real protobuf, per-GPU sockets, descriptor as
    SCM_RIGHTS beside one byte) gets rules installed, a pool descriptor with its metadata, and a registration."""
    prefix = tmp_path / "rxdm"
    P = pb["UnixSocketProto"]
    pci = "0000:1b:00.0"
    d = start_daemon(prefix, "--pool-mb", "8", "--gpu-pci", pci + ",0000:2c:00.0")
    try:
        def rule(port):
            m = P()
            r = m.flow_steer_rule_request
            r.flow_steer_ntuple.flow_type = 1
            r.flow_steer_ntuple.src.ip_address, r.flow_steer_ntuple.src.port = "10.0.0.1", port
            r.flow_steer_ntuple.dst.ip_address, r.flow_steer_ntuple.dst.port = "10.0.0.2", 6000
            r.gpu_pci_addr = pci
            return m.SerializeToString()

        def reply_text(s):
            m = P()
            m.ParseFromString(read_frame(s))
            s.close()
            assert m.WhichOneof("payload") == "raw_bytes"
            return m.raw_bytes

        assert reply_text(call(prefix, "rx_rule_manager", rule(5000))) == b"Ok."
        assert reply_text(call(prefix, "rx_rule_manager", rule(5001))) == b"Ok."
        assert daemon_status(prefix)["flow_rules"] == 2
        assert reply_text(call(prefix, "rx_rule_uninstall", rule(5000))) == b"Ok."
        assert reply_text(call(prefix, "rx_rule_uninstall", rule(5000))).startswith(b"Not found")
        assert reply_text(call(prefix, "rx_rule_manager", P(raw_bytes=b"x").SerializeToString())).startswith(b"Invalid argument")
        assert daemon_status(prefix)["flow_rules"] == 1
        # the pool: descriptor first, then {int fd; size_t size; size_t align} as raw bytes
        s = call(prefix, "get_gpu_fd_" + pci, P(raw_bytes=pci.encode()).SerializeToString())
        data, fds, _flags, _addr = socket.recv_fds(s, 1, 1)
        s.close()
        assert len(data) == 1 and len(fds) == 1
        meta = reply_text(call(prefix, "get_gpu_metadata_" + pci, P(raw_bytes=pci.encode()).SerializeToString()))
        assert len(meta) == 24
        _fd, size, align = struct.unpack("<i4xQQ", meta)
        assert size == 8 << 20 and align == 4096
        assert os.fstat(fds[0]).st_size == size
        os.pwrite(fds[0], b"\x5a" * 16, 4096)
        # a second import sees the same memory
        s = call(prefix, "get_gpu_fd_" + pci, P(raw_bytes=pci.encode()).SerializeToString())
        _, fds2, _, _ = socket.recv_fds(s, 1, 1)
        s.close()
        assert os.pread(fds2[0], 16, 4096) == b"\x5a" * 16
        os.close(fds[0])
        os.close(fds2[0])
        assert (prefix / ("get_gpu_fd_0000:2c:00.0")).exists()
        # registration lives as long as its connection
        m = P()
        m.application_register_request.register_client = True
        keep = call(prefix, "rxdm_application_registry", m.SerializeToString())
        ok = P()
        ok.ParseFromString(read_frame(keep))
        assert ok.raw_bytes == b"Ok."
        st = daemon_status(prefix)
        assert st["applications"] == 1 and st["flow_rules"] == 1
        # the process "crashes": its keep-alive connection closes with a rule still installed, and the daemon cleans up
        keep.close()
        for _ in range(100):
            if daemon_status(prefix)["applications"] == 0:
                break
        st = daemon_status(prefix)
        assert st["applications"] == 0 and st["flow_rules"] == 0
    finally:
        log = stop_daemon(d)
    assert f"application {os.getpid()} went away; 1 flow rule(s) of process {os.getpid()} withdrawn" in log, log[-2000:]


def test_plugin_client_against_the_daemon_in_the_protobuf_format(host_lib, tmp_path):
    prefix = tmp_path / "rxdm"
    d = start_daemon(prefix, "--pool-mb", "8")
    try:
        env = dict(os.environ, TCPXB_TEST_RXDM_PREFIX=str(prefix), TCPXB_TEST_RXDM_WIRE="proto")
        r = subprocess.run([str(LIB / "tcpxb_unit_tests"), "rxdm_daemon"], capture_output=True, text=True, timeout=60, env=env)
        assert r.returncode == 0, r.stdout + r.stderr
        assert "ok rxdm_daemon_roundtrip" in r.stdout and "skipped" not in r.stdout
    finally:
        log = stop_daemon(d)
    assert "protobuf wire format" in log and "deregistered" in log


@pytest.mark.parametrize("pool", ["host", "device"])
def test_transfers_through_the_protobuf_format_daemon(host_lib, tmp_path, pool):
    """The whole transport with its rx pool, flow rules and registration served in the reference's wire format
    (device-pointer receives on the stand-in device; a device pool is told from a host pool by its descriptor)."""
    prefix = tmp_path / "rxdm"
    d = start_daemon(prefix, "--pool-mb", "32", *(["--device-pool"] if pool == "device" else []), env=dict(os.environ, TCPXB_FAKE_GPU="1"))
    try:
        env = dict(os.environ, TCPXB_FAKE_GPU="1", NCCL_GPUDIRECTTCPX_RX_BUF_MGR="daemon", NCCL_GPUDIRECTTCPX_RXDM_WIRE="proto",
                   NCCL_GPUDIRECTTCPX_UNIX_CLIENT_PREFIX=str(prefix), NCCL_GPUDIRECTTCPX_RECV_MODE="unpack", NCCL_PROTO="Simple",
                   NCCL_ALGO="Ring")
        r = subprocess.run([str(LIB / "tcpxb_loopback"), "--plugin", str(host_lib), "--ptr", "cuda", "--sizes", "0,1000,300000,4194304",
                            "--inflight", "8", "--iters", "2"], capture_output=True, text=True, timeout=300, env=env)
        assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
        assert "loopback PASSED" in r.stdout
        st = daemon_status(prefix)
        assert st["flow_rules"] == 0 and st["applications"] == 0 and st["pools"] == 1
    finally:
        log = stop_daemon(d)
    assert f"32 MiB of {pool} memory" in log, log[-2000:]


def test_plugin_client_against_a_protobuf_library_daemon(host_lib, pb, tmp_path):
    """This repository's client against a daemon written here in Python on the protobuf library: the other
    direction of the compatibility claim.  It serves a memfd pool for GPU "host", checks every request it
    parses, and answers as the reference's daemon does."""
    prefix = tmp_path / "rxdm"
    prefix.mkdir()
    P = pb["UnixSocketProto"]
    pool_bytes = 8 << 20
    pool_fd = os.memfd_create("pool")
    os.ftruncate(pool_fd, pool_bytes)
    seen = {"rules": [], "apps": 0, "registered": 0, "deregistered": 0, "errors": []}
    lock = threading.Lock()
    stop = threading.Event()
    keepalive = []

    def native_status_reply():
        # this repository's status service (the reference has none): magic, type, reserved, then the reply member of a 136-byte union
        body = struct.pack("<i64s4xQQQ", 0, b"Ok.", len(seen["rules"]), seen["apps"], 1)
        return struct.pack("<IHH", 0x4d445852, 0x8000, 0) + body.ljust(136, b"\0")

    def serve(name, conn):
        try:
            if name == "rxdm_status":
                read_frame(conn)
                with lock:
                    conn.sendall(frame(native_status_reply()))
                return
            m = P()
            m.ParseFromString(read_frame(conn))
            kind = m.WhichOneof("payload")
            if name in ("rx_rule_manager", "rx_rule_uninstall"):
                assert kind == "flow_steer_rule_request", kind
                r = m.flow_steer_rule_request
                assert r.flow_steer_ntuple.flow_type == 1 and not r.HasField("queue_id")
                key = (r.flow_steer_ntuple.src.ip_address, r.flow_steer_ntuple.src.port, r.flow_steer_ntuple.dst.ip_address,
                       r.flow_steer_ntuple.dst.port, r.gpu_pci_addr)
                assert key[0] == "127.0.0.1" and key[2] == "127.0.0.1" and 0 < key[1] < 65536 and 0 < key[3] < 65536
                with lock:
                    if name == "rx_rule_manager":
                        seen["rules"].append(key)
                    else:
                        seen["rules"].remove(key)
                conn.sendall(frame(P(raw_bytes=b"Ok.").SerializeToString()))
            elif name == "get_gpu_fd_host":
                assert kind == "raw_bytes"
                if m.raw_bytes == b"host":
                    socket.send_fds(conn, [b"\0"], [pool_fd])
                else:
                    conn.sendall(frame(P(raw_bytes=b"Invalid argument: no such GPU").SerializeToString()))
            elif name == "get_gpu_metadata_host":
                assert kind == "raw_bytes" and m.raw_bytes == b"host"
                conn.sendall(frame(P(raw_bytes=struct.pack("<i4xQQ", pool_fd, pool_bytes, 4096)).SerializeToString()))
            elif name == "rxdm_application_registry":
                assert kind == "application_register_request"
                conn.sendall(frame(P(raw_bytes=b"Ok.").SerializeToString()))
                if m.application_register_request.register_client:
                    with lock:
                        seen["apps"] += 1
                        seen["registered"] += 1
                    keepalive.append(conn)
                    conn.settimeout(30)
                    try:
                        while conn.recv(1):
                            pass
                    except OSError:
                        pass
                    with lock:
                        seen["apps"] -= 1
                else:
                    with lock:
                        seen["deregistered"] += 1
        except Exception as e:  # surfaces in the assertions below
            with lock:
                seen["errors"].append(f"{name}: {e!r}")
        finally:
            conn.close()

    listeners = []
    for name in ("rx_rule_manager", "rx_rule_uninstall", "get_gpu_fd_host", "get_gpu_metadata_host", "rxdm_application_registry", "rxdm_status"):
        ls = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        ls.bind(str(prefix / name))
        ls.listen(16)
        ls.settimeout(0.2)
        listeners.append((name, ls))

    def accept_loop(name, ls):
        while not stop.is_set():
            try:
                conn, _ = ls.accept()
            except socket.timeout:
                continue
            conn.settimeout(5)
            threading.Thread(target=serve, args=(name, conn), daemon=True).start()

    threads = [threading.Thread(target=accept_loop, args=l, daemon=True) for l in listeners]
    for t in threads:
        t.start()
    try:
        env = dict(os.environ, TCPXB_TEST_RXDM_PREFIX=str(prefix), TCPXB_TEST_RXDM_WIRE="proto")
        r = subprocess.run([str(LIB / "tcpxb_unit_tests"), "rxdm_daemon"], capture_output=True, text=True, timeout=60, env=env)
    finally:
        stop.set()
        for t in threads:
            t.join()
        for _, ls in listeners:
            ls.close()
        os.close(pool_fd)
    assert r.returncode == 0 and "ok rxdm_daemon_roundtrip" in r.stdout, r.stdout + r.stderr
    assert seen["errors"] == [], seen["errors"]
    assert seen["registered"] == 1 and seen["deregistered"] == 1 and seen["rules"] == []
