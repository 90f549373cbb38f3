#!/usr/bin/env python3
"""Headline benchmark: net-path all_reduce, bus GB/s.

One step = one bf16 all_reduce of `--size-mb` MiB per GPU whose inter-node stage
crosses loopback TCP sockets.  N GPUs form 2 emulated nodes of N/2 GPUs; a single GPU
is its own network peer (a twin node with the same data).

  python bench.py --gpus 1 --steps 10 --warmup 3
  python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
         --master-port 29500 bench.py --gpus 8 --steps 10 --warmup 3

Arms (`--impl`):
  ours         the hierarchical engine: pinned staging -> striped sockets -> rx page pool ->
               fused unpack + reduce (+ NVLink fan-out) kernels
  plain        the same engine, unfused (unpack to a bounce buffer, separate add, peer copies)
  nccl-socket  stock NCCL over its built-in socket transport, nodes told apart by NCCL_HOSTID
  nccl-plugin  stock NCCL with this repository's net plugin loaded, same node emulation
  reference    the unmodified reference; prints why it cannot run here

Rank 0 prints one JSON line.  `value` is the all_reduce bus bandwidth in GB/s
(bytes per GPU / time x 2(n-1)/n, n = ranks, a single GPU counting as a pair of
twins), timed on the device with CUDA events, max over ranks; `config.aggregate_GBps`
is N x bytes per GPU per second.  `e2e` repeats the measurement through the public
API with the step's input copied from pinned host memory and an 8-byte checksum of
the result read back, every step, inside the timed region.  The `ours` arm also
reports: a short size sweep (`sweep`), the box's raw socket ceiling for the same
number of streams and the step's fraction of it (`rawsock_ceiling_GBps`,
`frac_of_rawsock`: cache-resident 512 KiB blocks; `rawsock_uncached_GBps`,
`frac_of_rawsock_uncached`: 64 MiB per thread, the case of buffers that GPU DMA fills
and drains), and the same step over NCCL's socket transport run as a child job
after the engine has shut down (`nccl_socket`, `vs_nccl_socket`).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import socket
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "net-path all_reduce bus GB/s (bf16, 2 emulated nodes over loopback sockets); unpack+reduce % roofline in unpack_microbench"
SWEEP_BYTES = (1 << 10, 64 << 10, 4 << 20, 64 << 20)


def rails_and_threads(cores: int, world: int, nics: int = 0, nthreads: int = 0):
    """Rails (virtual NICs) and helper threads per connection for `world` ranks sharing `cores`
    cores; values given by the caller (> 0) are kept.  Helper threads sleep when they have
    nothing to do, so a rank may have more of them than cores: measured on 4 cores per rank,
    4 rails x 1 thread moved 14.2 GB/s against 11.7 for 2 x 1; with 16 cores 4 x 2 is as good
    as anything.  4 cores per rank -> 4 x 1, 8 -> 4 x 1, 16 -> 4 x 2."""
    per_rank = max(1, cores // max(world, 1))
    if nics <= 0:
        nics = min(4, per_rank)
    if nthreads <= 0:
        nthreads = max(1, min(4, per_rank // 2 // nics))
    return nics, nthreads


def bus_factor(world: int) -> float:
    n = max(world, 2)
    return 2.0 * (n - 1) / n


def parse_args(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "plain", "nccl-socket", "nccl-plugin"])
    ap.add_argument("--size-mb", type=int, default=256, help="all_reduce bytes per GPU (MiB)")
    ap.add_argument("--nics", type=int, default=0, help="virtual NICs = rails per rank (0 = from the core count)")
    ap.add_argument("--nthreads", type=int, default=0, help="helper threads (= sockets) per comm (0 = from the core count)")
    ap.add_argument("--nsocks-per-thread", type=int, default=1)
    ap.add_argument("--chunk-kb", type=int, default=128)
    ap.add_argument("--request-kb", type=int, default=1024)
    ap.add_argument("--unpack-ctas", type=int, default=16)
    ap.add_argument("--inflight", type=int, default=4, help="requests in flight per rail (0 = engine default)")
    ap.add_argument("--idle-sleep-us", type=int, default=0, help="driving thread: longest sleep when idle (0 = default, -1 = spin)")
    ap.add_argument("--pool-mb", type=int, default=1024, help="rx page pool per GPU (MiB)")
    ap.add_argument("--plugin-recv-mode", default="host", choices=["host", "unpack"], help="nccl-plugin arm: who unpacks")
    ap.add_argument("--nic-speed-mbps", type=int, default=200000, help="nccl-plugin arm: link speed the plugin reports per virtual NIC (NCCL sizes its channels from it)")
    ap.add_argument("--pin", default="none", choices=["none", "block", "pair"],
                    help="CPU affinity of each rank's process: none; block = rank r gets the r-th slice of the cores; "
                         "pair = the two ranks of a rail (same local index in the two nodes) get neighbouring slices")
    ap.add_argument("--no-microbench", action="store_true")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-compare", action="store_true", help="skip the raw-socket ceiling and the NCCL socket child run")
    ap.add_argument("--e2e-serial", action="store_true", help="end-to-end loop: copy each step's input in line instead of prefetching it")
    ap.add_argument("--microbench-only", action="store_true", help="run only the unpack-kernel microbench (1 GPU)")
    ap.add_argument("--micro-iters", type=int, default=20)
    ap.add_argument("--micro-warm", type=int, default=4)
    return ap.parse_args(argv)


def thread_cpu_seconds():
    """(user, system) CPU seconds of every thread of this process, keyed by (tid, name)."""
    out = {}
    try:
        tick = os.sysconf("SC_CLK_TCK")
        for tid in os.listdir("/proc/self/task"):
            st = Path(f"/proc/self/task/{tid}/stat").read_text()
            name = st[st.index("(") + 1:st.rindex(")")]
            f = st[st.rindex(")") + 2:].split()
            out[(tid, name)] = (int(f[11]) / tick, int(f[12]) / tick)
    except OSError:
        pass
    return out


def cpu_ms_per_step(before, after, steps):
    """Where a step's CPU time goes, per class of thread: the thread that drives the engine,
    the sending and the receiving socket helpers, everything else (CUDA, Python)."""
    main_tid = str(os.getpid())
    acc = {"driver": [0.0, 0.0], "tx_helpers": [0.0, 0.0], "rx_helpers": [0.0, 0.0], "other": [0.0, 0.0]}
    for key, (u, s) in after.items():
        u0, s0 = before.get(key, (0.0, 0.0))
        tid, name = key
        cls = "driver" if tid == main_tid else "tx_helpers" if name.startswith("tcpxb-tx") else \
            "rx_helpers" if name.startswith("tcpxb-rx") else "other"
        acc[cls][0] += u - u0
        acc[cls][1] += s - s0
    return {k: {"user": round(v[0] * 1e3 / max(steps, 1), 2), "sys": round(v[1] * 1e3 / max(steps, 1), 2)} for k, v in acc.items()}


def reference_arm():
    reason = ("reference is a CMake C++ library, not a pip-installable package, and needs protobuf, abseil, GTest, "
              "an NCCL source tree, the devmem-TCP kernel API and the RxDM daemon; none exist on this box")
    if int(os.environ.get("RANK", "0")) != 0:
        return 0  # one line per job, also when launched as N ranks
    marker = ROOT / "baseline" / "reference_install.log"
    if marker.exists():
        reason += f" (install attempt recorded in baseline/{marker.name})"
    print(json.dumps({"impl": "reference", "unavailable": reason}))
    return 0


def unpack_microbench(torch, peaks, iters=20, warm=4):
    """Config-2 microbench: 64 MiB assembled from 4096-byte fragments at permuted pool
    offsets; plain copy and fused bf16 sum; fraction of the measured copy bandwidth.
    Then the kernels as the net path runs them: one 4 MiB request of 1024 fragments with
    the page pool in pinned host memory (read over PCIe) and in HBM, 16 and 148 CTAs."""
    from nccl_plugin_gpudirecttcpx_b200.ops import unpack as U
    dev = torch.device("cuda")
    pool_bytes = 1 << 30
    total = (64 << 20) - 4096 + 2222  # the last fragment is ragged
    pool = torch.randn(pool_bytes // 4, device=dev).view(torch.bfloat16)
    variants = 8  # 8 x 64 MiB of distinct pool pages and 3 destinations: larger than L2 between iterations
    descs = [U.descriptors_to_device(U.permuted_fragments(total, pool_bytes, seed=i)) for i in range(variants)]
    dsts = [torch.randn((64 << 20) // 2, device=dev).to(torch.bfloat16) for _ in range(3)]
    st = U.status_buffer()

    # bring clocks and caches to their loaded state before the first measurement
    for i in range(40):
        U.unpack_copy(pool, dsts[i % 3], descs[i % variants], status=st)
    torch.cuda.synchronize()

    def timed(fn, n_iter=iters):
        for i in range(warm):
            fn(i)
        torch.cuda.synchronize()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_iter)]
        for i in range(n_iter):
            ev[i][0].record()
            fn(i)
            ev[i][1].record()
        torch.cuda.synchronize()
        ts = sorted(a.elapsed_time(b) for a, b in ev)
        # and the same launches back to back inside one bracket (no event between them)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(n_iter):
            fn(i)
        b.record()
        torch.cuda.synchronize()
        return ts[len(ts) // 2] * 1e-3, a.elapsed_time(b) / n_iter * 1e-3

    def graphed(fn, n_iter=iters):
        """The same launches captured once in a CUDA graph and replayed: what the GPU needs per
        launch when the host (here Python + ctypes, ~10 us per call) is out of the way."""
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for i in range(n_iter):
                    fn(i)
            g.replay()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / n_iter * 1e-3
        except Exception as e:  # capture is an extra, never a reason to lose the other numbers
            sys.stderr.write(f"graph capture failed: {e}\n")
            return None

    copy_fn = lambda i: U.unpack_copy(pool, dsts[i % 3], descs[i % variants], status=st)
    red_fn = lambda i: U.unpack_reduce(pool, dsts[i % 3], descs[i % variants], status=st)
    t_copy, tb_copy = timed(copy_fn)
    t_red, tb_red = timed(red_fn)
    tg_copy, tg_red = graphed(copy_fn), graphed(red_fn)
    # the same launches allowed to start early (programmatic dependent launch): the next launch is scheduled
    # while the previous one runs and waits for its completion on the device, so the gap between kernels goes
    copy_pdl = lambda i: U.unpack_copy(pool, dsts[i % 3], descs[i % variants], status=st, early_launch=True)
    red_pdl = lambda i: U.unpack_reduce(pool, dsts[i % 3], descs[i % variants], status=st, early_launch=True)
    tp_copy, tpb_copy = timed(copy_pdl)
    tp_red, tpb_red = timed(red_pdl)
    tpg_copy, tpg_red = graphed(copy_pdl), graphed(red_pdl)
    # fused reduce + fan-out with the three "peers" emulated by buffers on this GPU (no NVLink in
    # this number: it shows the kernel's cost of writing four copies of every reduced fragment)
    peers = [torch.empty((64 << 20) // 2, dtype=torch.bfloat16, device=dev) for _ in range(3)]
    t_fan, tb_fan = timed(lambda i: U.unpack_reduce_fanout(pool, dsts[i % 3], dsts[i % 3], peers, descs[i % variants], status=st))
    # the same result without fusion: unpack to a bounce buffer, add in a second pass, three copies
    bounce = torch.empty((64 << 20) // 2, dtype=torch.bfloat16, device=dev)
    n_el = total // 2 // 8 * 8

    def unfused(i):
        acc = dsts[i % 3]
        U.unpack_copy(pool, bounce, descs[i % variants], status=st)
        U.peer_reduce(acc[:n_el], [acc, bounce], 0)
        for p in peers:
            p.copy_(acc)

    t_unf, tb_unf = timed(unfused)
    flat = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
    ref_fn = lambda i: dsts[i % 3].view(torch.uint8).copy_(flat)
    t_ref, tb_ref = timed(ref_fn)
    tg_ref = graphed(ref_fn)
    hbm = peaks.get("hbm_gbs", 6650.0)
    tag = "of measured" if "hbm_gbs" in peaks else "of fallback"
    out = {
        "unpack_copy_us": t_copy * 1e6, "unpack_copy_GBps": 2 * total / t_copy / 1e9,
        "unpack_copy_frac_hbm": 2 * total / t_copy / 1e9 / hbm,
        "unpack_reduce_us": t_red * 1e6, "unpack_reduce_GBps": 3 * total / t_red / 1e9,
        "unpack_reduce_frac_hbm": 3 * total / t_red / 1e9 / hbm, "roofline": tag,
        "back_to_back": {"unpack_copy_us": tb_copy * 1e6, "unpack_copy_frac_hbm": 2 * total / tb_copy / 1e9 / hbm,
                         "unpack_reduce_us": tb_red * 1e6, "unpack_reduce_frac_hbm": 3 * total / tb_red / 1e9 / hbm,
                         "torch_copy_64MiB_us": tb_ref * 1e6, "torch_copy_64MiB_frac_hbm": 2 * (64 << 20) / tb_ref / 1e9 / hbm},
        "torch_copy_64MiB_us": t_ref * 1e6,
        "graph_replay": None if not (tg_copy and tg_red and tg_ref) else {
            "unpack_copy_us": tg_copy * 1e6, "unpack_copy_frac_hbm": 2 * total / tg_copy / 1e9 / hbm,
            "unpack_reduce_us": tg_red * 1e6, "unpack_reduce_frac_hbm": 3 * total / tg_red / 1e9 / hbm,
            "torch_copy_64MiB_us": tg_ref * 1e6, "torch_copy_64MiB_frac_hbm": 2 * (64 << 20) / tg_ref / 1e9 / hbm,
            "note": "20 launches captured in one CUDA graph, one replay timed"},
        "early_launch": {
            "unpack_copy_us": tp_copy * 1e6, "unpack_copy_frac_hbm": 2 * total / tp_copy / 1e9 / hbm,
            "unpack_reduce_us": tp_red * 1e6, "unpack_reduce_frac_hbm": 3 * total / tp_red / 1e9 / hbm,
            "back_to_back_unpack_copy_us": tpb_copy * 1e6, "back_to_back_unpack_copy_frac_hbm": 2 * total / tpb_copy / 1e9 / hbm,
            "back_to_back_unpack_reduce_us": tpb_red * 1e6, "back_to_back_unpack_reduce_frac_hbm": 3 * total / tpb_red / 1e9 / hbm,
            "graph_replay_unpack_copy_us": None if not tpg_copy else tpg_copy * 1e6,
            "graph_replay_unpack_copy_frac_hbm": None if not tpg_copy else 2 * total / tpg_copy / 1e9 / hbm,
            "graph_replay_unpack_reduce_us": None if not tpg_red else tpg_red * 1e6,
            "graph_replay_unpack_reduce_frac_hbm": None if not tpg_red else 3 * total / tpg_red / 1e9 / hbm,
            "note": "opts.early_launch = 1 (programmatic dependent launch) on every launch"},
        "unpack_reduce_fanout3_us": t_fan * 1e6, "unpack_reduce_fanout3_GBps": 6 * total / t_fan / 1e9,
        "unpack_reduce_fanout3_frac_hbm": 6 * total / t_fan / 1e9 / hbm,
        "unpack_reduce_fanout3_back_to_back_us": tb_fan * 1e6,
        "unpack_reduce_fanout3_back_to_back_frac_hbm": 6 * total / tb_fan / 1e9 / hbm,
        "unfused_unpack_add_3copies_us": t_unf * 1e6, "unfused_back_to_back_us": tb_unf * 1e6,
        "fusion_speedup_back_to_back": tb_unf / tb_fan,
        "status": st.tolist()[0],
    }
    del flat, peers, bounce

    # --- the kernels in the configuration the net path runs: one 4 MiB request (1024 fragments)
    req = 4 << 20
    host_pool = torch.empty(256 << 20, dtype=torch.uint8, pin_memory=True)
    host_pool.view(torch.bfloat16).normal_()
    pool_u8 = pool.view(torch.uint8)
    nvar = 16  # 16 x 4 MiB of distinct pool pages per placement
    hdescs = [U.descriptors_to_device(U.permuted_fragments(req, 256 << 20, seed=100 + i)) for i in range(nvar)]
    ddescs = [U.descriptors_to_device(U.permuted_fragments(req, pool_bytes, seed=200 + i)) for i in range(nvar)]
    acc = dsts[0]
    net = {}
    # pinned memory is addressable from the device at the same address (unified addressing)
    for place, pl, ds in (("host_pool", host_pool, hdescs), ("hbm_pool", pool_u8, ddescs)):
        for ctas in (16, 148):
            def one(i, pl=pl, ds=ds, ctas=ctas):
                off = (i % 8) * (req // 2)
                U.unpack_reduce(pl, acc[off:off + req // 2], ds[i % nvar], status=st, max_ctas=ctas)
            t1, tb = timed(one, n_iter=16)
            net[f"net_path_unpack_reduce_{place}_{ctas}ctas_us"] = round(t1 * 1e6, 2)
            net[f"net_path_unpack_reduce_{place}_{ctas}ctas_back_to_back_us"] = round(tb * 1e6, 2)
            net[f"net_path_unpack_reduce_{place}_{ctas}ctas_GBps_of_payload"] = round(req / tb / 1e9, 1)
    net["net_path_note"] = ("one 4 MiB request = 1024 fragments of 4 KiB; host_pool = pinned host memory read over PCIe by the "
                            "kernel (the transport's default placement), hbm_pool = pool in device memory")
    net["status"] = st.tolist()[0]
    out.update(net)
    del pool, descs, dsts, host_pool, hdescs, ddescs
    torch.cuda.empty_cache()
    return out


def check_all_reduce(torch, res, numel, rank, world, dev):
    """The whole result against the fp32 sum of every rank's seeded input.  The tolerance
    scales with the values: each of the path's roundings (one per reduction level) is at
    most 2^-8 of the partial sum it rounds, so 2^-8 x levels x sum of |inputs| bounds the error."""
    peers = list(range(world)) if world > 1 else [0, 0]
    want = torch.zeros(numel, dtype=torch.float32, device=dev)
    mag = torch.zeros(numel, dtype=torch.float32, device=dev)
    for r in peers:
        gr = torch.Generator(device=dev).manual_seed(1234 + r)
        x = torch.randn(numel, device=dev, generator=gr).to(torch.bfloat16).float()
        want += x
        mag += x.abs()
    levels = max(1, math.ceil(math.log2(len(peers))))
    tol = mag * (2.0 ** -8 * levels) + 1e-6
    diff = (res.float() - want).abs()
    bad = int((diff > tol).sum().item())
    return {"checked_elems": int(numel), "bad_elems": bad, "max_abs_err": float(diff.max().item()),
            "max_err_over_tol": float((diff / tol).max().item())}


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_rawsock(streams: int, span_mb: int = 0, sndbuf_kb: int = 0):
    """Plain send/recv loops over loopback TCP, `streams` connections.  `span_mb` = 0: every thread reuses one
    512 KiB block (cache-resident, the kindest case); otherwise each thread walks a buffer of that many MiB,
    like a transport whose staging and landing memory is written and read by GPU DMA and never cache-warm."""
    from nccl_plugin_gpudirecttcpx_b200.utils import native
    exe = native.LIB_DIR / "tcpxb_rawsock"
    if not exe.exists():
        return None
    try:
        cmd = [str(exe), "--streams", str(streams), "--mb-per-stream", "1024"] + (["--span-mb", str(span_mb)] if span_mb else []) + \
            (["--sndbuf-kb", str(sndbuf_kb)] if sndbuf_kb else [])
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=120)
        for line in r.stdout.splitlines():
            if line.startswith("{"):
                return json.loads(line)
    except Exception:
        return None
    return None


def run_child_arm(impl: str, args, world: int):
    """Runs this script's `impl` arm as a separate job on the same GPUs and returns its JSON line."""
    cmd = [sys.executable]
    if world > 1:
        cmd += ["-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                "--master-port", str(free_port())]
    cmd += [str(ROOT / "bench.py"), "--impl", impl, "--gpus", str(world), "--steps", str(args.steps), "--warmup", str(args.warmup),
            "--size-mb", str(args.size_mb), "--no-microbench", "--no-compare", "--pin", args.pin]
    if args.no_sweep:
        cmd.append("--no-sweep")
    drop = ("NCCL_", "TORCHELASTIC", "MASTER_", "RANK", "LOCAL_RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE", "GROUP_", "ROLE_", "TORCH_NCCL")
    env = {k: v for k, v in os.environ.items() if not k.startswith(drop)}
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    except subprocess.TimeoutExpired:
        return {"error": "child run timed out"}
    for line in r.stdout.splitlines():
        if line.startswith("{"):
            try:
                return json.loads(line)
            except ValueError:
                continue
    return {"error": "no result line", "rc": r.returncode, "stderr_tail": r.stderr[-400:]}


def timed_steps(torch, step, steps, barrier):
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    barrier()
    return e0.elapsed_time(e1) / steps


def main():
    args = parse_args()
    if args.impl == "reference":
        return reference_arm()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if args.gpus > 1 and world == 1:
        raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    nccl_arm = args.impl.startswith("nccl")
    G = max(1, world // 2)
    if args.pin != "none" and world > 1 and hasattr(os, "sched_setaffinity"):
        # before any thread exists: helper threads, CUDA's and NCCL's inherit the mask
        avail = sorted(os.sched_getaffinity(0))
        per = max(1, len(avail) // world)
        slot = rank if args.pin == "block" else (rank % G) * 2 + rank // G
        mine = avail[slot * per:(slot + 1) * per]
        if mine:
            os.sched_setaffinity(0, mine)
    total_cores = os.cpu_count() or 16
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else total_cores
    if args.pin != "none" and world > 1:
        cores = cores * world  # the helpers below size threads from the box's cores shared by all ranks

    if nccl_arm:
        if world < 2:
            if rank == 0:
                print(json.dumps({"impl": args.impl, "unavailable": "NCCL has no network path with a single rank; run with --gpus 2 or more"}))
            return 0
        # must be in the environment before NCCL initialises
        from nccl_plugin_gpudirecttcpx_b200.parallel.plugin_env import plugin_env, socket_settings_for
        auto = socket_settings_for(cores, world)
        env = plugin_env(nics=args.nics if args.nics > 0 else 4, nthreads=args.nthreads if args.nthreads > 0 else auto["nthreads"],
                         nsocks_per_thread=args.nsocks_per_thread, chunk_bytes=args.chunk_kb << 10,
                         builtin_socket=(args.impl == "nccl-socket"), recv_mode=args.plugin_recv_mode, rx_pool_mb=args.pool_mb,
                         speed_mbps=args.nic_speed_mbps)
        if G > 1:  # nodes are told apart by host id, so NVLink stays on inside a node
            env.pop("NCCL_P2P_DISABLE", None)
            env.pop("NCCL_SHM_DISABLE", None)
            env["NCCL_HOSTID"] = f"tcpxb-node-{rank // G}"
        os.environ.update(env)

    import torch
    import torch.distributed as dist

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except Exception:
        peaks = {}
    if args.microbench_only:
        print(json.dumps({"unpack_microbench": unpack_microbench(torch, peaks, args.micro_iters, args.micro_warm)}))
        return 0

    from nccl_plugin_gpudirecttcpx_b200.utils.clocks import ClockSampler
    from nccl_plugin_gpudirecttcpx_b200.ops import unpack as U

    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    nbytes = args.size_mb << 20
    numel = nbytes // 2
    eng = None
    if not nccl_arm:
        from nccl_plugin_gpudirecttcpx_b200.parallel.engine import HierarchicalEngine, default_transport_env
        # Socket helpers are CPU work and all ranks share the box: aim at about one helper
        # thread per core (measured: 4 cores per rank run best with 2 rails x 1 thread,
        # 8 with 4 x 1, 16 with 4 x 2).
        args.nics, args.nthreads = rails_and_threads(cores, world, args.nics, args.nthreads)
        default_transport_env(nics=args.nics, nthreads=args.nthreads, nsocks_per_thread=args.nsocks_per_thread,
                              chunk_bytes=args.chunk_kb << 10, pool_mb=args.pool_mb)
        eng = HierarchicalEngine(gpus_per_node=G, buffer_bytes=nbytes if G > 1 else 0, request_bytes=args.request_kb << 10,
                                 unpack_ctas=args.unpack_ctas, plain_mode=(args.impl == "plain"), device=dev,
                                 max_inflight=args.inflight, idle_sleep_us=args.idle_sleep_us)
        transport = {"cpu_cores": cores, "pin": args.pin, "nics": args.nics, "threads": args.nthreads, "socks_per_thread": args.nsocks_per_thread,
                     "chunk_kb": args.chunk_kb, "request_kb": args.request_kb, "unpack_ctas": args.unpack_ctas,
                     "sndbuf_kb": int(os.environ.get("NCCL_GPUDIRECTTCPX_SOCKET_SNDBUF", "0")) >> 10,
                     "streams_per_direction_on_the_box": max(world, 1) * args.nics * args.nthreads * args.nsocks_per_thread}
    else:
        transport = {"cpu_cores": cores, "pin": args.pin, "env": {k: v for k, v in os.environ.items() if k.startswith("NCCL_") and "PLUGIN" not in k}}
    is_engine = eng is not None

    # seeded synthetic input, N(0,1) bf16; every rank a different stream
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    x_dev = torch.randn(numel, device=dev, generator=g).to(torch.bfloat16)
    if is_engine and G > 1:
        x_in = eng.work_view(numel, torch.bfloat16)
        x_in.copy_(x_dev)
    else:
        x_in = x_dev
    out = torch.empty_like(x_dev) if (is_engine and G == 1) else None
    nccl_buf = torch.empty_like(x_dev) if nccl_arm else None

    def all_reduce_of(src):
        """One all_reduce of `src` through the arm's public API; returns the result tensor."""
        if is_engine:
            return eng.all_reduce(src, out)
        nccl_buf.copy_(src)  # NCCL reduces in place: the input is kept for the next step
        dist.all_reduce(nccl_buf)
        return nccl_buf

    def step():
        return all_reduce_of(x_in)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # correctness of one step before timing: the whole result against the sum of the seeded inputs
    res = step()
    torch.cuda.synchronize()
    check = check_all_reduce(torch, res, numel, rank, world, dev)
    if world == 1:
        check["exact_2x"] = bool(torch.equal(res, (x_dev.float() * 2).to(torch.bfloat16)))
    if check["bad_elems"] != 0 or check.get("exact_2x") is False:
        raise SystemExit(f"all_reduce result is wrong: {check}")
    if is_engine and eng.device_status()[0] != 0:
        raise SystemExit(f"unpack kernels reported {eng.device_status()}")
    want_sum = int(U.checksum(res.view(torch.uint8)).item())  # every later step has the same input, so the same result

    for _ in range(max(args.warmup - 1, 0)):
        step()
    barrier()
    s0 = eng.stats() if is_engine else None
    cpu0 = thread_cpu_seconds()
    sampler = ClockSampler(local).start() if rank == 0 else None
    ms = timed_steps(torch, step, args.steps, barrier)
    s1 = eng.stats() if is_engine else None
    cpu_ms = cpu_ms_per_step(cpu0, thread_cpu_seconds(), args.steps)

    # end to end through the public API: pinned host input in, checksum out, every step
    host_in = torch.empty(numel, dtype=torch.bfloat16, pin_memory=True)
    host_in.copy_(x_dev)
    host_out = torch.empty(1, dtype=torch.int64, pin_memory=True)
    csum = torch.empty(1, dtype=torch.int64, device=dev)

    # The input of step i + 1 is copied on a second stream while step i runs, as a
    # training loop's input prefetch does; every step's copy, collective, checksum and
    # read-back lies inside the timed region.  --e2e-serial puts the copy in line.
    copy_stream = torch.cuda.Stream(device=dev)
    main_stream = torch.cuda.current_stream(dev)
    stage = [torch.empty_like(x_dev), torch.empty_like(x_dev)]
    prefetch = not args.e2e_serial
    ready = [torch.cuda.Event(), torch.cuda.Event()]
    freed = [torch.cuda.Event(), torch.cuda.Event()]

    def issue_copy(i):
        b = i % 2
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(freed[b])             # the step that last used this buffer is done with it
            stage[b].copy_(host_in, non_blocking=True)   # host -> device: input of step i
            ready[b].record(copy_stream)

    def e2e_run(n_steps):
        last = 0
        for b in range(2):
            freed[b].record(main_stream)
        if prefetch:
            issue_copy(0)
        for i in range(n_steps):
            b = i % 2
            if not prefetch:
                issue_copy(i)
            elif i + 1 < n_steps:
                issue_copy(i + 1)
            main_stream.wait_event(ready[b])
            r = all_reduce_of(stage[b])
            freed[b].record(main_stream)
            U.checksum(r.view(torch.uint8), out=csum)
            host_out.copy_(csum, non_blocking=True)      # device -> host: this step's result
            main_stream.synchronize()
            last = int(host_out.item())
        return last

    e2e_run(2)
    barrier()
    f0e, f1e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0e.record()
    last_sum = e2e_run(args.steps)
    f1e.record()
    barrier()
    ms_e2e = f0e.elapsed_time(f1e) / args.steps
    clocks = sampler.stop() if sampler else None

    t = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = t[0].item(), t[1].item()

    # a short sweep over message sizes, for the small-message half of the metric: 2 timed steps each from 4 MiB
    # up, 20 below (a pair of steps of 0.1 ms each says little), 3 warm-up steps before either
    sweep = []
    if not args.no_sweep:
        for sb in SWEEP_BYTES:
            n_el = max(sb // 2, 8 * max(world, 2))
            src = x_in[:n_el]
            if nccl_arm:
                small = torch.empty_like(src)
                fn = lambda: (small.copy_(src), dist.all_reduce(small))
            elif G > 1:
                fn = lambda: eng.all_reduce(src)
            else:
                small_out = torch.empty_like(src)
                fn = lambda: eng.all_reduce(src, small_out)
            for _ in range(3):
                fn()
            t_ms = timed_steps(torch, fn, 2 if sb >= (4 << 20) else 20, barrier)
            tt = torch.tensor([t_ms], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            sweep.append({"bytes": n_el * 2, "ms": round(tt.item(), 4),
                          "busbw_GBps": round(n_el * 2 / (tt.item() * 1e-3) / 1e9 * bus_factor(world), 4)})

    micro = None
    if rank == 0 and is_engine and not args.no_microbench:
        micro = unpack_microbench(torch, peaks, args.micro_iters, args.micro_warm)

    launches, drv, net_bytes, frags = 0, None, 0, 0
    if is_engine:
        launches = int(s1.kernel_launches - s0.kernel_launches)
        drv = {k: round((getattr(s1, k) - getattr(s0, k)) * 1e3 / max(args.steps, 1), 3)
               for k in ("t_post_recv", "t_post_send", "t_test_recv", "t_launch", "t_consume", "t_test_send", "t_idle", "t_sleep",
                         "tx_idle", "tx_blocked", "rx_idle", "rx_blocked")}
        drv["sleeps"] = int((s1.sleeps - s0.sleeps) // max(args.steps, 1))
        net_bytes = (s1.bytes_received - s0.bytes_received) // max(args.steps, 1)
        frags = (s1.fragments - s0.fragments) // max(args.steps, 1)
        eng.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return 0

    # ---- rank 0 only from here; the other ranks have left and the GPUs are idle
    busbw = nbytes / (ms * 1e-3) / 1e9 * bus_factor(world)
    busbw_e2e = nbytes / (ms_e2e * 1e-3) / 1e9 * bus_factor(world)
    line = {
        "metric": METRIC, "value": busbw, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (seeded N(0,1) bf16)", "impl": args.impl,
        "config": {
            "model": "all_reduce, net path" + (" through the hierarchical engine" if is_engine else " through stock NCCL"),
            "global_batch": None, "seq_len": None, "bytes_per_gpu": nbytes,
            "parallelism": f"2 emulated nodes x {G} GPU(s)" + (" (single GPU is its own peer)" if world == 1 else ""),
            "l2_policy": "inputs larger than L2: in+out = %d MiB per GPU" % (2 * args.size_mb),
            "aggregate_GBps": world * nbytes / (ms * 1e-3) / 1e9,
            "transport": transport, "check": check, "cpu_ms_per_step_rank0": cpu_ms,
        },
        "e2e": {"value": busbw_e2e, "unit": "GB/s", "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": 8,
                "ms_per_step": ms_e2e, "checksum": last_sum, "checksum_matches_device_timed_result": last_sum == want_sum,
                "input_copy": "prefetched on a second stream during the previous step" if prefetch else "in line"},
        "gpu_launches": launches,
        "clocks": clocks,
    }
    if is_engine:
        line["config"].update({"net_bytes_per_gpu_per_step": int(net_bytes), "fragments_per_step": int(frags),
                               "driver_thread_ms_per_step": drv})
    else:
        line["gpu_launches_note"] = "kernels of NCCL and torch only are counted as 0: none of this repository's kernels is launched by this arm's own code"
    if sweep:
        line["sweep"] = sweep
    if micro:
        line["unpack_microbench"] = micro
    if is_engine and not args.no_compare:
        streams = transport["streams_per_direction_on_the_box"]
        raw = run_rawsock(streams)
        if raw:
            # the step moves N x (bytes per GPU / G) through the box's sockets
            net_GBps = world * (nbytes / G) / (ms * 1e-3) / 1e9
            line["rawsock_ceiling_GBps"] = raw["GBps"]
            line["rawsock_streams"] = streams
            line["net_stage_GBps"] = net_GBps
            line["frac_of_rawsock"] = net_GBps / raw["GBps"] if raw["GBps"] else None
            # the same loops with buffers that do not fit the caches and the send buffer the transport uses
            sndbuf_kb = int(os.environ.get("NCCL_GPUDIRECTTCPX_SOCKET_SNDBUF", "0")) >> 10
            cold = run_rawsock(streams, span_mb=64, sndbuf_kb=sndbuf_kb)
            if cold and cold.get("GBps"):
                line["rawsock_uncached_sndbuf_kb"] = sndbuf_kb
                line["rawsock_uncached_GBps"] = cold["GBps"]
                line["frac_of_rawsock_uncached"] = net_GBps / cold["GBps"]
        if world > 1:
            child = run_child_arm("nccl-socket", args, world)
            if child and "value" in child:
                line["nccl_socket"] = {"busbw_GBps": child["value"], "ms_per_step": child["ms_per_step"],
                                       "e2e_busbw_GBps": child["e2e"]["value"], "sweep": child.get("sweep")}
                line["vs_nccl_socket"] = busbw / child["value"] if child["value"] else None
                line["e2e_vs_nccl_socket"] = busbw_e2e / child["e2e"]["value"] if child["e2e"]["value"] else None
            else:
                line["nccl_socket"] = child
    print(json.dumps(line), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
