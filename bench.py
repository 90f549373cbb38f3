#!/usr/bin/env python3
"""Headline benchmark: net-path all_reduce through the hierarchical engine.

One step = one bf16 all_reduce of `--size-mb` MiB per GPU whose inter-node stage
crosses the transport (pinned staging -> striped TCP sockets on loopback -> rx page
pool -> fused unpack+reduce(+NVLink fan-out) kernel).  N GPUs form 2 emulated nodes
of N/2 GPUs; a single GPU is its own network peer (a twin node with the same data).

  python bench.py --gpus 1 --steps 10 --warmup 3
  python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
         --master-port 29500 bench.py --gpus 8 --steps 10 --warmup 3

Rank 0 prints one JSON line.  `value` is the whole-job aggregate: N x bytes per GPU
all-reduced per second (GB/s), timed on the device with CUDA events, max over
ranks.  `e2e` repeats the measurement through the public API with the step's input
copied from pinned host memory and an 8-byte checksum of the result read back,
every step, inside the timed region; the copy of the next step's input runs on a
second stream during the current step (`--e2e-serial` puts it in line).
`--impl reference` reports why the unmodified reference cannot run here.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = ("net-path all_reduce GB/s, whole-job aggregate (bf16, 2 emulated nodes over loopback sockets; "
          "bus GB/s in config.busbw_GBps, unpack+reduce % roofline in unpack_microbench)")


def rails_and_threads(cores: int, world: int, nics: int = 0, nthreads: int = 0):
    """Rails (virtual NICs) and helper threads per connection for `world` ranks sharing `cores`
    cores; values given by the caller (> 0) are kept.  About one helper thread per core and
    direction: 4 cores per rank -> 2 x 1, 8 -> 4 x 1, 16 -> 4 x 2."""
    per_dir = max(1, min(8, cores // max(world, 1) // 2))
    if nics <= 0:
        nics = min(4, per_dir)
    if nthreads <= 0:
        nthreads = max(1, per_dir // nics)
    return nics, nthreads


def parse_args():
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
    ap.add_argument("--request-kb", type=int, default=4096)
    ap.add_argument("--unpack-ctas", type=int, default=16)
    ap.add_argument("--no-microbench", action="store_true")
    ap.add_argument("--e2e-serial", action="store_true", help="end-to-end loop: copy each step's input in line instead of prefetching it")
    ap.add_argument("--microbench-only", action="store_true", help="run only the unpack-kernel microbench (1 GPU)")
    ap.add_argument("--micro-iters", type=int, default=20)
    ap.add_argument("--micro-warm", type=int, default=4)
    return ap.parse_args()


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
    offsets; plain copy and fused bf16 sum; fraction of the measured copy bandwidth."""
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

    def timed(fn):
        for i in range(warm):
            fn(i)
        torch.cuda.synchronize()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
        for i in range(iters):
            ev[i][0].record()
            fn(i)
            ev[i][1].record()
        torch.cuda.synchronize()
        ts = sorted(a.elapsed_time(b) for a, b in ev)
        # and the same launches back to back inside one bracket (no event between them)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(iters):
            fn(i)
        b.record()
        torch.cuda.synchronize()
        return ts[len(ts) // 2] * 1e-3, a.elapsed_time(b) / iters * 1e-3

    t_copy, tb_copy = timed(lambda i: U.unpack_copy(pool, dsts[i % 3], descs[i % variants], status=st))
    t_red, tb_red = timed(lambda i: U.unpack_reduce(pool, dsts[i % 3], descs[i % variants], status=st))
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
    t_ref, tb_ref = timed(lambda i: dsts[i % 3].view(torch.uint8).copy_(flat))
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
        "unpack_reduce_fanout3_us": t_fan * 1e6, "unpack_reduce_fanout3_GBps": 6 * total / t_fan / 1e9,
        "unpack_reduce_fanout3_frac_hbm": 6 * total / t_fan / 1e9 / hbm,
        "unpack_reduce_fanout3_back_to_back_us": tb_fan * 1e6,
        "unpack_reduce_fanout3_back_to_back_frac_hbm": 6 * total / tb_fan / 1e9 / hbm,
        "unfused_unpack_add_3copies_us": t_unf * 1e6, "unfused_back_to_back_us": tb_unf * 1e6,
        "fusion_speedup_back_to_back": tb_unf / tb_fan,
        "status": st.tolist()[0],
    }
    del pool, descs, dsts, flat, peers, bounce
    torch.cuda.empty_cache()
    return out


def main():
    args = parse_args()
    if args.impl == "reference":
        return reference_arm()

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if args.gpus > 1 and world == 1:
        raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if args.microbench_only:
        try:
            peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
        except Exception:
            peaks = {}
        print(json.dumps({"unpack_microbench": unpack_microbench(torch, peaks, args.micro_iters, args.micro_warm)}))
        return 0

    from nccl_plugin_gpudirecttcpx_b200.parallel.engine import HierarchicalEngine, default_transport_env
    from nccl_plugin_gpudirecttcpx_b200.utils.clocks import ClockSampler
    from nccl_plugin_gpudirecttcpx_b200.ops import unpack as U

    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    # Socket helpers are CPU work and all ranks share the box: aim at about one helper
    # thread per core (measured: 4 cores per rank run best with 2 rails x 1 thread,
    # 8 with 4 x 1, 16 with 4 x 2).
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 16)
    args.nics, args.nthreads = rails_and_threads(cores, world, args.nics, args.nthreads)
    default_transport_env(nics=args.nics, nthreads=args.nthreads, nsocks_per_thread=args.nsocks_per_thread,
                          chunk_bytes=args.chunk_kb << 10, pool_mb=1024)
    G = max(1, world // 2)
    nbytes = args.size_mb << 20
    numel = nbytes // 2
    eng = HierarchicalEngine(gpus_per_node=G, buffer_bytes=nbytes if G > 1 else 0, request_bytes=args.request_kb << 10,
                             unpack_ctas=args.unpack_ctas, plain_mode=(args.impl == "plain"), device=dev)

    peaks = {}
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except Exception:
        pass

    # seeded synthetic input, N(0,1) bf16; every rank a different stream
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    x_dev = torch.randn(numel, device=dev, generator=g).to(torch.bfloat16)
    if G > 1:
        x_in = eng.work_view(numel, torch.bfloat16)
        x_in.copy_(x_dev)
    else:
        x_in = x_dev
    out = torch.empty_like(x_dev) if G == 1 else None

    def step():
        return eng.all_reduce(x_in, out)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # correctness of one step before timing: compare with the sum of the seeded inputs
    res = step()
    torch.cuda.synchronize()
    check_n = min(numel, 1 << 20)
    want = torch.zeros(check_n, dtype=torch.float32, device=dev)
    peers = range(world) if world > 1 else (0, 0)
    for r in peers:
        gr = torch.Generator(device=dev).manual_seed(1234 + r)
        want += torch.randn(numel, device=dev, generator=gr).to(torch.bfloat16)[:check_n].float()
    err = (res[:check_n].float() - want).abs().max().item()
    tol = 0.06 * max(2, world)
    if not err <= tol:
        raise SystemExit(f"all_reduce result is wrong: max abs err {err} > {tol}")
    if eng.device_status()[0] != 0:
        raise SystemExit(f"unpack kernels reported {eng.device_status()}")

    for _ in range(max(args.warmup - 1, 0)):
        step()
    barrier()
    s0 = eng.stats()
    k0, f0, b0 = s0.kernel_launches, s0.fragments, s0.bytes_received
    sampler = ClockSampler(local).start() if rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    s1 = eng.stats()
    launches = s1.kernel_launches - k0

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
        if not args.e2e_serial:
            issue_copy(0)
        for i in range(n_steps):
            b = i % 2
            if args.e2e_serial:
                issue_copy(i)
            elif i + 1 < n_steps:
                issue_copy(i + 1)
            main_stream.wait_event(ready[b])
            r = eng.all_reduce(stage[b], out)
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

    micro = None
    if rank == 0 and not args.no_microbench:
        micro = unpack_microbench(torch, peaks, args.micro_iters, args.micro_warm)

    if rank == 0:
        agg = world * nbytes / (ms * 1e-3) / 1e9
        agg_e2e = world * nbytes / (ms_e2e * 1e-3) / 1e9
        nodes = 2
        busbw = nbytes / (ms * 1e-3) / 1e9 * 2 * (max(world, 2) - 1) / max(world, 2)
        line = {
            "metric": METRIC, "value": agg, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (seeded N(0,1) bf16)", "impl": args.impl,
            "config": {
                "model": "all_reduce through the hierarchical engine", "global_batch": None, "seq_len": None,
                "bytes_per_gpu": nbytes, "parallelism": f"{nodes} emulated nodes x {G} GPU(s)" + (" (single GPU is its own peer)" if world == 1 else ""),
                "l2_policy": "inputs larger than L2: in+out = %d MiB per GPU" % (2 * args.size_mb),
                "transport": {"cpu_cores": cores, "nics": args.nics, "threads": args.nthreads, "socks_per_thread": args.nsocks_per_thread,
                              "chunk_kb": args.chunk_kb, "request_kb": args.request_kb, "unpack_ctas": args.unpack_ctas},
                "busbw_GBps": busbw, "net_bytes_per_gpu_per_step": (s1.bytes_received - b0) // max(args.steps, 1),
                "fragments_per_step": (s1.fragments - f0) // max(args.steps, 1), "max_abs_err": err,
                "driver_thread_ms_per_step": {k: round((getattr(s1, k) - getattr(s0, k)) * 1e3 / max(args.steps, 1), 3)
                                              for k in ("t_post_recv", "t_post_send", "t_test_recv", "t_launch",
                                                        "t_consume", "t_test_send", "t_idle")},
            },
            "e2e": {"value": agg_e2e, "unit": "GB/s", "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": 8,
                    "ms_per_step": ms_e2e, "checksum": last_sum,
                    "input_copy": "in line" if args.e2e_serial else "prefetched on a second stream during the previous step"},
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        if micro:
            line["unpack_microbench"] = micro
        print(json.dumps(line), flush=True)
    eng.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
