"""Size sweeps of all_reduce / all_gather / reduce_scatter over the net path.

  python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
      -m nccl_plugin_gpudirecttcpx_b200.parallel.sweep --path engine --gpus-per-node 4 \
      --ops all_reduce --min-bytes 1024 --max-bytes 8589934592

Paths: `engine` (hierarchical engine, fused unpack kernels), `engine-plain` (same
engine with the unfused baseline: unpack to a bounce buffer, separate add, copies to
the peers), `nccl-plugin` / `nccl-unpack` (stock NCCL over this plugin) and
`nccl-socket` (stock NCCL over its own socket transport, same socket settings).
Emulated nodes: `--gpus-per-node G` consecutive ranks share a node (NCCL paths use
NCCL_HOSTID for that).  Every number is device-timed with CUDA events and reduced
with MAX over ranks; rank 0 prints one JSON line per (op, dtype, size).
Sizes are bytes per rank for all_reduce, total output bytes for all_gather and total
input bytes for reduce_scatter, as nccl-tests counts them.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def parse_args(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--path", default="engine", choices=["engine", "engine-plain", "nccl-plugin", "nccl-unpack", "nccl-socket"])
    ap.add_argument("--gpus-per-node", type=int, default=1)
    ap.add_argument("--ops", default="all_reduce")
    ap.add_argument("--dtypes", default="bf16")
    ap.add_argument("--min-bytes", type=int, default=1024)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--factor", type=int, default=4)
    ap.add_argument("--sizes", default="", help="explicit comma-separated byte sizes (overrides min/max/factor)")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--nics", type=int, default=4)
    ap.add_argument("--nthreads", type=int, default=0, help="helper threads per connection (0 = from the cores per rank)")
    ap.add_argument("--request-kb", type=int, default=1024, help="engine paths: bytes per network request")
    ap.add_argument("--inflight", type=int, default=4, help="engine paths: requests in flight per rail")
    ap.add_argument("--nsocks-per-thread", type=int, default=1)
    ap.add_argument("--chunk-kb", type=int, default=512)
    return ap.parse_args(argv)


def main(argv=None) -> int:
    args = parse_args(argv)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    G = args.gpus_per_node
    nccl_path = args.path.startswith("nccl")
    if args.nthreads <= 0:
        cores_per_rank = max(1, len(os.sched_getaffinity(0)) // max(1, int(os.environ.get("LOCAL_WORLD_SIZE", str(world)))))
        # NCCL paths: 2 threads below 6 cores per rank, else 4 (what NCCL's socket transport liked best);
        # engine paths: helper threads beyond the rails only when cores are plentiful
        args.nthreads = (2 if cores_per_rank < 6 else 4) if nccl_path else max(1, min(4, cores_per_rank // 2 // max(1, args.nics)))
    if nccl_path:
        from .plugin_env import plugin_env
        env = plugin_env(nics=args.nics, nthreads=args.nthreads, nsocks_per_thread=args.nsocks_per_thread,
                         chunk_bytes=args.chunk_kb << 10, builtin_socket=(args.path == "nccl-socket"),
                         recv_mode="unpack" if args.path == "nccl-unpack" else "host")
        if G > 1:
            env.pop("NCCL_P2P_DISABLE", None)
            env.pop("NCCL_SHM_DISABLE", None)
            env["NCCL_HOSTID"] = f"tcpxb-node-{rank // G}"
        os.environ.update(env)

    import torch
    import torch.distributed as dist

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    sizes = [int(v) for v in args.sizes.split(",") if v]
    s = args.min_bytes
    while not args.sizes and s <= args.max_bytes:
        sizes.append(s)
        s *= args.factor
    eng = None
    if not nccl_path:
        from .engine import HierarchicalEngine, default_transport_env
        default_transport_env(nics=args.nics, nthreads=args.nthreads, nsocks_per_thread=args.nsocks_per_thread,
                              chunk_bytes=args.chunk_kb << 10)
        eng = HierarchicalEngine(gpus_per_node=G, buffer_bytes=max(sizes) if G > 1 else 0,
                                 request_bytes=args.request_kb << 10, max_inflight=args.inflight,
                                 plain_mode=(args.path == "engine-plain"), device=dev)
    nodes = max(2, world // G) if world > 1 else 2
    ranks = world if world > 1 else 2  # the single rank stands for a pair of twin nodes
    dtypes = {"bf16": torch.bfloat16, "fp32": torch.float32}
    for op in args.ops.split(","):
        for dname in args.dtypes.split(","):
            dtype = dtypes[dname]
            for nbytes in sizes:
                es = dtype.itemsize
                align = ranks * 16
                if op == "all_reduce":
                    n = max(nbytes // es // align * align, align)
                    x = torch.randn(n, device=dev).to(dtype)
                    if eng is not None:
                        xin = eng.work_view(n, dtype) if G > 1 else x
                        if G > 1:
                            xin.copy_(x)
                        fn = lambda: eng.all_reduce(xin)
                    else:
                        fn = lambda: dist.all_reduce(x)
                    factor = 2 * (ranks - 1) / ranks
                    moved = n * es
                elif op == "all_gather":
                    per = max(nbytes // ranks // es // 16 * 16, 16)
                    x = torch.randn(per, device=dev).to(dtype)
                    if eng is not None:
                        fn = lambda: eng.all_gather(x)
                    else:
                        out = torch.empty(per * world, dtype=dtype, device=dev)
                        fn = lambda: dist.all_gather_into_tensor(out, x)
                    factor = (ranks - 1) / ranks
                    moved = per * es * ranks
                else:
                    blocks = world if world > 1 else 1
                    per = max(nbytes // ranks // es // 16 * 16, 16)
                    x = torch.randn(per * blocks, device=dev).to(dtype)
                    if eng is not None:
                        xin = x
                        if G > 1:
                            xin = eng.work_view(per * blocks, dtype)
                            xin.copy_(x)
                        fn = lambda: eng.reduce_scatter(xin)
                    else:
                        out = torch.empty(per, dtype=dtype, device=dev)
                        fn = lambda: dist.reduce_scatter_tensor(out, x)
                    factor = (ranks - 1) / ranks
                    moved = per * es * ranks
                for _ in range(args.warmup):
                    fn()
                if world > 1:
                    dist.barrier()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                iters = args.iters if moved < (1 << 30) else max(2, args.iters // 2)
                e0.record()
                for _ in range(iters):
                    fn()
                e1.record()
                torch.cuda.synchronize()
                t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev, dtype=torch.float64)
                if world > 1:
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = t.item()
                if rank == 0:
                    alg = moved / (ms * 1e-3) / 1e9
                    print(json.dumps({"sweep": args.path, "op": op, "dtype": dname, "bytes": moved, "world": world, "gpus_per_node": G,
                                      "ms": round(ms, 4), "algbw_GBps": round(alg, 3), "busbw_GBps": round(alg * factor, 3)}), flush=True)
    if eng is not None:
        if rank == 0 and eng.device_status()[0] != 0:
            print(json.dumps({"sweep": args.path, "device_status": eng.device_status()}), flush=True)
        eng.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
