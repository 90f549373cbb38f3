"""One small, fixed workload per kernel of this library, for profiler captures.

    python -m nccl_plugin_gpudirecttcpx_b200.ops.profile_case --kernel reduce_fanout
    ncu --set full --clock-control none -k regex:unpack_kernel -s 2 -c 1 -o prof \
        python -m nccl_plugin_gpudirecttcpx_b200.ops.profile_case --kernel reduce_fanout

Every case moves 64 MiB assembled from 16 384 fragments of 4096 bytes at permuted offsets of
a 256 MiB pool (larger than L2, well under a GB on the device in total), bf16 payload, and
launches its kernel `--iters` times (default 3) after nothing else: a capture of launch 3
(`-s 2 -c 1`) sees a warmed-up kernel and ends in seconds.  One GPU: the "peers" of the fan-out
kernels are three more buffers on the same device, so the capture shows the kernel's
instruction mix and memory traffic, not NVLink.  Prints one JSON line with the CUDA-event time
of the last launch.
"""
from __future__ import annotations

import argparse
import json
import sys

KERNELS = ("copy", "reduce", "reduce_l2", "fanout", "reduce_fanout", "peer_reduce", "checksum", "copy_host_pool", "reduce_host_pool")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--kernel", choices=KERNELS, required=True)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--mb", type=int, default=64, help="bytes assembled per launch (MiB)")
    ap.add_argument("--ctas", type=int, default=0, help="CTA limit of the unpack kernels (0 = one per SM)")
    args = ap.parse_args(argv)

    import torch
    from . import unpack as U
    from .. import ops

    dev = torch.device("cuda")
    total = args.mb << 20
    pool_bytes = 256 << 20
    g = torch.Generator(device=dev).manual_seed(1)
    pool = torch.randn(pool_bytes // 2, device=dev, generator=g).to(torch.bfloat16)
    if args.kernel in ("copy_host_pool", "reduce_host_pool"):
        # the transport's default rx pool placement: pinned host memory the kernel reads over PCIe
        host = torch.empty(pool_bytes // 2, dtype=torch.bfloat16).pin_memory()
        host.copy_(pool)
        pool = host
    descs = U.descriptors_to_device(U.permuted_fragments(total, pool_bytes, seed=5))
    n_el = total // 2
    dst = torch.randn(n_el, device=dev, generator=g).to(torch.bfloat16)
    peers = [torch.empty(n_el, dtype=torch.bfloat16, device=dev) for _ in range(3)]
    st = U.status_buffer()
    flat = torch.randn(total // 2, device=dev, generator=g).to(torch.bfloat16)
    srcs = [flat] + peers
    out_q = torch.empty(n_el // 4, dtype=torch.bfloat16, device=dev)
    kw = {"max_ctas": args.ctas} if args.ctas else {}

    def run():
        k = args.kernel
        if k in ("copy", "copy_host_pool"):
            U.unpack_copy(pool, dst, descs, status=st, **kw)
        elif k in ("reduce", "reduce_host_pool"):
            U.unpack_reduce(pool, dst, descs, status=st, **kw)
        elif k == "reduce_l2":
            U.unpack_reduce(pool, dst, descs, status=st, impl=U.REDUCE_L2, **kw)
        elif k == "fanout":
            U.unpack_fanout(pool, dst, peers, descs, status=st, **kw)
        elif k == "reduce_fanout":
            U.unpack_reduce_fanout(pool, dst, dst, peers, descs, status=st, **kw)
        elif k == "peer_reduce":
            # the intra-node reduce-scatter stage: a quarter of four 64 MiB buffers summed
            ops.peer_reduce(out_q, srcs, shard_off=(total // 4))
        elif k == "checksum":
            ops.checksum(flat.view(torch.uint8))

    ms = 0.0
    for _ in range(max(args.iters, 1)):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
    print(json.dumps({"kernel": args.kernel, "mb": args.mb, "iters": args.iters, "last_launch_us": round(ms * 1e3, 2),
                      "status": st.tolist()[0]}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
