"""NVLink side of the fused unpack kernels, measured on 2, 4 or 8 GPUs of one box.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 \
        -m nccl_plugin_gpudirecttcpx_b200.parallel.fanout_bench

Every rank unpacks 64 MiB (16 384 fragments of 4096 bytes at permuted offsets of a local
256 MiB pool, bf16) and, in the same kernel, stores each fragment into the output buffer
of every other rank: all ranks at once, so every GPU's NVLink ports carry (G - 1) x 64 MiB
out and as much in.  Variants:

  fanout_peer          K3, bulk stores to each peer's mapping (`cp.async.bulk` shared -> global)
  fanout_nvls          K3, one `multimem.st` per 16 bytes through the switch's multicast object
  reduce_fanout_peer   K3r, fragment + local accumulator, the sum stored to every peer
  reduce_fanout_nvls   K3r with the `multimem.st` fan-out
  reduce_into_all_nvls `multimem.red`: the fragment is added into every GPU's accumulator in the switch
  unfused              the baseline: unpack_copy to a bounce buffer, a separate add, G - 1 peer copies

Times are CUDA-event times of `--iters` back-to-back launches, max over ranks; rank 0 prints
one JSON line per variant with the NVLink egress rate per GPU and its fraction of the link
rate measured on this pool (770 GB/s per direction, `--link-gbps` to override).  Results are
checked against the local unpack once per variant.  The kernels wait for nobody (completion
flags are off here; ranks meet at torch.distributed barriers between variants).
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mb", type=int, default=64)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--link-gbps", type=float, default=770.0)
    ap.add_argument("--no-nvls", action="store_true")
    args = ap.parse_args(argv)

    import torch
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm
    from ..ops import unpack as U
    from .. import ops

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        print(json.dumps({"fanout_bench": "needs 2 or more ranks"}))
        return 0
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)

    total = args.mb << 20
    n_el = total // 2
    pool_bytes = 256 << 20
    g = torch.Generator(device=dev).manual_seed(10 + rank)
    pool = torch.randn(pool_bytes // 2, device=dev, generator=g).to(torch.bfloat16)
    descs_np = U.permuted_fragments(total, pool_bytes, seed=20 + rank)
    descs = U.descriptors_to_device(descs_np)
    acc0 = torch.randn(n_el, device=dev, generator=g).to(torch.bfloat16)
    st = U.status_buffer()

    # the output buffer every rank exposes: world slots of 64 MiB, slot r is written by rank r
    out = symm.empty(world * n_el, dtype=torch.bfloat16, device=dev)
    out.zero_()
    hdl = symm.rendezvous(out, group=dist.group.WORLD)
    mc = 0 if args.no_nvls else int(getattr(hdl, "multicast_ptr", 0) or 0)
    slot_off = rank * total
    my_slot = out[rank * n_el:(rank + 1) * n_el]
    peer_ptrs = [int(p) + slot_off for r, p in enumerate(hdl.buffer_ptrs) if r != rank]
    bounce = torch.empty(n_el, dtype=torch.bfloat16, device=dev)
    peer_views = None  # torch tensors over the peers' slots, for the unfused copies

    def sync():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    # reference results, computed locally
    want_copy = torch.empty(n_el, dtype=torch.bfloat16, device=dev)
    U.unpack_copy(pool, want_copy, descs, status=st)
    want_sum = acc0.clone()
    U.unpack_reduce(pool, want_sum, descs, status=st)
    sync()

    variants = []
    variants.append(("fanout_peer", lambda: U.unpack_fanout(pool, my_slot, peer_ptrs, descs, status=st), None, want_copy))
    if mc:
        variants.append(("fanout_nvls", lambda: U.unpack_fanout(pool, my_slot, peer_ptrs, descs, status=st, mc_dst=mc + slot_off), None, want_copy))
    variants.append(("reduce_fanout_peer", lambda: U.unpack_reduce_fanout(pool, acc0, my_slot, peer_ptrs, descs, status=st), None, want_sum))
    if mc:
        variants.append(("reduce_fanout_nvls", lambda: U.unpack_reduce_fanout(pool, acc0, my_slot, peer_ptrs, descs, status=st, mc_dst=mc + slot_off),
                         None, want_sum))

    def unfused():
        U.unpack_copy(pool, bounce, descs, status=st)
        ops.peer_reduce(my_slot, [acc0, bounce], 0)
        for v in peer_views:
            v.copy_(my_slot, non_blocking=True)

    results = []
    egress = (world - 1) * total

    def time_variant(name, fn, check):
        for _ in range(args.warmup):
            fn()
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record()
        sync()
        t = torch.tensor([e0.elapsed_time(e1) / args.iters], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ok = True
        if check is not None:
            # my slot here, and my slot as the next rank sees it in its own buffer
            ok = bool(torch.equal(my_slot, check))
            # and what the previous rank stored into this GPU's buffer against that rank's expectation
            prev = (rank - 1) % world
            held = out[prev * n_el:(prev + 1) * n_el].clone()
            want_all = [torch.empty_like(check) for _ in range(world)]
            dist.all_gather(want_all, check)
            ok = ok and bool(torch.equal(held, want_all[prev]))
        okt = torch.tensor([1 if ok else 0], device=dev)
        dist.all_reduce(okt, op=dist.ReduceOp.MIN)
        ms = t.item()
        row = {"fanout_bench": name, "world": world, "mb": args.mb, "us_per_launch": round(ms * 1e3, 2),
               "nvlink_egress_GBps_per_gpu": round(egress / (ms * 1e-3) / 1e9, 1),
               "frac_of_link": round(egress / (ms * 1e-3) / 1e9 / args.link_gbps, 3), "link_GBps": args.link_gbps,
               "correct": bool(okt.item()), "status": st.tolist()[0]}
        results.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)

    for name, fn, _, check in variants:
        time_variant(name, fn, check)

    if mc:
        # reduce-into-all: every GPU's accumulator (its whole `out` buffer region of slot s) gets the fragment of rank s added
        def red_all():
            U.unpack_reduce_fanout(pool, None, my_slot, peer_ptrs, descs, status=st, mc_dst=mc + slot_off)
        out.zero_()
        sync()
        time_variant("reduce_into_all_nvls", red_all, None)

    # the unfused baseline needs tensors over the peers' slots
    try:
        peer_views = [hdl.get_buffer(r, (n_el,), torch.bfloat16, storage_offset=rank * n_el) for r in range(world) if r != rank]
        time_variant("unfused", unfused, want_sum)
    except Exception as e:  # older torch: no get_buffer with an offset
        if rank == 0:
            print(json.dumps({"fanout_bench": "unfused", "skipped": str(e)[:200]}), flush=True)

    sync()
    dist.destroy_process_group()
    return 0 if all(r["correct"] for r in results) else 1


if __name__ == "__main__":
    sys.exit(main())
