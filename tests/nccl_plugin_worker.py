"""Worker for the multi-GPU plugin tests: run under torch.distributed.run.

Every rank builds seeded inputs for all ranks, so each can compute the expected
result of a collective locally and compare it with what NCCL delivered through
the net transport.  Prints one JSON line per rank.
"""
import json
import os
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch
import torch.distributed as dist


def main():
    import faulthandler
    faulthandler.dump_traceback_later(int(os.environ.get("TCPXB_TEST_DUMP_AFTER", "60")), exit=False)
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    G = int(os.environ.get("TCPXB_TEST_GPUS_PER_NODE", "1"))
    if G > 1:  # emulated nodes of G GPUs: same host id inside a node, before NCCL initialises
        os.environ["NCCL_HOSTID"] = f"tcpxb-node-{rank // G}"
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    sizes = [int(s) for s in os.environ.get("TCPXB_TEST_SIZES", "256,65536,4194304").split(",")]
    rep = int(os.environ.get("TCPXB_TEST_REPEAT_SMALL", "0"))
    if rep:
        n = int(os.environ.get("TCPXB_TEST_REPEAT_ELEMS", "256"))
        pattern = ""
        for it in range(rep):
            ins = [torch.randn(n, generator=torch.Generator().manual_seed(77 * it + r)).to(torch.float32) for r in range(world)]
            x = ins[rank].to(dev)
            dist.all_reduce(x)
            torch.cuda.synchronize()
            want = torch.stack(ins).sum(0)
            pattern += "." if (x.cpu() - want).abs().max().item() < 1e-3 else "X"
        print(f"rank {rank} repeat pattern: {pattern}", flush=True)
    ok = True
    detail = []
    samples = []  # a few result values per case, for comparing two transports with each other
    for dtype in (torch.bfloat16, torch.float32):
        for n in sizes:
            gens = [torch.Generator().manual_seed(1000 * r + n % 997) for r in range(world)]
            ins = [torch.randn(n, generator=g).to(dtype) for g in gens]
            x = ins[rank].to(dev)
            dist.all_reduce(x)
            want = torch.stack([t.float() for t in ins]).sum(0)
            err = (x.float().cpu() - want).abs().max().item()
            tol = 0.05 * world if dtype == torch.bfloat16 else 1e-4 * world
            good = err <= tol
            samples.append([round(v, 6) for v in x.float().cpu()[:: max(1, n // 8)][:8].tolist()])
            # all_gather: exact
            outs = [torch.empty(n, dtype=dtype, device=dev) for _ in range(world)]
            dist.all_gather(outs, ins[rank].to(dev))
            good = good and all(torch.equal(o.cpu(), i) for o, i in zip(outs, ins))
            # reduce_scatter
            if n % world == 0:
                out = torch.empty(n // world, dtype=dtype, device=dev)
                dist.reduce_scatter_tensor(out, ins[rank].to(dev))
                w = want[rank * (n // world):(rank + 1) * (n // world)]
                good = good and (out.float().cpu() - w).abs().max().item() <= tol
            ok = ok and good
            detail.append((str(dtype), n, err, good))
    # a short timing sample, device-timed
    n = int(os.environ.get("TCPXB_TEST_BW_ELEMS", str(16 << 20)))
    x = torch.randn(n, device=dev).to(torch.bfloat16)
    for _ in range(2):
        dist.all_reduce(x)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    iters = 5
    e0.record()
    for _ in range(iters):
        dist.all_reduce(x)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    t = torch.tensor([ms], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    busbw = n * 2 / (t.item() * 1e-3) * 2 * (world - 1) / world / 1e9
    print(json.dumps({"rank": rank, "world": world, "G": G, "ok": bool(ok), "allreduce_ms": t.item(), "busbw_GBps": busbw,
                      "detail": detail, "samples": samples}), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
