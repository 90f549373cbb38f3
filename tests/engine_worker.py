"""Worker for the multi-GPU engine tests (run under torch.distributed.run).

Ranks form `world / G` emulated nodes of G GPUs.  Every rank can rebuild every
rank's seeded input, so results are checked locally against a plain PyTorch fp32
sum.  Prints one JSON line per rank and exits non-zero on a mismatch.
"""
import faulthandler
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch
import torch.distributed as dist


def main():
    faulthandler.dump_traceback_later(int(os.environ.get("TCPXB_TEST_DUMP_AFTER", "100")), exit=True)
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    G = int(os.environ.get("TCPXB_TEST_GPUS_PER_NODE", "1"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from nccl_plugin_gpudirecttcpx_b200.parallel.engine import HierarchicalEngine, default_transport_env
    default_transport_env(nics=2, nthreads=2, nsocks_per_thread=1, pool_mb=256)
    numels = [int(s) for s in os.environ.get("TCPXB_TEST_NUMELS", "4096,1048576,3145728").split(",")]
    buf_bytes = max(numels) * 4 * 2
    eng = HierarchicalEngine(gpus_per_node=G, buffer_bytes=buf_bytes if G > 1 else 0, request_bytes=1 << 20,
                             use_nvls=bool(int(os.environ.get("TCPXB_TEST_NVLS", "0"))),
                             plain_mode=bool(int(os.environ.get("TCPXB_TEST_PLAIN", "0"))))
    ok = True
    detail = []
    for dtype in (torch.bfloat16, torch.float32):
        for n in numels:
            ins = [torch.randn(n, generator=torch.Generator().manual_seed(100 * r + n % 911)).to(dtype) for r in range(world)]
            want = torch.stack([t.float() for t in ins]).sum(0)
            tol = 0.04 * world if dtype == torch.bfloat16 else 1e-4 * world
            for rep in range(2):  # twice: buffers and flag epochs are reused
                y = eng.all_reduce(ins[rank].to(dev))
                torch.cuda.synchronize()
                err = (y.float().cpu() - want).abs().max().item()
                good = err <= tol
                ok = ok and good
                detail.append(("all_reduce", str(dtype), n, rep, err, good))
            if n % world == 0:
                g = eng.all_gather(ins[rank][: n // world].to(dev))
                torch.cuda.synchronize()
                wantg = torch.cat([t[: n // world] for t in ins])
                good = torch.equal(g.cpu(), wantg)
                ok = ok and good
                detail.append(("all_gather", str(dtype), n, 0, 0.0, good))
                r = eng.reduce_scatter(ins[rank].to(dev))
                torch.cuda.synchronize()
                per = n // world
                err = (r.float().cpu() - want[rank * per:(rank + 1) * per]).abs().max().item()
                good = err <= tol
                ok = ok and good
                detail.append(("reduce_scatter", str(dtype), n, 0, err, good))
    # asynchronous form on tensors of the caller's own, the last one in place: three buckets queued at once
    # on the engine's thread and stream, waited for out of order
    n3 = 98304
    xs3 = [[torch.randn(n3 * (k + 1), generator=torch.Generator().manual_seed(13 * r + k)).float() for r in range(world)] for k in range(3)]
    mine3 = [b[rank].to(dev) for b in xs3]
    outs3 = [torch.empty_like(mine3[0]), torch.empty_like(mine3[1]), mine3[2]]
    works = [eng.all_reduce_async(t, out=o) for t, o in zip(mine3, outs3)]
    good = True
    for k in (2, 0, 1):
        y = works[k].wait()
        torch.cuda.synchronize()
        good = good and y is outs3[k] and torch.allclose(y.cpu(), torch.stack(xs3[k]).sum(0), atol=1e-4 * world) and works[k].done()
    ok = ok and good
    detail.append(("all_reduce_async_x3", "f32", n3, 0, 0.0, good))
    status = eng.device_status()
    ok = ok and status[0] == 0
    bad = [d for d in detail if not d[-1]]
    print(json.dumps({"rank": rank, "world": world, "G": G, "ok": bool(ok), "checks": len(detail), "bad": bad[:6],
                      "nvls": bool(getattr(eng, "nvls", False)),
                      "device_status": status}), flush=True)
    eng.close()
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
