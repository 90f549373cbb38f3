"""Worker for the CPU engine tests: gloo ranks, the engine on the stand-in device.

Ranks form `world / G` emulated nodes of G "GPUs".  Every rank rebuilds every rank's
seeded input and checks its results against a plain PyTorch fp32 sum.  Modes
(TCPXB_TEST_MODE): `collectives` (default) and `rank_leaves`, in which the last rank
exits between two steps and the others must get an error, not a hang.
"""
import faulthandler
import json
import os
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
sys.path.insert(0, str(Path(__file__).resolve().parent))

import torch
import torch.distributed as dist


def main():
    faulthandler.dump_traceback_later(int(os.environ.get("TCPXB_TEST_DUMP_AFTER", "150")), exit=True)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    G = int(os.environ.get("TCPXB_TEST_GPUS_PER_NODE", "1"))
    mode = os.environ.get("TCPXB_TEST_MODE", "collectives")
    if world > 1:
        dist.init_process_group("gloo")
    from nccl_plugin_gpudirecttcpx_b200.parallel.engine import default_transport_env
    from standin_engine import StandinEngine
    default_transport_env(nics=2, nthreads=2, nsocks_per_thread=1, pool_mb=64, chunk_bytes=128 * 1024)
    numels = [int(s) for s in os.environ.get("TCPXB_TEST_NUMELS", "3072,786432").split(",")]
    buf_bytes = max(max(numels), 1000003 + 64) * 4  # the largest case in fp32, padding included
    eng = StandinEngine(gpus_per_node=G, buffer_bytes=buf_bytes if G > 1 else 0, request_bytes=256 << 10,
                        plain_mode=bool(int(os.environ.get("TCPXB_TEST_PLAIN", "0"))),
                        reduce_impl=int(os.environ.get("TCPXB_TEST_REDUCE_IMPL", "0")),
                        idle_sleep_us=int(os.environ.get("TCPXB_TEST_IDLE_SLEEP_US", "0")),
                        wake_on_events=bool(int(os.environ.get("TCPXB_TEST_WAKE_ON_EVENTS", "0"))))
    ranks = world if world > 1 else 2  # a single rank is its own twin

    if mode == "rank_leaves":
        x = torch.ones(98304, dtype=torch.float32)  # a multiple of every layout's unit
        y = eng.all_reduce(x)
        first_ok = bool(torch.all(y == ranks).item())
        dist.barrier()  # a step boundary: nothing is in flight
        if rank == world - 1:
            print(json.dumps({"rank": rank, "left": True, "first_ok": first_ok}), flush=True)
            os._exit(0)  # no clean shutdown: the process is simply gone
        time.sleep(0.5)
        t0 = time.time()
        outcome = "completed"
        try:
            if os.environ.get("TCPXB_TEST_ASYNC") == "1":
                eng.all_reduce_async(x, out=torch.empty_like(x)).wait()  # the job's error surfaces at the join
            else:
                eng.all_reduce(x)
            if eng.device_status()[0] != 0:
                outcome = "device_status"
        except RuntimeError as e:
            outcome = "error: " + str(e)[:120]
        print(json.dumps({"rank": rank, "left": False, "first_ok": first_ok, "outcome": outcome,
                          "seconds": round(time.time() - t0, 2), "device_status": eng.device_status()}), flush=True)
        os._exit(0)

    ok = True
    detail = []
    for dtype in (torch.bfloat16, torch.float32):
        for n in numels:
            ins = [torch.randn(n, generator=torch.Generator().manual_seed(100 * r + n % 911)).to(dtype) for r in range(world)]
            if world == 1:
                ins = ins * 2
            want = torch.stack([t.float() for t in ins]).sum(0)
            tol = 0.04 * ranks if dtype == torch.bfloat16 else 1e-4 * ranks
            for rep in range(2):  # twice: buffers and flag epochs are reused
                y = eng.all_reduce(ins[rank].clone())
                diff = (y.float() - want).abs()
                err = diff.max().item()
                good = err <= tol
                ok = ok and good
                where = ""
                if not good:  # which elements, and do they heal once every rank is past the step
                    badix = (diff > tol).nonzero().flatten()
                    time.sleep(1.0)
                    later = ((y.float() - want).abs() > tol).sum().item()
                    where = f"{badix.numel()} bad in [{badix[0].item()}, {badix[-1].item()}], {later} still bad a second later"
                detail.append(("all_reduce", str(dtype), n, rep, err, good, where) if where else ("all_reduce", str(dtype), n, rep, err, good))
            if n % ranks == 0:
                per = n // ranks
                g = eng.all_gather(ins[rank][:per].clone())
                wantg = torch.cat([t[:per] for t in ins])
                good = torch.equal(g.clone(), wantg)
                ok = ok and good
                detail.append(("all_gather", str(dtype), n, 0, 0.0, good))
                src = ins[rank].clone() if world > 1 else ins[0][:per].clone()
                r = eng.reduce_scatter(src)
                wantr = want[rank * per:(rank + 1) * per] if world > 1 else 2 * ins[0][:per].float()
                err = (r.float() - wantr).abs().max().item()
                good = err <= tol
                ok = ok and good
                detail.append(("reduce_scatter", str(dtype), n, 0, err, good))
    # sizes that are no multiple of the native granularity are padded inside the binding
    for n in (1, 1000003):
        xs = [torch.randn(n, generator=torch.Generator().manual_seed(7 * r + n)).float() for r in range(world)]
        if world == 1:
            xs = xs * 2
        y = eng.all_reduce(xs[rank].clone())
        good = tuple(y.shape) == (n,) and torch.allclose(y, torch.stack(xs).sum(0), atol=1e-4 * ranks)
        ok = ok and good
        detail.append(("all_reduce_odd", "f32", n, 0, 0.0, good))
    if True:
        # in place (out is the input tensor); with several GPUs per node the native call stages it through the symmetric buffers
        xs = [torch.randn(600000, generator=torch.Generator().manual_seed(3 * r + 1)).float() for r in range(world)]
        if world == 1:
            xs = xs * 2
        mine = xs[rank].clone()
        y = eng.all_reduce(mine, mine)
        good = y is mine and torch.allclose(mine, torch.stack(xs).sum(0), atol=1e-4 * ranks)
        ok = ok and good
        detail.append(("all_reduce_in_place", "f32", 600000, 0, 0.0, good))
    if True:
        # asynchronous form: three buckets queued at once on the engine's thread, waited for out of order
        xs3 = [[torch.randn(98304 * (k + 1), generator=torch.Generator().manual_seed(13 * r + k)).float() for r in range(world)]
               for k in range(3)]
        if world == 1:
            xs3 = [b * 2 for b in xs3]
        mine3 = [b[rank].clone() for b in xs3]
        works = [eng.all_reduce_async(t, out=torch.empty_like(t)) for t in mine3]  # own outputs: several jobs are outstanding
        good = True
        for k in (2, 0, 1):
            y = works[k].wait()
            good = good and torch.allclose(y, torch.stack(xs3[k]).sum(0), atol=1e-4 * ranks) and works[k].done()
        ok = ok and good
        detail.append(("all_reduce_async_x3", "f32", 98304, 0, 0.0, good))
    # asynchronous all_gather and reduce_scatter: one job of each at a time (with several GPUs per node their
    # buffers are the symmetric ones), the reduce_scatter queued behind the all_gather
    per = 4096
    xs = [torch.randn(per * ranks, generator=torch.Generator().manual_seed(17 * r + 3)).float() for r in range(world)]
    if world == 1:
        xs = xs * 2
    wg = eng.all_gather_async(xs[rank][:per].clone())
    g = wg.wait().clone()
    good = torch.equal(g, torch.cat([t[:per] for t in xs])) and wg.done()
    if world > 1:
        wr = eng.reduce_scatter_async(xs[rank].clone())
        r_ = wr.wait()
        good = good and torch.allclose(r_, torch.stack(xs).sum(0)[rank * per:(rank + 1) * per], atol=1e-4 * ranks)
    ok = ok and good
    detail.append(("all_gather_reduce_scatter_async", "f32", per, 0, 0.0, good))
    # all_gather and reduce_scatter blocks that are no multiple of 16 bytes
    per = 1001
    xs = [torch.randn(per * ranks, generator=torch.Generator().manual_seed(11 * r + 5)).float() for r in range(world)]
    if world == 1:
        xs = xs * 2
    g = eng.all_gather(xs[rank][:per].clone())
    good = torch.equal(g.clone(), torch.cat([t[:per] for t in xs]))
    ok = ok and good
    detail.append(("all_gather_odd", "f32", per, 0, 0.0, good))
    if world > 1:
        r = eng.reduce_scatter(xs[rank].clone())
        wantr = torch.stack(xs).sum(0)[rank * per:(rank + 1) * per]
    else:
        r = eng.reduce_scatter(xs[0][:per].clone())
        wantr = 2 * xs[0][:per]
    good = tuple(r.shape) == (per,) and torch.allclose(r, wantr, atol=1e-4 * ranks)
    ok = ok and good
    detail.append(("reduce_scatter_odd", "f32", per, 0, 0.0, good))
    if world > 1 and G == 1:
        # point to point around the ring of nodes
        msg = torch.full((100000,), float(rank), dtype=torch.float32)
        got = torch.empty_like(msg)
        if rank % 2 == 0:
            eng.send_next(msg); eng.recv_prev(got)
        else:
            eng.recv_prev(got); eng.send_next(msg)
        good = bool(torch.all(got == float((rank - 1) % world)).item())
        ok = ok and good
        detail.append(("send_recv", "f32", 100000, 0, 0.0, good))
    status = eng.device_status()
    ok = ok and status[0] == 0
    st = eng.stats()
    bad = [d for d in detail if not d[5]]
    print(json.dumps({"rank": rank, "world": world, "G": G, "ok": bool(ok), "checks": len(detail), "bad": bad[:6],
                      "device_status": status, "unpack_launches": st.unpack_launches, "fragments": st.fragments}), flush=True)
    eng.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
