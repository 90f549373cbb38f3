"""Data-parallel training step through torch.distributed with the plugin loaded.

  python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
      -m nccl_plugin_gpudirecttcpx_b200.parallel.ddp --transport plugin --gpus-per-node 4

Ranks are split into emulated nodes with NCCL_HOSTID, so NCCL keeps NVLink inside a
node and sends the inter-node part of every gradient all_reduce through the net
transport: this plugin (`plugin`: host buffers; `unpack`: NCCL's kernels unpack from
the rx page pool) or NCCL's own socket transport (`socket`, the baseline, with the
same thread / socket / chunk settings).  `engine` keeps NCCL for set-up only and
reduces every gradient bucket through the hierarchical engine (fused unpack + reduce +
NVLink fan-out kernels) from a DDP communication hook; the hook queues buckets on the
engine's own thread and stream (`all_reduce_async`), so backward keeps running while
buckets are on the wire.  Model, optimizer and bucketing are stock
PyTorch: Llama-style decoder, AdamW, DistributedDataParallel with 25 MB buckets
overlapped with backward.  Synthetic uniform token ids, random-init weights.
Rank 0 prints one JSON line with the device-timed step time (max over ranks).
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def parse_args(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--transport", default="plugin", choices=["plugin", "unpack", "socket", "nvlink", "engine"])
    ap.add_argument("--engine-class", default="nccl_plugin_gpudirecttcpx_b200.parallel.engine:HierarchicalEngine",
                    help="module:Class of the engine behind --transport engine")
    ap.add_argument("--gpus-per-node", type=int, default=4)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--micro-batch", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--bucket-mb", type=int, default=25)
    ap.add_argument("--tiny", action="store_true", help="2-layer toy model (tests)")
    ap.add_argument("--backend", default="nccl", choices=["nccl", "gloo"])
    ap.add_argument("--nics", type=int, default=4)
    ap.add_argument("--nthreads", type=int, default=4)
    ap.add_argument("--engine-buffer-kb", type=int, default=0,
                    help="--transport engine, several GPUs per node: size of the symmetric buffers (0 = bucket cap + largest parameter); larger buckets travel in pieces")
    return ap.parse_args(argv)


def setup_env(args, rank: int) -> None:
    """Must run before NCCL is initialised."""
    if args.backend != "nccl":
        return
    from .plugin_env import plugin_env
    if args.transport in ("nvlink", "engine"):
        return  # one real node for NCCL: its own intra-node transports, no emulation
    env = plugin_env(nics=args.nics, nthreads=args.nthreads, builtin_socket=(args.transport == "socket"),
                     recv_mode="unpack" if args.transport == "unpack" else "host")
    # nodes are told apart by host id, so P2P and SHM stay on inside a node
    env.pop("NCCL_P2P_DISABLE", None)
    env.pop("NCCL_SHM_DISABLE", None)
    env["NCCL_HOSTID"] = f"tcpxb-node-{rank // args.gpus_per_node}"
    os.environ.update(env)


class EngineBucketReducer:
    """Averages DDP's gradient buckets through the hierarchical engine.

    The hook queues each bucket, in place, on the engine's own thread and stream
    (`all_reduce_async`, ordered behind the point backward has reached on the current
    stream) and returns a future at once, so backward keeps running while buckets are on
    the wire and several buckets can be queued.  A small waiter thread only turns finished
    jobs into completed futures, in order: it joins the job, scales the bucket on a side
    stream that waits for the engine's kernels, and completes the future (which carries
    that stream's event on CUDA)."""

    def __init__(self, engine, ranks: int, device):
        import queue
        import threading
        import torch
        self.engine, self.ranks, self.device = engine, ranks, device
        self.cuda = device.type == "cuda"
        self.stream = torch.cuda.Stream(device=device) if self.cuda else None
        self.buckets = 0
        self._unit = engine._all_reduce_unit()
        self._q = queue.Queue()
        self._thread = threading.Thread(target=self._complete, name="tcpxb-ddp", daemon=True)
        self._thread.start()

    def hook(self, _state, bucket):
        import torch
        buf = bucket.buffer()
        fut = torch.futures.Future(devices=[self.device]) if self.cuda else torch.futures.Future()
        try:
            flat = buf.reshape(-1) if buf.is_contiguous() else None
            if flat is None:
                raise ValueError("DDP handed over a bucket that is not contiguous")
            # A bucket may be larger than the engine's symmetric buffers (DDP's first step reduces
            # all gradients as one bucket before it has rebuilt its buckets): it travels in pieces.
            cap = getattr(self.engine, "buffer_bytes", 0) if self.engine.G > 1 else 0
            piece_elems = flat.numel() if cap <= 0 else max(self._unit, cap // self._unit * self._unit) // flat.element_size()
            jobs = []
            for lo in range(0, flat.numel(), piece_elems):
                piece = flat[lo:lo + piece_elems]
                nbytes = piece.numel() * piece.element_size()
                staged = None
                if nbytes % self._unit != 0:
                    # off the native granularity: travel zero-padded in a tensor of the job's own
                    padded = (nbytes + self._unit - 1) // self._unit * self._unit
                    staged = torch.zeros(padded // piece.element_size(), dtype=piece.dtype, device=piece.device)
                    staged[:piece.numel()].copy_(piece)
                t = staged if staged is not None else piece
                jobs.append((self.engine.all_reduce_async(t, out=t), piece, staged))
            self._q.put((jobs, buf, fut))
        except Exception as e:
            fut.set_exception(e)
        return fut

    def _finish(self, jobs, buf):
        for work, piece, staged in jobs:
            res = work.wait()  # the current stream now waits for the engine's kernels
            if staged is not None:
                piece.copy_(res[:piece.numel()])
        buf.div_(self.ranks)
        self.buckets += 1

    def _complete(self):
        import torch
        if self.cuda:
            torch.cuda.set_device(self.device)
        while True:
            item = self._q.get()
            if item is None:
                return
            jobs, buf, fut = item
            try:
                if self.cuda:
                    with torch.cuda.stream(self.stream):
                        self._finish(jobs, buf)
                        fut.set_result(buf)   # records this stream's event for whoever waits
                else:
                    self._finish(jobs, buf)
                    fut.set_result(buf)
            except Exception as e:  # the training thread gets the error from the future
                fut.set_exception(e)

    def close(self):
        self._q.put(None)
        self._thread.join(timeout=30)
        self.engine.close()


def make_engine_reducer(args, dev, world: int, model):
    """Engine sized for the largest bucket DDP can form: the cap plus one whole parameter."""
    import importlib
    from .engine import default_transport_env
    mod, _, cls = args.engine_class.partition(":")
    engine_cls = getattr(importlib.import_module(mod), cls)
    default_transport_env(nics=args.nics, nthreads=args.nthreads)
    G = args.gpus_per_node if world > 1 else 1
    largest = max(p.numel() * p.element_size() for p in model.parameters())
    buffer_bytes = ((args.bucket_mb << 20) + largest + (1 << 20) - 1) >> 20 << 20
    if args.engine_buffer_kb > 0:
        buffer_bytes = args.engine_buffer_kb << 10
    eng = engine_cls(gpus_per_node=G, buffer_bytes=buffer_bytes if G > 1 else 0, device=dev)
    return EngineBucketReducer(eng, world if world > 1 else 2, dev)


def main(argv=None) -> int:
    args = parse_args(argv)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    setup_env(args, rank)

    import torch
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as DDP

    from ..models import LlamaConfig, LlamaDecoder

    use_cuda = args.backend == "nccl"
    if use_cuda:
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    torch.manual_seed(1234)  # same initial weights everywhere
    cfg = LlamaConfig.tiny() if args.tiny else LlamaConfig()
    dtype = torch.bfloat16 if use_cuda else torch.float32
    model = LlamaDecoder(cfg).to(device=dev, dtype=dtype)
    ddp = DDP(model, device_ids=[local] if use_cuda else None, bucket_cap_mb=args.bucket_mb, gradient_as_bucket_view=True)
    reducer = None
    if args.transport == "engine":
        reducer = make_engine_reducer(args, dev, world, model)
        ddp.register_comm_hook(None, reducer.hook)
    opt = torch.optim.AdamW(ddp.parameters(), lr=1e-4, weight_decay=0.1, fused=use_cuda)
    seq = min(args.seq_len, 64) if args.tiny else args.seq_len
    gen = torch.Generator(device=dev).manual_seed(99 + rank)

    def step():
        tokens = torch.randint(0, cfg.vocab_size, (args.micro_batch, seq + 1), device=dev, generator=gen)
        loss = ddp(tokens[:, :-1], tokens[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    losses = []
    for _ in range(args.warmup):
        losses.append(step().item())
    dist.barrier()
    if use_cuda:
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    else:
        import time
        t0 = time.time()
    for _ in range(args.steps):
        loss = step()
    if use_cuda:
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
    else:
        ms = (time.time() - t0) * 1e3 / args.steps
    losses.append(loss.item())
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    # replicas must agree after the same updates
    w = next(model.parameters()).detach().float().flatten()[:1024].clone()
    w_ref = w.clone()
    dist.broadcast(w_ref, 0)
    in_sync = bool(torch.allclose(w, w_ref))
    if rank == 0:
        n_params = model.num_parameters()
        tokens_per_step = world * args.micro_batch * seq
        print(json.dumps({
            "bench": "ddp_llama_step", "transport": args.transport, "world": world, "gpus_per_node": args.gpus_per_node,
            "ms_per_step": t.item(), "tokens_per_s": tokens_per_step / (t.item() * 1e-3), "params": n_params,
            "grad_bytes_per_step": n_params * (2 if use_cuda else 4), "bucket_mb": args.bucket_mb,
            "micro_batch": args.micro_batch, "seq_len": seq, "loss_first": losses[0], "loss_last": losses[-1],
            "replicas_in_sync": in_sync, "dtype": str(dtype), "data": "synthetic uniform token ids, random init",
            "engine_buckets": reducer.buckets if reducer else None,
        }), flush=True)
    if reducer is not None:
        if use_cuda:
            torch.cuda.synchronize()
        reducer.close()
    dist.barrier()
    dist.destroy_process_group()
    return 0 if in_sync else 1


if __name__ == "__main__":
    sys.exit(main())
