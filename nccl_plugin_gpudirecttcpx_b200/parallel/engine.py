"""Python face of the hierarchical collective engine (csrc/engine/engine.cc).

One `HierarchicalEngine` per rank.  Ranks are grouped into emulated nodes of
`gpus_per_node` consecutive ranks; traffic between nodes goes through the
transport's sockets and is unpacked, reduced and fanned out to the local GPUs by
the sm_100a kernels, traffic inside a node uses NVLink peer mappings obtained from
torch symmetric memory.  With a single rank the engine is its own network peer (a
twin node holding the same data), so the whole path runs on one GPU.

torch.distributed is used for plumbing only: exchanging the 128-byte connect
handles and rendezvous of the symmetric buffers.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from ..utils import native

HANDLE_BYTES = 128
DTYPE_CODE = {torch.bfloat16: 1, torch.float32: 2}


class _Config(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in (
        "rank", "world", "gpus_per_node", "gpu_dev", "request_bytes", "max_inflight", "unpack_ctas",
        "reduce_impl", "use_nvls", "plain_mode", "idle_spin_us", "idle_sleep_us", "wake_on_events")]


class EngineStats(ctypes.Structure):
    _fields_ = [("bytes_sent", ctypes.c_uint64), ("bytes_received", ctypes.c_uint64),
                ("requests", ctypes.c_uint64), ("unpack_launches", ctypes.c_uint64),
                ("fragments", ctypes.c_uint64), ("kernel_launches", ctypes.c_uint64),
                ("seconds_net_wait", ctypes.c_double)] + [
                    (n, ctypes.c_double) for n in ("t_post_recv", "t_post_send", "t_test_recv", "t_launch",
                                                   "t_consume", "t_test_send", "t_idle", "t_sleep")] + [
                                                       ("sleeps", ctypes.c_uint64)] + [
                                                           (n, ctypes.c_double) for n in ("tx_idle", "tx_blocked", "rx_idle", "rx_blocked")]


_lib = None


def bind_engine_api(lib):
    """Declares the engine's C entry points on a loaded library and returns it."""
    vp, u64, ci = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int
    lib.tcpxb_engine_create.restype = vp
    lib.tcpxb_engine_create.argtypes = [ctypes.POINTER(_Config)]
    lib.tcpxb_engine_destroy.argtypes = [vp]
    lib.tcpxb_engine_rails.argtypes = [vp]
    lib.tcpxb_engine_listen.argtypes = [vp, vp]
    lib.tcpxb_engine_connect.argtypes = [vp, vp]
    lib.tcpxb_engine_set_peers.argtypes = [vp, vp, vp, vp, vp, u64]
    lib.tcpxb_engine_all_reduce.argtypes = [vp, vp, vp, u64, ci, vp]
    lib.tcpxb_engine_all_gather.argtypes = [vp, vp, vp, u64, vp]
    lib.tcpxb_engine_reduce_scatter.argtypes = [vp, vp, vp, u64, ci, vp]
    lib.tcpxb_engine_send_next.argtypes = [vp, vp, u64, vp]
    lib.tcpxb_engine_recv_prev.argtypes = [vp, vp, u64, vp]
    for name in ("tcpxb_engine_all_reduce_async", "tcpxb_engine_reduce_scatter_async"):
        getattr(lib, name).restype = u64
        getattr(lib, name).argtypes = [vp, vp, vp, u64, ci, vp]
    lib.tcpxb_engine_all_gather_async.restype = u64
    lib.tcpxb_engine_all_gather_async.argtypes = [vp, vp, vp, u64, vp]
    lib.tcpxb_engine_test.argtypes = [vp, u64, ctypes.POINTER(ci)]
    lib.tcpxb_engine_wait.argtypes = [vp, u64]
    lib.tcpxb_engine_stream_wait.argtypes = [vp, u64, vp]
    lib.tcpxb_engine_release.argtypes = [vp, u64]
    lib.tcpxb_engine_stats.argtypes = [vp, ctypes.POINTER(EngineStats)]
    lib.tcpxb_engine_device_status.argtypes = [vp, ctypes.POINTER(ctypes.c_uint32 * 4)]
    lib.tcpxb_engine_last_error.restype = ctypes.c_char_p
    return lib


def _e():
    global _lib
    if _lib is None:
        _lib = bind_engine_api(native.load("libnccl-net.so"))
    return _lib


from .plugin_env import LOOPBACK_SNDBUF, loopback_sndbuf  # noqa: E402,F401


def default_transport_env(nics: int = 4, nthreads: int = 4, nsocks_per_thread: int = 1,
                          chunk_bytes: int = 512 * 1024, pool_mb: int = 1024, sndbuf: int = -1) -> None:
    """Environment defaults for the transport under the engine (only where unset).  `sndbuf`: SO_SNDBUF of
    the data sockets; -1 = `loopback_sndbuf` for this box's cores per rank (affinity mask / LOCAL_WORLD_SIZE)."""
    if sndbuf < 0:
        sndbuf = loopback_sndbuf(len(os.sched_getaffinity(0)) // max(1, int(os.environ.get("LOCAL_WORLD_SIZE", "1"))))
    for k, v in {
        "NCCL_GPUDIRECTTCPX_SOCKET_SNDBUF": str(sndbuf),
        "NCCL_GPUDIRECTTCPX_SOCKET_IFNAME": "lo",
        "NCCL_GPUDIRECTTCPX_VIRTUAL_NICS": str(nics),
        "NCCL_SOCKET_NTHREADS": str(nthreads),
        "NCCL_NSOCKS_PERTHREAD": str(nsocks_per_thread),
        "NCCL_DYNAMIC_CHUNK_SIZE": str(chunk_bytes),
        "NCCL_GPUDIRECTTCPX_RX_POOL_BYTES": str(pool_mb << 20),
        "NCCL_GPUDIRECTTCPX_CUDA_BUFFERS": "1",
    }.items():
        os.environ.setdefault(k, v)


class AsyncWork:
    """A collective queued on the engine's own thread and stream (`all_reduce_async`).

    `wait()` blocks the calling host thread until the network part is over and the last
    kernel is queued, makes the caller's current stream wait for those kernels, and returns
    the result tensor.  `done()` polls without blocking.  Errors of the job surface here."""

    def __init__(self, engine: "HierarchicalEngine", ticket: int, result: torch.Tensor, keep=()):
        self._engine, self._ticket, self._result, self._keep = engine, ticket, result, keep

    def done(self) -> bool:
        if not self._ticket:
            return True  # already waited for
        flag = ctypes.c_int(0)
        self._engine._check(self._engine._api.tcpxb_engine_test(self._engine._h, self._ticket, ctypes.byref(flag)))
        return bool(flag.value)

    def wait(self) -> torch.Tensor:
        if self._ticket:
            eng = self._engine
            eng._check(eng._api.tcpxb_engine_wait(eng._h, self._ticket))
            eng._check(eng._api.tcpxb_engine_stream_wait(eng._h, self._ticket, eng._stream()))
            eng._check(eng._api.tcpxb_engine_release(eng._h, self._ticket))
            self._ticket = 0
            self._keep = ()
        return self._result


class HierarchicalEngine:
    """Collectives whose inter-node stage runs through the transport and whose receive
    side is the fused unpack kernel.  The plain calls are host-blocking and stream-ordered;
    `all_reduce_async` queues the same work on a thread and a stream of the engine's own."""

    def __init__(self, gpus_per_node: int = 1, buffer_bytes: int = 0, request_bytes: int = 1 << 20,
                 max_inflight: int = 4, unpack_ctas: int = 16, reduce_impl: int = 0, use_nvls: bool = False,
                 plain_mode: bool = False, device: Optional[torch.device] = None,
                 idle_spin_us: int = 0, idle_sleep_us: int = 0, wake_on_events: bool = False):
        import torch.distributed as dist
        self._api = self._load_api()
        self._dist = dist if dist.is_available() and dist.is_initialized() else None
        self.rank = self._dist.get_rank() if self._dist else 0
        self.world = self._dist.get_world_size() if self._dist else 1
        self.G = gpus_per_node
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.nodes = max(2, self.world // self.G) if self.world > 1 else 2
        cfg = _Config(self.rank, self.world, self.G, self.device.index or 0, request_bytes, max_inflight, unpack_ctas,
                      reduce_impl, int(use_nvls), int(plain_mode), idle_spin_us, idle_sleep_us, int(wake_on_events))
        self._h = self._api.tcpxb_engine_create(ctypes.byref(cfg))
        if not self._h:
            raise RuntimeError("engine create failed: " + self._api.tcpxb_engine_last_error().decode())
        self.rails = self._api.tcpxb_engine_rails(self._h)
        self._connect()
        self.work = self.out = None
        self._keep = []
        if self.G > 1:
            if buffer_bytes <= 0:
                raise ValueError("buffer_bytes is required when gpus_per_node > 1")
            self._setup_symmetric(buffer_bytes, use_nvls)

    # ------------------------------------------------------------------ set-up
    def _load_api(self):
        """The native library with the engine's entry points (the plugin, built for sm_100a)."""
        return _e()

    def _synchronize(self) -> None:
        torch.cuda.synchronize(self.device)

    def _check(self, rc: int) -> None:
        if rc != 0:
            raise RuntimeError("engine call failed: " + self._api.tcpxb_engine_last_error().decode())

    def _connect(self) -> None:
        mine = ctypes.create_string_buffer(self.rails * HANDLE_BYTES)
        self._check(self._api.tcpxb_engine_listen(self._h, mine))
        if self.world == 1:
            nxt = mine.raw
        else:
            allh = [None] * self.world
            self._dist.all_gather_object(allh, mine.raw)
            node, local = divmod(self.rank, self.G)
            nxt = allh[((node + 1) % (self.world // self.G)) * self.G + local]
        buf = ctypes.create_string_buffer(nxt, len(nxt))
        self._check(self._api.tcpxb_engine_connect(self._h, buf))

    def _setup_symmetric(self, buffer_bytes: int, use_nvls: bool) -> None:
        import torch.distributed._symmetric_memory as symm
        dist = self._dist
        node = self.rank // self.G
        group = None
        for n in range(self.world // self.G):
            g = dist.new_group(list(range(n * self.G, (n + 1) * self.G)))
            if n == node:
                group = g
        n_el = (buffer_bytes + 3) // 4
        self.buffer_bytes = n_el * 4
        bufs = {}
        for name, count in (("work", n_el), ("out", n_el), ("flags", 64)):
            t = symm.empty(count, dtype=torch.int32, device=self.device)
            t.zero_()
            hdl = symm.rendezvous(t, group=group)
            bufs[name] = (t, hdl)
        self._synchronize()
        dist.barrier(group)
        self._keep = bufs
        self.work = bufs["work"][0]
        self.out = bufs["out"][0]
        arr = lambda ptrs: (ctypes.c_void_p * self.G)(*[int(p) for p in ptrs])
        mc = 0
        if use_nvls:
            mc = int(getattr(bufs["out"][1], "multicast_ptr", 0) or 0)
        self.nvls = bool(mc)
        self._check(self._api.tcpxb_engine_set_peers(self._h, arr(bufs["work"][1].buffer_ptrs), arr(bufs["out"][1].buffer_ptrs),
                                                arr(bufs["flags"][1].buffer_ptrs), mc or None, self.buffer_bytes))

    # -------------------------------------------------------------- collectives
    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def _all_reduce_unit(self) -> int:
        """Byte granularity of the native all_reduce: every GPU's shard (and, on a ring of
        more than two nodes, every piece of it) is a whole number of 16-byte vectors."""
        return self.G * (self.nodes if self.nodes > 2 else 1) * 16

    def all_reduce(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Sum over all ranks, any number of elements (sizes that are not a multiple of the
        native granularity are zero-padded on the way in and trimmed on the way out).
        G == 1: any contiguous tensors.  G > 1: `x` is staged into the symmetric work buffer
        and the result is a view of the symmetric output."""
        nbytes = x.numel() * x.element_size()
        code = DTYPE_CODE[x.dtype]
        unit = self._all_reduce_unit()
        padded = (nbytes + unit - 1) // unit * unit
        if self.G == 1:
            if padded != nbytes:
                xin = torch.zeros(padded // x.element_size(), dtype=x.dtype, device=x.device)
                xin[:x.numel()].copy_(x.reshape(-1))
                res = torch.empty_like(xin)
                self._check(self._api.tcpxb_engine_all_reduce(self._h, xin.data_ptr(), res.data_ptr(), padded, code, self._stream()))
                res = res[:x.numel()].view(x.shape)
                if out is not None:
                    out.copy_(res)
                    return out
                return res
            if out is None:
                out = torch.empty_like(x)
            self._check(self._api.tcpxb_engine_all_reduce(self._h, x.data_ptr(), out.data_ptr(), nbytes, code, self._stream()))
            return out
        if padded > self.buffer_bytes:
            raise ValueError(f"all_reduce of {nbytes} bytes does not fit the {self.buffer_bytes}-byte symmetric buffers")
        if padded == nbytes and x.is_contiguous() and (out is None or out.is_contiguous()):
            # the native call stages tensors that live outside the symmetric buffers itself
            dst = out.data_ptr() if out is not None else self.out.data_ptr()
            self._check(self._api.tcpxb_engine_all_reduce(self._h, x.data_ptr(), dst, nbytes, code, self._stream()))
            return out if out is not None else self.out.view(torch.uint8)[:nbytes].view(x.dtype).view(x.shape)
        wb = self.work.view(torch.uint8)
        w = wb[:nbytes].view(x.dtype)
        if x.data_ptr() != w.data_ptr():
            w.copy_(x.reshape(-1))
        if padded != nbytes:
            wb[nbytes:padded].zero_()
        self._check(self._api.tcpxb_engine_all_reduce(self._h, self.work.data_ptr(), self.out.data_ptr(), padded, code, self._stream()))
        res = self.out.view(torch.uint8)[:nbytes].view(x.dtype).view(x.shape)
        if out is not None:
            out.copy_(res)
            return out
        return res

    def _event_after_current_stream(self):
        """A CUDA event at the current point of the caller's stream: (object to keep alive, raw handle)."""
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        return ev, ev.cuda_event

    def all_reduce_async(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> AsyncWork:
        """`all_reduce` without blocking the caller: the engine's own thread drives the network
        and queues the kernels on the engine's own stream, after everything the caller's current
        stream holds at the time of the call.  Several calls may be outstanding; they run in
        order.  `x` must be contiguous with a size that is a multiple of the native granularity
        (32 bytes between two single-GPU nodes) and must stay untouched until `wait()`; `out`
        may be `x`.  With several GPUs per node the job stages `x` and `out` through the
        symmetric buffers itself; without `out` the result is a view of the symmetric output,
        which the next call overwrites."""
        nbytes = x.numel() * x.element_size()
        code = DTYPE_CODE[x.dtype]
        unit = self._all_reduce_unit()
        if nbytes % unit != 0 or not x.is_contiguous() or (out is not None and not out.is_contiguous()):
            raise ValueError(f"all_reduce_async needs contiguous tensors whose size is a multiple of {unit} bytes")
        if self.G == 1:
            res = out if out is not None else torch.empty_like(x)
            src, dst = x.data_ptr(), res.data_ptr()
        else:
            if nbytes > self.buffer_bytes:
                raise ValueError(f"all_reduce of {nbytes} bytes does not fit the {self.buffer_bytes}-byte symmetric buffers")
            res = out if out is not None else self.out.view(torch.uint8)[:nbytes].view(x.dtype).view(x.shape)
            src, dst = x.data_ptr(), res.data_ptr()
        keep, after = self._event_after_current_stream()
        ticket = self._api.tcpxb_engine_all_reduce_async(self._h, src, dst, nbytes, code, after)
        if not ticket:
            raise RuntimeError("engine call failed: " + self._api.tcpxb_engine_last_error().decode())
        return AsyncWork(self, ticket, res, keep=(keep, x, res))

    def all_gather_async(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> AsyncWork:
        """`all_gather` on the engine's own thread and stream.  `x` contiguous, its byte size a multiple
        of 16.  With one GPU per node `out` (world x x.numel() elements) may be given; with several the
        result is a view of the symmetric output buffer, so one such job may be outstanding at a time."""
        nbytes = x.numel() * x.element_size()
        blocks = self.nodes * self.G
        if nbytes % 16 != 0 or not x.is_contiguous():
            raise ValueError("all_gather_async needs a contiguous block whose size is a multiple of 16 bytes")
        if self.G == 1:
            res = out if out is not None else torch.empty(blocks * x.numel(), dtype=x.dtype, device=x.device)
            if res.numel() * res.element_size() != blocks * nbytes or not res.is_contiguous():
                raise ValueError(f"out must be contiguous and hold {blocks} blocks of {nbytes} bytes")
            dst = res.data_ptr()
        else:
            if out is not None:
                raise ValueError("with several GPUs per node the result lives in the symmetric output buffer")
            if nbytes * blocks > self.buffer_bytes:
                raise ValueError(f"all_gather of {blocks} x {nbytes} bytes does not fit the {self.buffer_bytes}-byte symmetric buffers")
            res = self.out.view(torch.uint8)[:nbytes * blocks].view(x.dtype)
            dst = self.out.data_ptr()
        keep, after = self._event_after_current_stream()
        ticket = self._api.tcpxb_engine_all_gather_async(self._h, x.data_ptr(), dst, nbytes, after)
        if not ticket:
            raise RuntimeError("engine call failed: " + self._api.tcpxb_engine_last_error().decode())
        return AsyncWork(self, ticket, res, keep=(keep, x, res))

    def reduce_scatter_async(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> AsyncWork:
        """`reduce_scatter` on the engine's own thread and stream.  `x` contiguous, divisible into one part
        per rank whose byte size is a multiple of 16.  With several GPUs per node `x` is copied into the
        symmetric work buffer at once (unless it already is that buffer), so one such job may be
        outstanding at a time."""
        blocks = self.nodes * self.G if self.world > 1 else 1
        if x.numel() % blocks != 0 or not x.is_contiguous():
            raise ValueError(f"reduce_scatter_async needs a contiguous input that divides into {blocks} parts")
        per = x.numel() // blocks
        nbytes = per * x.element_size()
        if nbytes % 16 != 0:
            raise ValueError("reduce_scatter_async needs parts whose size is a multiple of 16 bytes")
        res = out if out is not None else torch.empty(per, dtype=x.dtype, device=x.device)
        if res.numel() != per or res.dtype != x.dtype or not res.is_contiguous():
            raise ValueError(f"out must be a contiguous tensor of {per} elements of {x.dtype}")
        src = x
        if self.G > 1:
            total = x.numel() * x.element_size()
            if total > self.buffer_bytes:
                raise ValueError(f"reduce_scatter input of {total} bytes does not fit the symmetric buffers")
            w = self.work.view(torch.uint8)[:total].view(x.dtype)
            if x.data_ptr() != w.data_ptr():
                w.copy_(x.reshape(-1))
            src = self.work
        keep, after = self._event_after_current_stream()
        ticket = self._api.tcpxb_engine_reduce_scatter_async(self._h, src.data_ptr(), res.data_ptr(), nbytes, DTYPE_CODE[x.dtype], after)
        if not ticket:
            raise RuntimeError("engine call failed: " + self._api.tcpxb_engine_last_error().decode())
        return AsyncWork(self, ticket, res, keep=(keep, x, res))

    def work_view(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """The symmetric work buffer as a tensor, for producers that write in place."""
        return self.work.view(torch.uint8)[:numel * dtype.itemsize].view(dtype)

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        """Concatenation of every rank's `x` in rank order.  Blocks whose byte size is not a
        multiple of 16 travel padded and are compacted on return."""
        nbytes = x.numel() * x.element_size()
        blocks = self.nodes * self.G
        if nbytes % 16 != 0:
            padded = (nbytes + 15) // 16 * 16
            xin = torch.zeros(padded, dtype=torch.uint8, device=x.device)
            xin[:nbytes].copy_(x.reshape(-1).view(torch.uint8))
            g = self.all_gather(xin)
            return g.view(blocks, padded)[:, :nbytes].contiguous().view(-1).view(x.dtype)
        if self.G == 1:
            out = torch.empty(blocks * x.numel(), dtype=x.dtype, device=x.device)
            self._check(self._api.tcpxb_engine_all_gather(self._h, x.data_ptr(), out.data_ptr(), nbytes, self._stream()))
            return out
        if nbytes * blocks > self.buffer_bytes:
            raise ValueError(f"all_gather of {blocks} x {nbytes} bytes does not fit the {self.buffer_bytes}-byte symmetric buffers")
        self._check(self._api.tcpxb_engine_all_gather(self._h, x.data_ptr(), self.out.data_ptr(), nbytes, self._stream()))
        return self.out.view(torch.uint8)[:nbytes * blocks].view(x.dtype)

    def reduce_scatter(self, x: torch.Tensor) -> torch.Tensor:
        """Sum over all ranks of `x`, of which this rank keeps its 1/world part (`x.numel()`
        must divide by the number of ranks).  Parts whose byte size is not a multiple of 16
        travel padded."""
        blocks = self.nodes * self.G if self.world > 1 else 1
        if x.numel() % blocks != 0:
            raise ValueError(f"reduce_scatter input of {x.numel()} elements does not divide into {blocks} parts")
        per = x.numel() // blocks
        nbytes = per * x.element_size()
        if nbytes % 16 != 0:
            per_padded = (nbytes + 15) // 16 * 16 // x.element_size()
            xin = torch.zeros(blocks, per_padded, dtype=x.dtype, device=x.device)
            xin[:, :per].copy_(x.reshape(blocks, per))
            return self.reduce_scatter(xin.view(-1))[:per].clone()
        out = torch.empty(per, dtype=x.dtype, device=x.device)
        src = x
        if self.G > 1:
            if x.numel() * x.element_size() > self.buffer_bytes:
                raise ValueError(f"reduce_scatter input of {x.numel() * x.element_size()} bytes does not fit the symmetric buffers")
            w = self.work.view(torch.uint8)[:x.numel() * x.element_size()].view(x.dtype)
            if x.data_ptr() != w.data_ptr():
                w.copy_(x.reshape(-1))
            src = self.work
        self._check(self._api.tcpxb_engine_reduce_scatter(self._h, src.data_ptr(), out.data_ptr(), nbytes, DTYPE_CODE[x.dtype], self._stream()))
        return out

    def send_next(self, x: torch.Tensor) -> None:
        self._check(self._api.tcpxb_engine_send_next(self._h, x.data_ptr(), x.numel() * x.element_size(), self._stream()))

    def recv_prev(self, x: torch.Tensor) -> None:
        self._check(self._api.tcpxb_engine_recv_prev(self._h, x.data_ptr(), x.numel() * x.element_size(), self._stream()))

    # -------------------------------------------------------------------- misc
    def stats(self) -> EngineStats:
        s = EngineStats()
        self._api.tcpxb_engine_stats(self._h, ctypes.byref(s))
        return s

    def device_status(self):
        w = (ctypes.c_uint32 * 4)()
        self._api.tcpxb_engine_device_status(self._h, ctypes.byref(w))
        return list(w)

    def close(self) -> None:
        if self._h:
            self._synchronize()
            self._api.tcpxb_engine_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
