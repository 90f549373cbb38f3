"""The collective engine on the host-only library's stand-in device (test double).

`StandinEngine` is `HierarchicalEngine` with three substitutions: the native library
is `libtcpxb_host.so` started with TCPXB_FAKE_GPU=1 (device memory = host memory, the
kernels' CPU statement in csrc/kernels/kernels_host.cc), tensors live on the CPU, and
the intra-node "NVLink peer mappings" are files in /dev/shm that every rank of an
emulated node maps.  Everything else (rails, requests, scatter lists, ring schedule,
flag barriers) is the product's own C++ code, so these runs cover the engine's
orchestration on machines without a GPU.
"""
import ctypes
import os
from pathlib import Path

import torch

os.environ.setdefault("TCPXB_FAKE_GPU", "1")

from nccl_plugin_gpudirecttcpx_b200 import _build
from nccl_plugin_gpudirecttcpx_b200.parallel.engine import HierarchicalEngine, bind_engine_api

_api = None


def _host_api():
    global _api
    if _api is None:
        lib = os.environ.get("TCPXB_TEST_HOST_LIB") or str(_build.build_host())
        _api = bind_engine_api(ctypes.CDLL(lib, mode=ctypes.RTLD_GLOBAL))
    return _api


def _shared_int32(path: str, count: int, create: bool) -> torch.Tensor:
    if create:
        with open(path, "wb") as f:
            f.truncate(count * 4)
    return torch.from_file(path, shared=True, size=count, dtype=torch.int32)


class StandinEngine(HierarchicalEngine):
    def __init__(self, **kw):
        kw["device"] = torch.device("cpu")
        kw["use_nvls"] = False
        super().__init__(**kw)

    def _load_api(self):
        return _host_api()

    def _synchronize(self) -> None:
        pass  # the stand-in device runs everything at once on the calling thread

    def _stream(self):
        return None

    def _event_after_current_stream(self):
        return None, None  # the stand-in's streams run everything at once: nothing to wait for

    def _setup_symmetric(self, buffer_bytes: int, use_nvls: bool) -> None:
        dist = self._dist
        node = self.rank // self.G
        tag = [os.urandom(6).hex()]
        dist.broadcast_object_list(tag, src=0)
        n_el = (buffer_bytes + 3) // 4
        self.buffer_bytes = n_el * 4
        counts = {"work": n_el, "out": n_el, "flags": 64}
        shm_dir = os.environ.get("TCPXB_TEST_SHM_DIR", "/dev/shm")
        path = lambda r, name: f"{shm_dir}/tcpxb_{tag[0]}_{r}_{name}"
        mine = {name: _shared_int32(path(self.rank, name), c, create=True) for name, c in counts.items()}
        for t in mine.values():
            t.zero_()
        dist.barrier()
        maps = {name: [] for name in counts}
        for l in range(self.G):
            r = node * self.G + l
            for name, c in counts.items():
                maps[name].append(mine[name] if r == self.rank else _shared_int32(path(r, name), c, create=False))
        dist.barrier()
        for name in counts:  # the mappings stay; the names can go
            Path(path(self.rank, name)).unlink(missing_ok=True)
        self._keep = maps
        self.work, self.out = mine["work"], mine["out"]
        self.nvls = False
        arr = lambda ts: (ctypes.c_void_p * self.G)(*[t.data_ptr() for t in ts])
        self._check(self._api.tcpxb_engine_set_peers(self._h, arr(maps["work"]), arr(maps["out"]), arr(maps["flags"]),
                                                     None, self.buffer_bytes))
