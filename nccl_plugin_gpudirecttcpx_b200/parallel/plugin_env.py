"""Environment that makes NCCL (and therefore torch.distributed) load the plugin and
push traffic between GPUs of one box through it.

A single 8-GPU box has no inter-node network, so "nodes" are emulated: NCCL's
peer-to-peer and shared-memory transports are disabled between the ranks that
should talk over the network, which leaves the net transport, and the plugin is
given `nics` virtual devices on the loopback interface.  The same generic socket
variables (NCCL_SOCKET_NTHREADS, NCCL_NSOCKS_PERTHREAD, NCCL_DYNAMIC_CHUNK_SIZE)
steer both this plugin and NCCL's own socket transport, so a fair comparison pins
them identically for both; `plugin_env(..., builtin_socket=True)` returns the
baseline variant of the same environment.
"""
from __future__ import annotations

import os
from typing import Dict, Optional

from ..utils import native


LOOPBACK_SNDBUF = 256 * 1024


def loopback_sndbuf(cores_per_rank: int) -> int:
    """SO_SNDBUF for data sockets over loopback on a box with this many cores per rank (0 = the
    kernel's auto-tuning).  Over loopback there is no bandwidth-delay product to cover, and with
    auto-tuning each stream parks megabytes of skbs inside the kernel that have left the caches by
    the time the receiver copies them out.  Where the cores are the limit a bounded buffer pays:
    4 ranks with 4 cores each, 256 MiB all_reduce, 17.6 - 18.5 ms per step with 128 - 384 KiB
    against 20.9 ms with auto-tuning; with 8 cores per rank 17.3 against 18.0.  Where cores are
    plentiful the deeper queue wins: 2 ranks with 16 cores each 15.4 ms against 13.3."""
    return LOOPBACK_SNDBUF if cores_per_rank <= 8 else 0


def socket_settings_for(cores: int, ranks_on_box: int) -> Dict[str, int]:
    """Helper threads per connection and chunk size for a box with `cores` CPU cores shared by
    `ranks_on_box` ranks.  From the measurements on 16- to 32-core boxes: with six or more cores per
    rank four threads and 512 KiB chunks are fastest; with fewer, two threads and 128 KiB chunks
    (more threads only take cores from the kernel's TCP work)."""
    per_rank = max(1, cores // max(1, ranks_on_box))
    if per_rank >= 6:
        return {"nthreads": 4, "chunk_bytes": 512 * 1024}
    return {"nthreads": 2, "chunk_bytes": 128 * 1024}


def plugin_env(nics: int = 4, nsocks_per_thread: int = 1, nthreads: int = 4, chunk_bytes: int = 512 * 1024,
               recv_mode: str = "host", rx_pool_mode: str = "host", rx_pool_mb: int = 1024,
               gdr: bool = False, builtin_socket: bool = False, speed_mbps: int = 200000,
               debug: Optional[str] = None, extra: Optional[Dict[str, str]] = None,
               sndbuf: int = -1, max_channels: int = -1) -> Dict[str, str]:
    """`nthreads=0` or `chunk_bytes=0` asks for the values `socket_settings_for` gives this box
    (core count from the affinity mask, ranks from LOCAL_WORLD_SIZE).  `sndbuf`: SO_SNDBUF of the
    plugin's data sockets (0 = the kernel's auto-tuning, -1 = 256 KiB up to eight cores per rank).  `max_channels`: NCCL_MAX_NCHANNELS /
    NCCL_MIN_NCHANNELS; -1 = 4 when the box has fewer than six cores per rank, otherwise NCCL's choice."""
    per_rank_cores = len(os.sched_getaffinity(0)) // max(1, int(os.environ.get("LOCAL_WORLD_SIZE", "1")))
    if sndbuf < 0:
        sndbuf = loopback_sndbuf(per_rank_cores)
    if nthreads <= 0 or chunk_bytes <= 0:
        auto = socket_settings_for(len(os.sched_getaffinity(0)), int(os.environ.get("LOCAL_WORLD_SIZE", "1")))
        nthreads = nthreads if nthreads > 0 else auto["nthreads"]
        chunk_bytes = chunk_bytes if chunk_bytes > 0 else auto["chunk_bytes"]
    env = {
        # every GPU is its own "node": nothing but the net transport is left
        "NCCL_P2P_DISABLE": "1",
        "NCCL_SHM_DISABLE": "1",
        "NCCL_IB_DISABLE": "1",
        "NCCL_SOCKET_IFNAME": "lo",
        "NCCL_SOCKET_NTHREADS": str(nthreads),
        "NCCL_NSOCKS_PERTHREAD": str(nsocks_per_thread),
        "NCCL_DYNAMIC_CHUNK_SIZE": str(chunk_bytes),
    }
    if builtin_socket:
        env["NCCL_NET"] = "Socket"
        env["NCCL_NET_PLUGIN"] = "none"
    else:
        lib = native.plugin_path()
        if not lib.exists():
            native.load("libnccl-net.so")
        env.update({
            "NCCL_NET_PLUGIN": str(lib),
            "LD_LIBRARY_PATH": f"{lib.parent}:{os.environ.get('LD_LIBRARY_PATH', '')}",
            "NCCL_GPUDIRECTTCPX_SOCKET_IFNAME": "lo",
            "NCCL_GPUDIRECTTCPX_VIRTUAL_NICS": str(nics),
            "NCCL_GPUDIRECTTCPX_RECV_MODE": recv_mode,
            "NCCL_GPUDIRECTTCPX_RX_POOL_MODE": rx_pool_mode,
            "NCCL_GPUDIRECTTCPX_RX_POOL_BYTES": str(rx_pool_mb << 20),
            "NCCL_GPUDIRECTTCPX_NIC_SPEED_MBPS": str(speed_mbps),
            # loopback has no bandwidth-delay product to cover: a bounded send buffer keeps each stream's
            # bytes inside the kernel few enough to stay in the caches (0 = the kernel's auto-tuning)
            "NCCL_GPUDIRECTTCPX_SOCKET_SNDBUF": str(sndbuf),
        })
        if recv_mode == "unpack":
            # NCCL's kernels unpack from the rx page pool: receive buffers are CUDA
            # pointers (GDR level SYS because the "NIC" hangs off the CPU), sends stay
            # in host memory, and only the Simple protocol knows the unpack path.
            env["NCCL_NET_GDR_LEVEL"] = "SYS"
            env["NCCL_NET_GDR_READ"] = "0"
            env["NCCL_PROTO"] = "Simple"
            # the unpack hook exists in the ring primitives; tree/PAT paths never call it
            env["NCCL_ALGO"] = "Ring"
        elif gdr:
            # plugin-side copies and kernels: only safe when no application thread
            # blocks in a synchronous CUDA call while a collective is in flight
            env["NCCL_GPUDIRECTTCPX_CUDA_BUFFERS"] = "1"
            env["NCCL_NET_GDR_LEVEL"] = "SYS"
            env["NCCL_NET_GDR_READ"] = "1"
    # NCCL opens one connection (with its helper threads) per channel and direction.  With few cores per
    # rank more channels only add threads: 4 ranks on 16 cores moved 19.5 - 22.9 GB/s (bus) through the plugin
    # with 4 channels against 14.9 with NCCL's own choice and 17.4 with 8; NCCL's socket transport is
    # indifferent (13.4 - 14.9 with 2, 4 or its own choice).  A generic NCCL variable: set for either transport.
    if max_channels < 0:
        per_rank = len(os.sched_getaffinity(0)) // max(1, int(os.environ.get("LOCAL_WORLD_SIZE", "1")))
        max_channels = 4 if per_rank < 6 else 0
    if max_channels > 0 and "NCCL_MAX_NCHANNELS" not in os.environ:
        env["NCCL_MAX_NCHANNELS"] = str(max_channels)
        env["NCCL_MIN_NCHANNELS"] = str(max_channels)
    if debug:
        env["NCCL_DEBUG"] = debug
        env["NCCL_DEBUG_SUBSYS"] = "INIT,NET,ENV"
    if extra:
        env.update(extra)
    return env


def use_plugin(**kw) -> Dict[str, str]:
    """Applies plugin_env() to os.environ (before torch.distributed initialises NCCL)."""
    env = plugin_env(**kw)
    os.environ.update(env)
    return env
