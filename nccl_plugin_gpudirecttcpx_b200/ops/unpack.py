"""Python bindings of the sm_100a unpack kernels, and their CPU oracle.

The kernels consume the scatter list the receive path produces: one
`{u32 src_off, u32 len, u64 dst_off}` record per rx page fragment (the layout the
reference fills in at src/sock/tcpx.h:178-180 for NCCL's in-kernel unpack).  The
functions here take torch CUDA tensors, pass raw pointers and the current stream
to the C ABI in `csrc/include/tcpxb/kernels.h`, and raise if the native library is
missing: there is no eager fallback on a GPU.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import numpy as np
import torch

from ..utils import native

FRAG_BYTES = 4096
DTYPE_U8, DTYPE_BF16, DTYPE_F32 = 0, 1, 2
REDUCE_SM, REDUCE_L2 = 0, 1
MAX_PEERS = 8
STATUS_WORDS = 4
ST_OK, ST_BOUNDS, ST_ALIGN, ST_TIMEOUT = 0, 1, 2, 3

DESC_DTYPE = np.dtype([("src_off", "<u4"), ("len", "<u4"), ("dst_off", "<u8")])


class _Opts(ctypes.Structure):
    _fields_ = [
        ("ready_count", ctypes.c_void_p),
        ("wait_ns", ctypes.c_uint64),
        ("peer_flags", ctypes.c_void_p * MAX_PEERS),
        ("flag_value", ctypes.c_uint32),
        ("ticket", ctypes.c_void_p),
        ("max_ctas", ctypes.c_int),
        ("early_launch", ctypes.c_int),
    ]


_lib = None


def _k():
    global _lib
    if _lib is None:
        lib = native.load("libtcpxb_kernels.so")
        vp, u64, u32, ci = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int
        lib.tcpxb_kernel_last_error.restype = ctypes.c_char_p
        lib.tcpxb_unpack_copy.argtypes = [vp, u64, vp, u64, vp, u32, vp, vp, vp]
        lib.tcpxb_unpack_reduce.argtypes = [vp, u64, vp, vp, u64, vp, u32, ci, ci, vp, vp, vp]
        lib.tcpxb_unpack_fanout.argtypes = [vp, u64, vp, u64, vp, ci, vp, u32, vp, vp, vp]
        lib.tcpxb_unpack_reduce_fanout.argtypes = [vp, u64, vp, vp, u64, vp, ci, vp, u32, ci, ci, vp, vp, vp]
        lib.tcpxb_unpack_fanout_nvls.argtypes = [vp, u64, vp, vp, u64, vp, ci, vp, u32, vp, vp, vp]
        lib.tcpxb_unpack_reduce_fanout_nvls.argtypes = [vp, u64, vp, vp, vp, u64, vp, ci, vp, u32, ci, vp, vp, vp]
        lib.tcpxb_wait_flags.argtypes = [vp, ci, u32, u64, vp, vp]
        lib.tcpxb_peer_reduce.argtypes = [vp, vp, ci, u64, u64, ci, vp]
        lib.tcpxb_checksum_scratch_bytes.restype = ctypes.c_size_t
        lib.tcpxb_checksum.argtypes = [vp, u64, vp, vp, vp]
        _lib = lib
    return _lib


def _check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(f"tcpxb kernel call failed ({rc}): {_k().tcpxb_kernel_last_error().decode()}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _nbytes(t: torch.Tensor) -> int:
    return t.numel() * t.element_size()


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return DTYPE_BF16
    if t.dtype == torch.float32:
        return DTYPE_F32
    raise TypeError(f"reduce supports bfloat16 and float32, got {t.dtype}")


def _need_cuda(*ts: Optional[torch.Tensor]) -> None:
    """Every tensor a kernel touches is device memory, or pinned host memory (which the device
    addresses directly: the transport's default rx page pool is such memory)."""
    for t in ts:
        if t is not None and not ((t.is_cuda or t.is_pinned()) and t.is_contiguous()):
            raise ValueError("tensors must be contiguous CUDA (or pinned host) tensors")


# ----------------------------------------------------------------- descriptors
def make_descriptors(src_off, length, dst_off) -> np.ndarray:
    """Packs three equal-length integer sequences into the 16-byte record array."""
    src_off = np.asarray(src_off, dtype=np.uint64)
    d = np.zeros(src_off.shape[0], dtype=DESC_DTYPE)
    d["src_off"] = src_off
    d["len"] = np.asarray(length, dtype=np.uint64)
    d["dst_off"] = np.asarray(dst_off, dtype=np.uint64)
    return d


def permuted_fragments(total_bytes: int, pool_bytes: int, seed: int, frag: int = FRAG_BYTES,
                       pool_page_base: int = 0) -> np.ndarray:
    """Scatter list for `total_bytes` contiguous destination bytes whose fragments sit at
    a seeded random permutation of pool pages; the last fragment is the ragged rest."""
    n = (total_bytes + frag - 1) // frag
    pages = pool_bytes // frag
    if n > pages:
        raise ValueError("pool too small")
    rng = np.random.default_rng(seed)
    perm = rng.permutation(pages)[:n].astype(np.uint64) + np.uint64(pool_page_base)
    lens = np.full(n, frag, dtype=np.uint64)
    if total_bytes % frag:
        lens[-1] = total_bytes % frag
    dst = np.arange(n, dtype=np.uint64) * np.uint64(frag)
    return make_descriptors(perm * np.uint64(frag), lens, dst)


def descriptors_to_device(descs: np.ndarray, device=None) -> torch.Tensor:
    """Uploads a record array as a uint8 CUDA tensor (16 bytes per record)."""
    raw = torch.from_numpy(descs.view(np.uint8).copy())
    return raw.to(device or torch.device("cuda"))


def status_buffer(device=None) -> torch.Tensor:
    return torch.zeros(STATUS_WORDS, dtype=torch.int32, device=device or torch.device("cuda"))


def _desc_args(descs: torch.Tensor):
    if descs.dtype != torch.uint8 or _nbytes(descs) % 16:
        raise ValueError("descs must be a uint8 tensor of 16-byte records")
    return descs.data_ptr(), _nbytes(descs) // 16


def _opts(ready_count=None, wait_ns=0, peer_flags: Sequence[int] = (), flag_value=0, ticket=None,
          max_ctas=0, early_launch=False):
    if ready_count is None and not peer_flags and not flag_value and not max_ctas and not wait_ns and not early_launch:
        return None, None
    o = _Opts()
    o.ready_count = ready_count if isinstance(ready_count, (int, type(None))) else ready_count.data_ptr()
    o.wait_ns = int(wait_ns)
    for i, f in enumerate(peer_flags):
        o.peer_flags[i] = int(f)
    o.flag_value = int(flag_value)
    o.ticket = None if ticket is None else ticket.data_ptr()
    o.max_ctas = int(max_ctas)
    o.early_launch = int(bool(early_launch))  # programmatic dependent launch: may start while the stream's previous kernel still runs
    return o, ctypes.byref(o)


def _peer_table(peers: Sequence) -> tuple:
    arr = (ctypes.c_void_p * max(1, len(peers)))()
    for i, p in enumerate(peers):
        arr[i] = p if isinstance(p, int) else p.data_ptr()
    return arr, len(peers)


# --------------------------------------------------------------------- kernels
def unpack_copy(pool: torch.Tensor, dst: torch.Tensor, descs: torch.Tensor,
                status: Optional[torch.Tensor] = None, **opts) -> None:
    """K1: dst[dst_off : dst_off+len] = pool[src_off : src_off+len] per record."""
    _need_cuda(pool, dst, descs, status)
    dptr, n = _desc_args(descs)
    o, oref = _opts(**opts)
    _check(_k().tcpxb_unpack_copy(pool.data_ptr(), _nbytes(pool), dst.data_ptr(), _nbytes(dst),
                                  dptr, n, _ptr(status), oref, _stream()))


def pack(src: torch.Tensor, staging: torch.Tensor, descs: torch.Tensor,
         status: Optional[torch.Tensor] = None, **opts) -> None:
    """K4, send-side gather: staging[dst_off : dst_off+len] = src[src_off : src_off+len] per
    record, e.g. from a strided or paged send buffer into one pinned, device-mapped staging
    area the sockets read from.  It is the unpack kernel with the roles of pool and
    destination swapped; contiguous sends use the copy engine instead."""
    unpack_copy(src, staging, descs, status=status, **opts)


def unpack_reduce(pool: torch.Tensor, acc: torch.Tensor, descs: torch.Tensor,
                  out: Optional[torch.Tensor] = None, impl: int = REDUCE_SM,
                  status: Optional[torch.Tensor] = None, **opts) -> None:
    """K2: out = acc + pool-fragments (element type of `acc`); in place when out is None."""
    _need_cuda(pool, acc, descs, out, status)
    dptr, n = _desc_args(descs)
    dst = acc if out is None else out
    o, oref = _opts(**opts)
    _check(_k().tcpxb_unpack_reduce(pool.data_ptr(), _nbytes(pool), acc.data_ptr(), dst.data_ptr(),
                                    _nbytes(dst), dptr, n, _dtype_code(acc), impl, _ptr(status),
                                    oref, _stream()))


def unpack_fanout(pool: torch.Tensor, dst: torch.Tensor, peers: Sequence, descs: torch.Tensor,
                  status: Optional[torch.Tensor] = None, mc_dst: Optional[int] = None, **opts) -> None:
    """K3: K1 plus a store of every fragment into each peer buffer (tensor or raw pointer).
    With `mc_dst` (an NVLS multicast address of dst) the fan-out is one multimem store."""
    _need_cuda(pool, dst, descs, status)
    dptr, n = _desc_args(descs)
    tbl, np_ = _peer_table(peers)
    o, oref = _opts(**opts)
    if mc_dst is None:
        _check(_k().tcpxb_unpack_fanout(pool.data_ptr(), _nbytes(pool), dst.data_ptr(), _nbytes(dst),
                                        tbl, np_, dptr, n, _ptr(status), oref, _stream()))
    else:
        _check(_k().tcpxb_unpack_fanout_nvls(pool.data_ptr(), _nbytes(pool), dst.data_ptr(), mc_dst,
                                             _nbytes(dst), tbl, np_, dptr, n, _ptr(status), oref,
                                             _stream()))


def unpack_reduce_fanout(pool: torch.Tensor, acc: Optional[torch.Tensor], dst: torch.Tensor,
                         peers: Sequence, descs: torch.Tensor, impl: int = REDUCE_SM,
                         status: Optional[torch.Tensor] = None, mc_dst: Optional[int] = None,
                         **opts) -> None:
    """K3r: dst = acc + fragments, the sum also stored to each peer.  impl=REDUCE_L2 (or
    acc=None with `mc_dst`) instead adds the fragments into dst and into every peer."""
    _need_cuda(pool, acc, dst, descs, status)
    dptr, n = _desc_args(descs)
    tbl, np_ = _peer_table(peers)
    o, oref = _opts(**opts)
    if mc_dst is None:
        _check(_k().tcpxb_unpack_reduce_fanout(pool.data_ptr(), _nbytes(pool), _ptr(acc),
                                               dst.data_ptr(), _nbytes(dst), tbl, np_, dptr, n,
                                               _dtype_code(dst), impl, _ptr(status), oref, _stream()))
    else:
        _check(_k().tcpxb_unpack_reduce_fanout_nvls(pool.data_ptr(), _nbytes(pool), _ptr(acc),
                                                    dst.data_ptr(), mc_dst, _nbytes(dst), tbl, np_,
                                                    dptr, n, _dtype_code(dst), _ptr(status), oref,
                                                    _stream()))


def wait_flags(flags: torch.Tensor, value: int, wait_ns: int = 0,
               status: Optional[torch.Tensor] = None) -> None:
    """Bounded device-side wait until every flags[i] >= value."""
    _need_cuda(flags, status)
    _check(_k().tcpxb_wait_flags(flags.data_ptr(), flags.numel(), value, wait_ns, _ptr(status), _stream()))


def peer_reduce(out: torch.Tensor, srcs: Sequence, shard_off: int) -> None:
    """out = sum_r srcs[r][shard_off : shard_off + out.nbytes] over peer-mapped buffers."""
    _need_cuda(out)
    tbl, n = _peer_table(srcs)
    _check(_k().tcpxb_peer_reduce(out.data_ptr(), tbl, n, shard_off, _nbytes(out), _dtype_code(out), _stream()))


_csum_scratch: dict = {}


def checksum(buf: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """64-bit sum of the buffer's little-endian 32-bit words, as a 1-element int64 CUDA tensor."""
    _need_cuda(buf, out)
    key = (buf.device.index, torch.cuda.current_stream().cuda_stream)
    if key not in _csum_scratch:
        _csum_scratch[key] = torch.zeros(_k().tcpxb_checksum_scratch_bytes(), dtype=torch.uint8, device=buf.device)
    if out is None:
        out = torch.empty(1, dtype=torch.int64, device=buf.device)
    _check(_k().tcpxb_checksum(buf.data_ptr(), _nbytes(buf), out.data_ptr(), _csum_scratch[key].data_ptr(), _stream()))
    return out


# ---------------------------------------------------------------------- oracle
def reference_unpack(pool: torch.Tensor, dst: torch.Tensor, descs: np.ndarray,
                     acc: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Plain PyTorch oracle on the CPU.  Copy: byte gather/scatter.  Reduce: the bytes are
    reinterpreted as the element type of `acc`, added in fp32 and rounded once."""
    pool_b = pool.detach().cpu().contiguous().view(torch.uint8)
    out = dst.detach().cpu().contiguous().clone()
    out_b = out.view(torch.uint8)
    pool_bytes, dst_bytes = pool_b.numel(), out_b.numel()
    acc_b = None if acc is None else acc.detach().cpu().contiguous().view(torch.uint8)
    for r in descs:
        so, ln, do = int(r["src_off"]), int(r["len"]), int(r["dst_off"])
        if ln == 0 or so + ln > pool_bytes or do + ln > dst_bytes:
            continue
        frag = pool_b[so:so + ln]
        if acc is None:
            out_b[do:do + ln] = frag
        else:
            es = acc.element_size()
            if (so % es) or (do % es) or (ln % es):
                continue
            a = acc_b[do:do + ln].clone().view(acc.dtype).to(torch.float32)
            f = frag.clone().view(acc.dtype).to(torch.float32)
            out_b[do:do + ln] = (a + f).to(acc.dtype).view(torch.uint8)
    return out
