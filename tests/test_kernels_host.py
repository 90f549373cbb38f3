"""The CPU statement of the kernel ABI (csrc/kernels/kernels_host.cc, part of the host-only
library) against the plain PyTorch oracle that the sm_100a kernels are tested against on the GPU
(ops.reference_unpack).  Two independent descriptions of the same operations must agree bit for bit.
"""
import ctypes

import numpy as np
import pytest
import torch

from nccl_plugin_gpudirecttcpx_b200 import _build
from nccl_plugin_gpudirecttcpx_b200.ops.unpack import make_descriptors, permuted_fragments, reference_unpack


class Opts(ctypes.Structure):
    _fields_ = [("ready_count", ctypes.c_void_p), ("wait_ns", ctypes.c_uint64), ("peer_flags", ctypes.c_void_p * 8),
                ("flag_value", ctypes.c_uint32), ("ticket", ctypes.c_void_p), ("max_ctas", ctypes.c_int)]


@pytest.fixture(scope="module")
def k():
    lib = ctypes.CDLL(str(_build.build_host()))
    vp, u64, u32, ci = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int
    lib.tcpxb_unpack_copy.argtypes = [vp, u64, vp, u64, vp, u32, vp, vp, vp]
    lib.tcpxb_unpack_reduce.argtypes = [vp, u64, vp, vp, u64, vp, u32, ci, ci, vp, vp, vp]
    lib.tcpxb_unpack_fanout.argtypes = [vp, u64, vp, u64, vp, ci, vp, u32, vp, vp, vp]
    lib.tcpxb_unpack_reduce_fanout.argtypes = [vp, u64, vp, vp, u64, vp, ci, vp, u32, ci, ci, vp, vp, vp]
    lib.tcpxb_wait_flags.argtypes = [vp, ci, u32, u64, vp, vp]
    lib.tcpxb_peer_reduce.argtypes = [vp, vp, ci, u64, u64, ci, vp]
    lib.tcpxb_checksum_noalloc.argtypes = [vp, u64, vp, vp]
    lib.tcpxb_kernel_last_error.restype = ctypes.c_char_p
    return lib


def _case(total, seed, tail=0):
    pool_bytes = (total + tail) * 2 + 8192
    descs = permuted_fragments(total, pool_bytes, seed)
    if tail:
        extra = make_descriptors([pool_bytes - 4096], [tail], [total])
        descs = np.concatenate([descs, extra])
    pool = torch.randint(0, 256, (pool_bytes,), dtype=torch.uint8, generator=torch.Generator().manual_seed(seed))
    return pool, descs


def _dptr(descs):
    return descs.ctypes.data_as(ctypes.c_void_p), len(descs)


@pytest.mark.parametrize("total,tail", [(4096 * 37, 0), (4096 * 64, 1), (4096 * 5, 4095), (0, 17)])
def test_copy_matches_oracle(k, total, tail):
    pool, descs = _case(total, 3, tail)
    dst = torch.full((total + tail + 64,), 0xEE, dtype=torch.uint8)
    want = reference_unpack(pool, dst, descs)
    status = torch.zeros(4, dtype=torch.int32)
    p, n = _dptr(descs)
    assert k.tcpxb_unpack_copy(pool.data_ptr(), pool.numel(), dst.data_ptr(), dst.numel(), p, n, status.data_ptr(), None, None) == 0
    assert torch.equal(dst, want) and status.tolist() == [0, 0, 0, 0]
    assert bool((dst[total + tail:] == 0xEE).all())  # nothing written past the last fragment


@pytest.mark.parametrize("dtype,code", [(torch.bfloat16, 1), (torch.float32, 2)])
@pytest.mark.parametrize("impl", [0, 1])
def test_reduce_matches_oracle(k, dtype, code, impl):
    total = 4096 * 48
    pool, descs = _case(total, 11)
    g = torch.Generator().manual_seed(5)
    # the pool holds arbitrary bytes: keep NaN/Inf patterns out of the comparison by building it from values
    vals = torch.randn(pool.numel() // dtype.itemsize, generator=g).to(dtype)
    pool = vals.view(torch.uint8).clone()
    acc = torch.randn(total // dtype.itemsize, generator=g).to(dtype)
    want = reference_unpack(pool, acc, descs, acc=acc)
    out = acc.clone()
    status = torch.zeros(4, dtype=torch.int32)
    p, n = _dptr(descs)
    rc = k.tcpxb_unpack_reduce(pool.data_ptr(), pool.numel(), None if impl else out.data_ptr(), out.data_ptr(),
                               out.numel() * out.element_size(), p, n, code, impl, status.data_ptr(), None, None)
    assert rc == 0 and status[0].item() == 0
    assert torch.equal(out.view(torch.uint8), want.view(torch.uint8))


def test_fanout_and_flags(k):
    total = 4096 * 16
    pool, descs = _case(total, 21)
    dst = torch.zeros(total, dtype=torch.uint8)
    peers = [torch.zeros(total, dtype=torch.uint8) for _ in range(3)]
    flags = torch.zeros(8, dtype=torch.int32)
    want = reference_unpack(pool, dst, descs)
    table = (ctypes.c_void_p * 3)(*[t.data_ptr() for t in peers])
    opts = Opts()
    for i in range(3):
        opts.peer_flags[i] = flags.data_ptr() + 4 * i
    opts.flag_value = 7
    status = torch.zeros(4, dtype=torch.int32)
    p, n = _dptr(descs)
    assert k.tcpxb_unpack_fanout(pool.data_ptr(), pool.numel(), dst.data_ptr(), total, table, 3, p, n, status.data_ptr(),
                                 ctypes.byref(opts), None) == 0
    assert torch.equal(dst, want) and all(torch.equal(t, want) for t in peers)
    assert flags.tolist() == [7, 7, 7, 0, 0, 0, 0, 0]
    # the counterpart: a wait on published flags returns at once, one on a flag nobody sets runs out
    assert k.tcpxb_wait_flags(flags.data_ptr(), 3, 7, 0, status.data_ptr(), None) == 0 and status[0].item() == 0
    assert k.tcpxb_wait_flags(flags.data_ptr(), 4, 7, 50_000_000, status.data_ptr(), None) == 0
    assert status.tolist()[:2] == [3, 3]  # TCPXB_ST_TIMEOUT at flag 3


def test_reduce_fanout_both_forms(k):
    total = 4096 * 8
    n_el = total // 4
    g = torch.Generator().manual_seed(9)
    frag = torch.randn(n_el, generator=g)
    pool = frag.view(torch.uint8).clone()
    descs = make_descriptors([0], [total], [0])
    p, n = _dptr(descs)
    acc = torch.randn(n_el, generator=g)
    dst = torch.zeros(n_el)
    peer = torch.full((n_el,), 100.0)
    table = (ctypes.c_void_p * 1)(peer.data_ptr())
    status = torch.zeros(4, dtype=torch.int32)
    # SM form: dst = acc + frag, and the sum is stored to the peer
    assert k.tcpxb_unpack_reduce_fanout(pool.data_ptr(), total, acc.data_ptr(), dst.data_ptr(), total, table, 1, p, n, 2, 0,
                                        status.data_ptr(), None, None) == 0
    assert torch.equal(dst, acc + frag) and torch.equal(peer, dst)
    # L2 form: the fragment is added into every buffer, each keeping its own sum
    dst2 = acc.clone()
    peer2 = torch.full((n_el,), 100.0)
    table2 = (ctypes.c_void_p * 1)(peer2.data_ptr())
    assert k.tcpxb_unpack_reduce_fanout(pool.data_ptr(), total, None, dst2.data_ptr(), total, table2, 1, p, n, 2, 1,
                                        status.data_ptr(), None, None) == 0
    assert torch.equal(dst2, acc + frag) and torch.equal(peer2, 100.0 + frag)
    assert k.tcpxb_unpack_reduce_fanout(pool.data_ptr(), total, acc.data_ptr(), dst2.data_ptr(), total, table2, 1, p, n, 2, 1,
                                        status.data_ptr(), None, None) != 0  # the L2 form is in place only
    assert b"in place" in k.tcpxb_kernel_last_error()


def test_status_words_for_bad_records(k):
    pool = torch.arange(8192, dtype=torch.int32).view(torch.uint8)[:8192].clone()
    dst = torch.zeros(8192, dtype=torch.uint8)
    descs = make_descriptors([0, 8000, 0, 4096], [4096, 4096, 4096, 4096], [0, 0, 8000, 4096])  # 2nd leaves the pool, 3rd the buffer
    status = torch.zeros(4, dtype=torch.int32)
    p, n = _dptr(descs)
    assert k.tcpxb_unpack_copy(pool.data_ptr(), 8192, dst.data_ptr(), 8192, p, n, status.data_ptr(), None, None) == 0
    assert status.tolist()[:3] == [1, 1, 2]  # TCPXB_ST_BOUNDS, first at record 1, two records skipped
    assert torch.equal(dst, reference_unpack(pool, torch.zeros(8192, dtype=torch.uint8), descs))
    # a reduce record that is not a whole number of elements is skipped with TCPXB_ST_ALIGN
    acc = torch.zeros(2048, dtype=torch.float32)
    descs = make_descriptors([0, 4096], [4096, 4094], [0, 4096])
    status.zero_()
    p, n = _dptr(descs)
    assert k.tcpxb_unpack_reduce(pool.data_ptr(), 8192, acc.data_ptr(), acc.data_ptr(), 8192, p, n, 2, 0, status.data_ptr(), None, None) == 0
    assert status.tolist()[:3] == [2, 1, 1]


def test_peer_reduce_and_checksum(k):
    g = torch.Generator().manual_seed(2)
    srcs = [torch.randn(4096, generator=g).to(torch.bfloat16) for _ in range(4)]
    out = torch.zeros(1024, dtype=torch.bfloat16)
    table = (ctypes.c_void_p * 4)(*[t.data_ptr() for t in srcs])
    assert k.tcpxb_peer_reduce(out.data_ptr(), table, 4, 2048 * 2, 1024 * 2, 1, None) == 0
    want = torch.stack([t[2048:3072].float() for t in srcs]).sum(0).to(torch.bfloat16)  # one rounding
    assert torch.equal(out, want)
    buf = torch.randint(0, 256, (10007,), dtype=torch.uint8, generator=g)
    padded = torch.cat([buf, torch.zeros(1, dtype=torch.uint8)]).view(torch.int32)
    want_sum = int((padded.to(torch.int64) & 0xFFFFFFFF).sum().item())
    got = ctypes.c_uint64(0)
    assert k.tcpxb_checksum_noalloc(buf.data_ptr(), buf.numel(), ctypes.byref(got), None) == 0
    assert got.value == want_sum


def test_streaming_ready_counter(k):
    """Records are consumed as a producer publishes them; a counter that stops short runs the
    bounded wait out once: the time-out is reported and the rest is left alone."""
    import threading
    import time
    total = 4096 * 32
    pool, descs = _case(total, 33)
    want = reference_unpack(pool, torch.zeros(total, dtype=torch.uint8), descs)
    counter = torch.zeros(1, dtype=torch.int32)
    opts = Opts()
    opts.ready_count = counter.data_ptr()
    opts.wait_ns = 2_000_000_000
    status = torch.zeros(4, dtype=torch.int32)
    dst = torch.zeros(total, dtype=torch.uint8)
    p, n = _dptr(descs)

    def producer():
        for i in range(1, n + 1):
            if i % 8 == 0:
                time.sleep(0.001)
            counter[0] = i

    t = threading.Thread(target=producer)
    t.start()
    rc = k.tcpxb_unpack_copy(pool.data_ptr(), pool.numel(), dst.data_ptr(), total, p, n, status.data_ptr(), ctypes.byref(opts), None)
    t.join()
    assert rc == 0 and status[0].item() == 0 and torch.equal(dst, want)
    # the producer stops after 10 records
    counter[0] = 10
    opts.wait_ns = 50_000_000
    dst.zero_()
    t0 = time.time()
    assert k.tcpxb_unpack_copy(pool.data_ptr(), pool.numel(), dst.data_ptr(), total, p, n, status.data_ptr(), ctypes.byref(opts), None) == 0
    assert time.time() - t0 < 1.0
    assert status.tolist()[:3] == [3, 10, 1]  # TCPXB_ST_TIMEOUT at record 10, reported once; nothing after it is attempted
    partial = reference_unpack(pool, torch.zeros(total, dtype=torch.uint8), descs[:10])
    assert torch.equal(dst, partial)
