"""Numerics of the sm_100a unpack kernels against the plain PyTorch CPU oracle."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from nccl_plugin_gpudirecttcpx_b200 import ops
from nccl_plugin_gpudirecttcpx_b200.ops import unpack as U

DEV = "cuda"
GUARD = 256


def _pool(nbytes, seed, dtype=torch.uint8):
    g = torch.Generator().manual_seed(seed)
    if dtype == torch.uint8:
        return torch.randint(0, 256, (nbytes,), dtype=torch.uint8, generator=g)
    return torch.randn(nbytes // dtype.itemsize, generator=g).to(dtype)


def _run_copy(pool_cpu, dst_bytes, descs, **kw):
    pool = pool_cpu.to(DEV)
    # guard bands on both sides of dst catch out-of-range stores
    buf = torch.full((dst_bytes + 2 * GUARD,), 0xA5, dtype=torch.uint8, device=DEV)
    dst = buf[GUARD:GUARD + dst_bytes]
    st = U.status_buffer()
    U.unpack_copy(pool, dst, U.descriptors_to_device(descs), status=st, **kw)
    torch.cuda.synchronize()
    assert bool((buf[:GUARD] == 0xA5).all()) and bool((buf[GUARD + dst_bytes:] == 0xA5).all())
    want = U.reference_unpack(pool_cpu, torch.full((dst_bytes,), 0xA5, dtype=torch.uint8), descs)
    return dst.cpu(), want, st.cpu()


@pytest.mark.parametrize("total", [4096 * 64 + 1234, 4096 * 2048, 1, 15, 16, 4095])
def test_copy_permuted(total):
    pool_bytes = 16 << 20
    pool = _pool(pool_bytes, 1)
    descs = U.permuted_fragments(total, pool_bytes, seed=7)
    dst_bytes = (total + 4095) // 4096 * 4096
    got, want, st = _run_copy(pool, dst_bytes, descs)
    assert torch.equal(got, want)
    assert st.tolist()[0] == U.ST_OK


@pytest.mark.parametrize("mis", [1, 2, 4, 8])
@pytest.mark.parametrize("which", ["src", "dst", "both", "len"])
def test_copy_unaligned_classes(mis, which):
    pool_bytes = 1 << 20
    pool = _pool(pool_bytes, 2)
    n = 97
    rng = np.random.default_rng(mis * 10 + len(which))
    pages = rng.permutation(pool_bytes // 8192)[:n].astype(np.uint64) * 8192
    src = pages + (mis if which in ("src", "both") else 0)
    lens = np.full(n, 4096 - (mis if which == "len" else 0), dtype=np.uint64)
    lens[::7] = rng.integers(1, 4096, size=len(lens[::7]))
    dst = np.arange(n, dtype=np.uint64) * 4200 + (mis if which in ("dst", "both") else 0)
    descs = U.make_descriptors(src, lens, dst)
    got, want, st = _run_copy(pool, 4200 * n + 64, descs)
    assert torch.equal(got, want)
    assert st.tolist()[0] == U.ST_OK


def test_copy_zero_count_and_zero_len_and_long():
    pool_bytes = 1 << 20
    pool = _pool(pool_bytes, 3)
    got, want, st = _run_copy(pool, 4096, U.make_descriptors([], [], []))
    assert torch.equal(got, want)
    # zero-length records between real ones, and one record longer than a slot
    descs = U.make_descriptors([0, 4096, 8192, 65536], [4096, 0, 100, 40000], [0, 4096, 4096, 8192])
    got, want, st = _run_copy(pool, 8192 + 40000, descs)
    assert torch.equal(got, want)
    assert st.tolist()[0] == U.ST_OK


def test_copy_bounds_violation_is_skipped_and_reported():
    pool_bytes = 1 << 20
    pool = _pool(pool_bytes, 4)
    descs = U.make_descriptors([0, pool_bytes - 100, 4096, 8192], [4096, 4096, 4096, 4096],
                               [0, 4096, 8192, 1 << 40])
    got, want, st = _run_copy(pool, 3 * 4096, descs)
    assert torch.equal(got, want)
    s = st.tolist()
    assert s[0] == U.ST_BOUNDS and s[2] == 2 and s[1] in (1, 3)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("impl", [U.REDUCE_SM, U.REDUCE_L2])
def test_reduce_matches_fp32_oracle(dtype, impl):
    pool_bytes = 8 << 20
    total = 4096 * 300 + 2 * 333 * 2
    pool = _pool(pool_bytes, 5, dtype)
    descs = U.permuted_fragments(total, pool_bytes, seed=11)
    n_el = (total + 4095) // 4096 * 4096 // dtype.itemsize
    acc_cpu = torch.randn(n_el, generator=torch.Generator().manual_seed(6)).to(dtype)
    acc = acc_cpu.to(DEV)
    st = U.status_buffer()
    U.unpack_reduce(pool.to(DEV), acc, U.descriptors_to_device(descs), impl=impl, status=st)
    torch.cuda.synchronize()
    want = U.reference_unpack(pool, acc_cpu, descs, acc=acc_cpu)
    got = acc.cpu()
    assert st.tolist()[0] == U.ST_OK
    if impl == U.REDUCE_SM or dtype == torch.float32:
        assert torch.equal(got.view(torch.uint8), want.view(torch.uint8))
    else:
        # the add happens outside the SM: allow one bf16 ulp
        g, w = got.float(), want.float()
        ulp = torch.maximum(w.abs(), torch.tensor(2.0 ** -126)) * 2.0 ** -7
        assert bool(((g - w).abs() <= ulp).all())


def test_early_launch_keeps_the_order_of_dependent_launches():
    """Launches that may start early (programmatic dependent launch) still see what the stream's
    previous kernel wrote: a torch kernel fills the accumulator, then four in-place sums of the same
    fragments follow back to back, each reading what the one before stored."""
    dtype = torch.float32
    pool_bytes = 8 << 20
    total = 4096 * 1500
    pool = _pool(pool_bytes, 21, dtype)
    descs = U.permuted_fragments(total, pool_bytes, seed=23)
    n_el = total // dtype.itemsize
    acc = torch.empty(n_el, dtype=dtype, device=DEV)
    pool_dev, d_dev = pool.to(DEV), U.descriptors_to_device(descs)
    st = U.status_buffer()
    torch.cuda.synchronize()
    acc.fill_(1.0)  # a kernel of another library directly before the first early launch
    for _ in range(4):
        U.unpack_reduce(pool_dev, acc, d_dev, status=st, early_launch=True)
    copy = torch.empty_like(acc)
    straight = np.zeros(total // 4096, dtype=U.DESC_DTYPE)  # fragment i of the sums to fragment i of the copy
    straight["src_off"] = straight["dst_off"] = np.arange(total // 4096, dtype=np.uint64) * 4096
    straight["len"] = 4096
    U.unpack_copy(acc.view(torch.uint8), copy.view(torch.uint8), U.descriptors_to_device(straight), status=st, early_launch=True)
    torch.cuda.synchronize()
    assert st.tolist()[0] == U.ST_OK
    want = torch.ones(n_el, dtype=dtype)
    for _ in range(4):
        want = U.reference_unpack(pool, want, descs, acc=want)
    assert torch.equal(acc.cpu(), want) and torch.equal(copy.cpu(), want)


def test_reduce_out_of_place_and_unaligned_elements():
    pool_bytes = 1 << 20
    pool = _pool(pool_bytes, 8, torch.bfloat16)
    src = np.array([0, 8192 + 2, 16384 + 6, 32768], dtype=np.uint64)
    lens = np.array([4096, 1000, 4096 - 6, 2], dtype=np.uint64)
    dst = np.array([0, 4096 + 2, 8192 + 10, 16384], dtype=np.uint64)
    descs = U.make_descriptors(src, lens, dst)
    acc_cpu = torch.randn(10000, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16)
    out = torch.zeros_like(acc_cpu).to(DEV)
    acc = acc_cpu.to(DEV)
    U.unpack_reduce(pool.to(DEV), acc, U.descriptors_to_device(descs), out=out)
    torch.cuda.synchronize()
    want = U.reference_unpack(pool, torch.zeros_like(acc_cpu), descs, acc=acc_cpu)
    assert torch.equal(out.cpu().view(torch.uint8), want.view(torch.uint8))
    assert torch.equal(acc.cpu().view(torch.uint8), acc_cpu.view(torch.uint8))


def test_reduce_odd_byte_fragment_reports_alignment():
    pool = _pool(1 << 16, 10, torch.bfloat16)
    descs = U.make_descriptors([1, 4096], [64, 64], [0, 64])
    acc = torch.zeros(256, dtype=torch.bfloat16, device=DEV)
    st = U.status_buffer()
    U.unpack_reduce(pool.to(DEV), acc, U.descriptors_to_device(descs), status=st)
    torch.cuda.synchronize()
    assert st.tolist()[0] == U.ST_ALIGN and st.tolist()[1] == 0
    assert torch.equal(acc[32:64].cpu().view(torch.uint8), pool.view(torch.uint8)[4096:4160])


@pytest.mark.parametrize("npeers", [1, 3, 7])
def test_fanout_emulated_peers_on_one_gpu(npeers):
    pool_bytes = 4 << 20
    total = 4096 * 200 + 777
    pool = _pool(pool_bytes, 12)
    descs = U.permuted_fragments(total, pool_bytes, seed=13)
    dst_bytes = 4096 * 201
    dst = torch.zeros(dst_bytes, dtype=torch.uint8, device=DEV)
    peers = [torch.zeros(dst_bytes, dtype=torch.uint8, device=DEV) for _ in range(npeers)]
    flags = torch.zeros(npeers, dtype=torch.int32, device=DEV)
    ticket = torch.zeros(1, dtype=torch.int32, device=DEV)
    st = U.status_buffer()
    U.unpack_fanout(pool.to(DEV), dst, peers, U.descriptors_to_device(descs), status=st,
                    peer_flags=[flags.data_ptr() + 4 * i for i in range(npeers)], flag_value=5,
                    ticket=ticket)
    U.wait_flags(flags, 5, status=st)
    torch.cuda.synchronize()
    want = U.reference_unpack(pool, torch.zeros(dst_bytes, dtype=torch.uint8), descs)
    assert torch.equal(dst.cpu(), want)
    for p in peers:
        assert torch.equal(p.cpu(), want)
    assert flags.tolist() == [5] * npeers and ticket.item() == 0 and st.tolist()[0] == U.ST_OK


@pytest.mark.parametrize("impl", [U.REDUCE_SM, U.REDUCE_L2])
def test_reduce_fanout_emulated_peers(impl):
    dtype = torch.bfloat16
    pool_bytes = 4 << 20
    total = 4096 * 100
    pool = _pool(pool_bytes, 14, dtype)
    descs = U.permuted_fragments(total, pool_bytes, seed=15)
    acc_cpu = torch.randn(total // 2, generator=torch.Generator().manual_seed(16)).to(dtype)
    dst = acc_cpu.to(DEV)
    if impl == U.REDUCE_SM:
        peers = [torch.zeros_like(dst) for _ in range(2)]
    else:
        peers = [acc_cpu.to(DEV) for _ in range(2)]
    U.unpack_reduce_fanout(pool.to(DEV), dst if impl == U.REDUCE_SM else None, dst, peers,
                           U.descriptors_to_device(descs), impl=impl)
    torch.cuda.synchronize()
    want = U.reference_unpack(pool, acc_cpu, descs, acc=acc_cpu)
    for t in [dst] + peers:
        g, w = t.cpu().float(), want.float()
        if impl == U.REDUCE_SM:
            assert torch.equal(g, w)
        else:
            assert bool(((g - w).abs() <= w.abs().clamp_min(2.0 ** -126) * 2.0 ** -7).all())


def test_streaming_ready_counter_and_bounded_timeout():
    pool_bytes = 1 << 20
    total = 4096 * 40
    pool = _pool(pool_bytes, 17)
    descs = U.permuted_fragments(total, pool_bytes, seed=18)
    d = U.descriptors_to_device(descs)
    want = U.reference_unpack(pool, torch.zeros(total, dtype=torch.uint8), descs)
    # all published: behaves like the plain kernel
    ready = torch.tensor([40], dtype=torch.int32, device=DEV)
    dst = torch.zeros(total, dtype=torch.uint8, device=DEV)
    st = U.status_buffer()
    U.unpack_copy(pool.to(DEV), dst, d, status=st, ready_count=ready)
    torch.cuda.synchronize()
    assert torch.equal(dst.cpu(), want) and st.tolist()[0] == U.ST_OK
    # only 10 ever published: the wait runs out, the kernel reports and returns
    ready = torch.tensor([10], dtype=torch.int32, device=DEV)
    dst = torch.zeros(total, dtype=torch.uint8, device=DEV)
    st = U.status_buffer()
    U.unpack_copy(pool.to(DEV), dst, d, status=st, ready_count=ready, wait_ns=20_000_000)
    torch.cuda.synchronize()
    assert st.tolist()[0] == U.ST_TIMEOUT
    assert torch.equal(dst.cpu()[:10 * 4096], want[:10 * 4096])
    # the context is still usable
    assert int(torch.ones(4, device=DEV).sum().item()) == 4


def test_stalled_ready_counter_drains_in_about_one_wait():
    """One CTA, 4096 records, a producer that stops after 5: the kernel gives up after one
    wait (not one wait per remaining record) and reports the time-out once per warp."""
    n = 4096
    pool_bytes = 1 << 20
    total = 4096 * n
    pool = torch.zeros(pool_bytes, dtype=torch.uint8, device=DEV)
    descs = U.make_descriptors(np.zeros(n, dtype=np.uint64), np.full(n, 4096), np.arange(n, dtype=np.uint64) * 4096)
    d = U.descriptors_to_device(descs)
    ready = torch.tensor([5], dtype=torch.int32, device=DEV)
    dst = torch.zeros(total, dtype=torch.uint8, device=DEV)
    st = U.status_buffer()
    wait_ns = 10_000_000
    U.unpack_copy(pool, dst, d, status=st, ready_count=ready, wait_ns=wait_ns, max_ctas=1)  # warm: module load
    torch.cuda.synchronize()
    st.zero_()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    U.unpack_copy(pool, dst, d, status=st, ready_count=ready, wait_ns=wait_ns, max_ctas=1)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    s = st.tolist()
    assert s[0] == U.ST_TIMEOUT
    assert ms < 5 * wait_ns * 1e-6, f"drain took {ms} ms for a {wait_ns * 1e-6} ms limit"
    assert 1 <= s[2] <= 16  # at most one report per warp of the CTA
    assert int(torch.ones(4, device=DEV).sum().item()) == 4


def test_slow_but_steady_producer_never_trips_the_limit():
    """The streaming limit is per wait: a launch that lasts many times wait_ns finishes
    cleanly as long as the producer keeps publishing."""
    n = 64
    pool_bytes = 1 << 20
    pool = _pool(pool_bytes, 31)
    descs = U.permuted_fragments(4096 * n, pool_bytes, seed=32)
    d = U.descriptors_to_device(descs)
    ready_host = torch.zeros(1, dtype=torch.int32).pin_memory()
    dst = torch.zeros(4096 * n, dtype=torch.uint8, device=DEV)
    st = U.status_buffer()
    wait_ns = 40_000_000
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        U.unpack_copy(pool.to(DEV), dst, d, status=st, ready_count=ready_host.data_ptr(), wait_ns=wait_ns, max_ctas=2)
    import time
    t0 = time.time()
    for k in range(1, 9):           # 8 steps of 15 ms: 120 ms in all, three times the limit
        time.sleep(0.015)
        ready_host[0] = k * n // 8
    side.synchronize()
    assert time.time() - t0 > 2 * wait_ns * 1e-9
    want = U.reference_unpack(pool, torch.zeros(4096 * n, dtype=torch.uint8), descs)
    assert st.tolist()[0] == U.ST_OK and torch.equal(dst.cpu(), want)


def test_fanout_flag_is_not_published_after_an_error():
    """A launch that records an error leaves the peers' completion flag alone."""
    pool_bytes = 1 << 20
    n = 40
    pool = _pool(pool_bytes, 33).to(DEV)
    good = U.permuted_fragments(4096 * n, pool_bytes, seed=34)
    bad = good.copy()
    bad[7]["src_off"] = pool_bytes - 8  # runs past the end of the pool
    dst = torch.zeros(4096 * n, dtype=torch.uint8, device=DEV)
    peer = torch.zeros(4096 * n, dtype=torch.uint8, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    ticket = torch.zeros(1, dtype=torch.int32, device=DEV)
    for descs, want_flag, want_status in ((bad, 0, U.ST_BOUNDS), (good, 5, U.ST_OK)):
        st = U.status_buffer()
        U.unpack_fanout(pool, dst, [peer], U.descriptors_to_device(descs), status=st,
                        peer_flags=[flag.data_ptr()], flag_value=5, ticket=ticket)
        torch.cuda.synchronize()
        assert st.tolist()[0] == want_status
        assert flag.item() == want_flag
        assert ticket.item() == 0  # left clean for the next launch either way


def test_wait_flags_timeout_returns_status():
    flags = torch.zeros(3, dtype=torch.int32, device=DEV)
    flags[1] = 9
    st = U.status_buffer()
    U.wait_flags(flags, 9, wait_ns=10_000_000, status=st)
    torch.cuda.synchronize()
    s = st.tolist()
    assert s[0] == U.ST_TIMEOUT and s[2] == 2


@pytest.mark.parametrize("nbytes", [0, 3, 4, 1000, (1 << 20) + 5, 64 << 20])
def test_checksum(nbytes):
    data = _pool(max(nbytes, 1), 19)[:nbytes]
    pad = torch.cat([data, torch.zeros((-nbytes) % 4, dtype=torch.uint8)])
    want = int(pad.numpy().view("<u4").astype(np.uint64).sum()) if nbytes else 0
    for _ in range(2):
        got = ops.checksum(data.to(DEV)).item() & 0xFFFFFFFFFFFFFFFF
        assert got == want


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_peer_reduce(dtype):
    n = 1 << 18
    srcs = [torch.randn(n, generator=torch.Generator().manual_seed(20 + i)).to(dtype) for i in range(4)]
    dsrcs = [s.to(DEV) for s in srcs]
    shard = n // 4
    out = torch.empty(shard, dtype=dtype, device=DEV)
    ops.peer_reduce(out, dsrcs, shard_off=2 * shard * dtype.itemsize)
    torch.cuda.synchronize()
    want = sum(s[2 * shard:3 * shard].float() for s in srcs).to(dtype)
    assert torch.equal(out.cpu(), want)


def test_pack_gathers_into_pinned_staging():
    """Send-side gather into pinned, device-mapped host memory (what the sockets would read)."""
    src = _pool(1 << 20, 21).to(DEV)
    staging = torch.zeros(64 * 1024, dtype=torch.uint8).pin_memory()
    n = 16
    rng = np.random.default_rng(5)
    src_off = rng.permutation((1 << 20) // 4096)[:n].astype(np.uint64) * 4096
    descs = U.make_descriptors(src_off, np.full(n, 4096), np.arange(n, dtype=np.uint64) * 4096)
    st = U.status_buffer()
    # the staging tensor lives in pinned host memory; the kernel gets its (unified) address
    lib = U._k()
    rc = lib.tcpxb_unpack_copy(src.data_ptr(), src.numel(), staging.data_ptr(), staging.numel(),
                               U.descriptors_to_device(descs).data_ptr(), n, st.data_ptr(), None,
                               torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    want = U.reference_unpack(src.cpu(), torch.zeros(64 * 1024, dtype=torch.uint8), descs)
    assert torch.equal(staging, want) and st.tolist()[0] == U.ST_OK
    # and through the Python wrapper on device buffers
    dst = torch.zeros(64 * 1024, dtype=torch.uint8, device=DEV)
    ops.pack(src, dst, U.descriptors_to_device(descs))
    torch.cuda.synchronize()
    assert torch.equal(dst.cpu(), want)
