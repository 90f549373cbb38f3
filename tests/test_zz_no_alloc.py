"""The allocation-free checksum entry point, called through its exported C symbol.

Some callers of this library may not allocate device memory: the transport's
progress loop runs on NCCL's proxy thread, where a cudaMalloc would synchronise
the device and can deadlock against a collective that is waiting for that very
thread, and embedders may run with a fixed amount of device memory.  For them
`tcpxb_checksum_noalloc` keeps its scratch in an array inside the library.  This
test checks it against the ordinary entry point (caller-provided scratch), twice in
a row because every call reuses the same array, and checks the size limit.
The file sorts last so that a run that stops at the first failure has already
executed every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_BYTES = 1 << 34


def _lib():
    from nccl_plugin_gpudirecttcpx_b200.utils import native
    lib = native.load("libtcpxb_kernels.so")
    vp, u64 = ctypes.c_void_p, ctypes.c_uint64
    lib.tcpxb_checksum_noalloc.argtypes = [vp, u64, vp, vp]
    lib.tcpxb_checksum_noalloc.restype = ctypes.c_int
    lib.tcpxb_checksum.argtypes = [vp, u64, vp, vp, vp]
    lib.tcpxb_checksum.restype = ctypes.c_int
    lib.tcpxb_checksum_scratch_bytes.restype = ctypes.c_size_t
    lib.tcpxb_kernel_last_error.restype = ctypes.c_char_p
    return lib


@pytest.mark.parametrize("nbytes", [4, 1000, (8 << 20) + 12, 160 << 20])
def test_noalloc_checksum_matches_the_allocating_entry_point(nbytes):
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    # everything the calls need is allocated up front; the calls under test allocate nothing
    scratch = torch.zeros(lib.tcpxb_checksum_scratch_bytes(), dtype=torch.uint8, device="cuda")
    want = torch.zeros(1, dtype=torch.int64, device="cuda")
    got = torch.zeros(2, dtype=torch.int64, device="cuda")
    bufs = [torch.randint(0, 256, (nbytes,), dtype=torch.uint8, device="cuda",
                          generator=torch.Generator("cuda").manual_seed(nbytes + i)) for i in range(2)]
    # one call first: the array's address is looked up once per device, which may load the module
    assert lib.tcpxb_checksum_noalloc(bufs[0].data_ptr(), 4, got.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    for i, buf in enumerate(bufs):  # two calls in a row share the library's scratch array
        assert lib.tcpxb_checksum(buf.data_ptr(), nbytes, want.data_ptr(), scratch.data_ptr(), stream) == 0
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = lib.tcpxb_checksum_noalloc(buf.data_ptr(), nbytes, got[i:].data_ptr(), stream)
        assert rc == 0, lib.tcpxb_kernel_last_error().decode()
        torch.cuda.synchronize()
        # the device's free memory is what it was: the call allocated nothing (no other
        # CUDA work of this process ran in between)
        assert torch.cuda.mem_get_info()[0] >= free_before
        assert got[i].item() == want.item()  # integer sums: equal, not merely close
        pad = torch.cat([buf, torch.zeros((-nbytes) % 4, dtype=torch.uint8, device="cuda")])
        assert (got[i].item() & 0xFFFFFFFFFFFFFFFF) == int(pad.view(torch.int32).to(torch.int64).bitwise_and(0xFFFFFFFF).sum().item())


def test_noalloc_checksum_rejects_oversize_without_launching():
    lib = _lib()
    out = torch.full((1,), -7, dtype=torch.int64, device="cuda")
    buf = torch.zeros(16, dtype=torch.uint8, device="cuda")
    rc = lib.tcpxb_checksum_noalloc(buf.data_ptr(), MAX_BYTES + 4, out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == -3
    assert b"at most 16 GiB" in lib.tcpxb_kernel_last_error()
    assert out.item() == -7
