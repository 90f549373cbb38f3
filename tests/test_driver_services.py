"""Driver-API services on a real GPU: dma-buf export of device memory and a device allocation
shared by file descriptor (what the rx buffer manager daemon hands to its clients)."""
import ctypes
import os
import stat

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from nccl_plugin_gpudirecttcpx_b200.utils import native
    lib = native.load("libnccl-net.so")
    lib.tcpxb_export_dmabuf.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_uint64)]
    lib.tcpxb_shared_pool_selftest.argtypes = [ctypes.c_int, ctypes.c_uint64]
    return lib


def test_dmabuf_export_of_a_registered_send_buffer():
    """A send buffer in device memory leaves as a dma-buf descriptor a devmem-capable NIC could bind
    (reference: src/gpu/tx_pool.cu:104-181).  The export needs no NIC."""
    lib = _lib()
    x = torch.empty(8 << 20, dtype=torch.uint8, device="cuda")
    fd, off = ctypes.c_int(-1), ctypes.c_uint64(0)
    rc = lib.tcpxb_export_dmabuf(x.data_ptr() + 12345, 1 << 20, ctypes.byref(fd), ctypes.byref(off))
    if rc != 0:
        pytest.skip("this driver does not export dma-bufs for cudaMalloc memory")
    try:
        assert fd.value >= 0
        assert off.value == (x.data_ptr() + 12345) % os.sysconf("SC_PAGE_SIZE")
        st = os.fstat(fd.value)
        assert not stat.S_ISREG(st.st_mode)  # an anonymous dma-buf inode, not a file
        assert "dmabuf" in os.readlink(f"/proc/self/fd/{fd.value}")
    finally:
        os.close(fd.value)
    # the context is still usable and the buffer untouched by the export
    x.fill_(7)
    assert int(x[12345].item()) == 7


def test_device_pool_shared_by_file_descriptor():
    """Create on the owner's side, export, import on the client's side: both mappings are the same
    device memory (reference: src/gpu/common.cu:25-65)."""
    assert _lib().tcpxb_shared_pool_selftest(torch.cuda.current_device(), 16 << 20) == 0
