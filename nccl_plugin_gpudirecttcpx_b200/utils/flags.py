"""Lists every environment variable the transport understands (name, kind, default, meaning).

    python -m nccl_plugin_gpudirecttcpx_b200.utils.flags          # table on stdout
"""
from __future__ import annotations

import ctypes
from typing import List, Tuple

from . import native


def flag_docs() -> List[Tuple[str, str, str, str]]:
    """(env, kind, default, doc) for each variable, straight from the native registry."""
    try:
        lib = native.load("libtcpxb_host.so")
    except Exception:
        lib = native.load("libnccl-net.so")
    lib.tcpxb_flag_count.restype = ctypes.c_int
    lib.tcpxb_flag_doc.argtypes = [ctypes.c_int] + [ctypes.POINTER(ctypes.c_char_p)] * 4
    out = []
    for i in range(lib.tcpxb_flag_count()):
        env, kind, dflt, doc = (ctypes.c_char_p() for _ in range(4))
        if lib.tcpxb_flag_doc(i, ctypes.byref(env), ctypes.byref(kind), ctypes.byref(dflt), ctypes.byref(doc)) == 0:
            out.append((env.value.decode(), kind.value.decode(), dflt.value.decode(), doc.value.decode()))
    return out


if __name__ == "__main__":
    rows = flag_docs()
    width = max(len(r[0]) for r in rows)
    for env, kind, dflt, doc in rows:
        print(f"{env:<{width}}  {kind:<6}  {dflt or '-':<12}  {doc}")
