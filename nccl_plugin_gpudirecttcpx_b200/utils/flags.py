"""Lists every environment variable the transport understands (name, kind, default, meaning).

    python -m nccl_plugin_gpudirecttcpx_b200.utils.flags              # table on stdout
    python -m nccl_plugin_gpudirecttcpx_b200.utils.flags --markdown   # the table of docs/environment.md
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


def markdown_table() -> str:
    lines = ["| variable | kind | default | meaning |", "|---|---|---|---|"]
    for env, kind, dflt, doc in flag_docs():
        lines.append(f"| `{env}` | {kind} | {('`' + dflt + '`') if dflt else '-'} | {doc} |")
    return "\n".join(lines) + "\n"


if __name__ == "__main__":
    import sys
    if "--markdown" in sys.argv[1:]:
        sys.stdout.write(markdown_table())
        sys.exit(0)
    rows = flag_docs()
    width = max(len(r[0]) for r in rows)
    for env, kind, dflt, doc in rows:
        print(f"{env:<{width}}  {kind:<6}  {dflt or '-':<12}  {doc}")
