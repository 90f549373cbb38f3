"""Child process of the daemon test: one all_reduce on one GPU with the rx pool imported from
tcpxb_rxdm (memfd mapped and registered with CUDA) instead of the in-process pool."""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch

from nccl_plugin_gpudirecttcpx_b200.parallel.engine import HierarchicalEngine, default_transport_env


def main():
    default_transport_env(nics=2, nthreads=2, pool_mb=64)
    eng = HierarchicalEngine(gpus_per_node=1, request_bytes=1 << 20)
    x = torch.randn(3 << 20, device="cuda").to(torch.bfloat16)
    y = eng.all_reduce(x)
    torch.cuda.synchronize()
    ok = torch.equal(y, (x.float() * 2).to(torch.bfloat16)) and eng.device_status()[0] == 0
    eng.close()
    print("rxdm engine ok" if ok else "rxdm engine MISMATCH", flush=True)
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
