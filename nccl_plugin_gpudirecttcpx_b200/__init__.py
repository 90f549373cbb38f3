"""B200-native NCCL net-transport plugin with the capabilities of nccl-plugin-gpudirecttcpx.

Layout:
  csrc/       C++17 host core, sm_100a CUDA kernels, plugin export, collective engine
  ops/        Python bindings of the device kernels (unpack / reduce / fan-out)
  parallel/   plugin loader for torch.distributed, hierarchical collectives, DDP harness
  models/     Llama-style decoder used by the data-parallel training benchmark
  utils/      native library loader, clocks sampling, timing helpers
"""
__version__ = "0.1.0"
