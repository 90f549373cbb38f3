"""The data-parallel harness on CPU: 2 gloo ranks, toy model.  Checks the host-side logic
(environment set-up is skipped for gloo, buckets, optimizer, replica agreement)."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from conftest import free_port

ROOT = Path(__file__).resolve().parent.parent


def _launch(nproc, extra, env=None, timeout=240):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()), "-m", "nccl_plugin_gpudirecttcpx_b200.parallel.ddp"] + extra
    e = dict(os.environ)
    e["PYTHONPATH"] = str(ROOT) + os.pathsep + e.get("PYTHONPATH", "")
    e.update(env or {})
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, cwd=str(ROOT), env=e)
    rows = [json.loads(l) for l in r.stdout.splitlines() if l.startswith('{"bench"')]
    return r, rows


def test_ddp_harness_two_cpu_ranks():
    r, rows = _launch(2, ["--backend", "gloo", "--tiny", "--steps", "3", "--warmup", "2", "--micro-batch", "2", "--bucket-mb", "1"])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert len(rows) == 1 and rows[0]["replicas_in_sync"] and rows[0]["world"] == 2
    assert rows[0]["loss_last"] < rows[0]["loss_first"] + 1.0


@pytest.mark.parametrize("nproc,gpn,buffer_kb", [(2, 1, 0), (4, 2, 0), (4, 2, 96)])
def test_ddp_buckets_through_the_engine_on_cpu_ranks(nproc, gpn, buffer_kb):
    """Gradient buckets averaged by the hierarchical engine (communication hook on the engine's asynchronous
    calls) on the stand-in device give the same training trajectory as gloo's own all_reduce; with 96 KiB
    symmetric buffers every bucket is larger than the buffers and travels in pieces."""
    common = ["--backend", "gloo", "--tiny", "--steps", "3", "--warmup", "2", "--micro-batch", "2", "--bucket-mb", "1"]
    env = {"PYTHONPATH": str(ROOT) + os.pathsep + str(ROOT / "tests"), "TCPXB_FAKE_GPU": "1", "OMP_NUM_THREADS": "1"}
    r, rows = _launch(nproc, common + ["--transport", "engine", "--engine-class", "standin_engine:StandinEngine",
                                       "--gpus-per-node", str(gpn), "--nics", "2", "--nthreads", "2",
                                       "--engine-buffer-kb", str(buffer_kb)], env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert len(rows) == 1 and rows[0]["replicas_in_sync"] and rows[0]["engine_buckets"] >= 5
    ref_r, ref = _launch(nproc, common, env={"OMP_NUM_THREADS": "1"})
    assert ref_r.returncode == 0 and len(ref) == 1
    assert abs(rows[0]["loss_last"] - ref[0]["loss_last"]) < 1e-3 and rows[0]["loss_first"] == ref[0]["loss_first"]


def test_llama_shapes_and_param_count():
    from nccl_plugin_gpudirecttcpx_b200.models import LlamaConfig, LlamaDecoder
    cfg = LlamaConfig.tiny()
    m = LlamaDecoder(cfg)
    tok = torch.randint(0, cfg.vocab_size, (2, 16))
    assert m(tok).shape == (2, 16, cfg.vocab_size)
    loss = m(tok, tok)
    loss.backward()
    assert all(p.grad is not None for p in m.parameters())
    full = LlamaConfig()
    per_layer = full.d_model * (full.d_model * 2 + 2 * full.d_model // 4) + 3 * full.d_model * full.ffn_dim + 2 * full.d_model
    assert per_layer * full.n_layers + full.vocab_size * full.d_model + full.d_model == 1235814400


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.parametrize("transport", ["plugin", "unpack"])
def test_ddp_step_over_the_plugin(transport):
    n = torch.cuda.device_count()
    world = 4 if n >= 4 else 2
    r, rows = _launch(world, ["--transport", transport, "--gpus-per-node", str(world // 2), "--tiny", "--steps", "3",
                              "--warmup", "2", "--nics", "2", "--nthreads", "2"])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert len(rows) == 1 and rows[0]["replicas_in_sync"]


@pytest.mark.gpu
def test_ddp_buckets_through_the_engine_one_gpu():
    """One GPU as its own network peer: every bucket goes through the transport and the fused kernels."""
    r, rows = _launch(1, ["--transport", "engine", "--tiny", "--steps", "3", "--warmup", "2", "--nics", "2", "--nthreads", "2"])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert len(rows) == 1 and rows[0]["replicas_in_sync"] and rows[0]["engine_buckets"] > 0
