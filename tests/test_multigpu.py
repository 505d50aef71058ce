"""Fused compute+collective kernels across real GPUs (one process per GPU under torch.distributed.run)."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(world: int, script: str, timeout: int = 600, **extra_env):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", **extra_env)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), os.path.join(HERE, script)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-4000:]
    return r.stdout


@pytest.mark.parametrize("nvls", ["0", "1"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_collectives_and_tiny_model(world, nvls):
    """``nvls`` = 1: the symmetric blocks are bound to an NVLink multicast object when the machine offers one (the one-shot
    all-reduce pushes with multimem.st, the bulk all-reduce of the prompt path reduces in the switch); 0: plain peer
    loads and stores. Both must give the same tokens and bit-identical rows on every rank."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    out = _run(world, "multigpu_worker.py", IFAB_NVLS=nvls)
    assert out.count("ok tiny model") == world
    if nvls == "0":
        assert "nvls on" not in out


@pytest.mark.parametrize("world", [2, 4, 8])
def test_bulk_gemm_allreduce(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    out = _run(world, "multigpu_bulk_worker.py")
    assert out.count("ok gemm_allreduce bulk") == world


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ep_dispatch_combine_all_to_all(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    out = _run(world, "ep_worker.py")
    assert out.count("ok ep all-to-all") == world


def test_ep_dispatch_combine_single_rank():
    """World 1: the same kernels with every peer pointer local (plan, gather, grouped GEMMs, return, combine)."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("ep_worker", os.path.join(HERE, "ep_worker.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.run(0, 1)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_allgather_fused_into_gemm(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    out = _run(world, "ag_gemm_worker.py")
    assert out.count("ok allgather gemm") == world


@pytest.mark.parametrize("world", [2, 4])
def test_dense_decoder_tensor_parallel_decode_prefill_and_batched_rows(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    out = _run(world, "dense_worker.py")
    assert out.count("ok dense tensor parallel") == world


@pytest.mark.parametrize("world", [2, 4])
def test_compiled_programs_across_ranks(world):
    """The hyper-connected latent-attention + routed-experts program (also with packed caches and learned sparse attention) and
    the dense grouped-query program, compiled for the job's width and run by every rank's plan engine: logits equal the CPU interpreter's (this rank's vocabulary shard), every
    rank samples the same tokens, and the captured one-row step continues the sequence."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    out = _run(world, "program_worker.py")
    assert out.count("ok hyper program") == world and out.count("ok learned program") == world and out.count("ok dense program") == world
