r"""GPU tier, several ranks (one process per GPU): fused peer-to-peer path vs the
collective-library path, the one-shot all-reduce, grouped DDP, bounded-wait time-out and
CUDA-graph replay of an expert-parallel step.  Skipped when fewer GPUs than ranks exist,
like the reference's distributed tests (``tests/test_ddp.py:31-33``)."""
import os

import pytest
import torch

from dist_launch import run_ranks

pytestmark = [pytest.mark.gpu]

# NVLS is switched off for these runs: no kernel here uses multimem, and a rank that died
# while bound to a multicast object could disturb the other GPUs.
ENV = {"NCCL_NVLS_ENABLE": "0"}
# Seconds a case may take before its ranks are killed (by pid).
TIMEOUT = int(os.environ.get("FMOE_TEST_TIMEOUT", "300"))


def _need(world):
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)


@pytest.mark.parametrize("case", ["fused_vs_general", "oracle", "exchange_tables", "uneven_tokens", "multi_layer",
                                  "recv_overflow", "shadow_fused", "swipe_device", "pipeline_gpu", "allreduce", "grouped_ddp", "wait_timeout",
                                  "graph_step", "smart_schedule", "slice_group", "capacity"])
def test_two_ranks(case):
    _need(2)
    codes = run_ranks("dist_gpu_worker.py", case, 2, timeout=TIMEOUT, extra_env=ENV)
    assert codes == [0, 0], codes


def test_nvls_allreduce():
    r"""Gradient all-reduce through NVSwitch multimem operations (``FMOE_USE_NVLS=1``)."""
    _need(2)
    codes = run_ranks("dist_gpu_worker.py", "allreduce_nvls", 2, timeout=TIMEOUT, extra_env=ENV)
    assert codes == [0, 0], codes


@pytest.mark.parametrize("case", ["fused_vs_general", "oracle", "exchange_tables", "multi_layer", "allreduce",
                                  "slice_group", "capacity", "smart_schedule"])
def test_many_ranks(case):
    world = int(os.environ.get("FMOE_TEST_WORLD", "4"))
    _need(world)
    codes = run_ranks("dist_gpu_worker.py", case, world, timeout=TIMEOUT, extra_env=ENV)
    assert codes == [0] * world, codes


@pytest.mark.parametrize("case", ["fused_vs_general", "oracle", "multi_layer", "graph_step"])
def test_one_rank_group(case):
    r"""The expert-parallel kernels (sender warps, arrival-gated tiles, return push, flags) in a
    one-rank process group: every peer table points at this GPU, so one GPU runs exactly the
    code of the multi-GPU path."""
    pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no GPU")
    env = dict(ENV)
    env["FMOE_FORCE_EP"] = "1"
    codes = run_ranks("dist_gpu_worker.py", case, 1, timeout=TIMEOUT, extra_env=env)
    assert codes == [0], codes


def test_data_parallel_in_one_process():
    r"""``nn.DataParallel`` replicas on several GPUs of one process (reference: tests/test_dp.py):
    the extension keeps per-device state, so replicas do not interfere."""
    _need(2)
    from fastmoe_b200 import FMoETransformerMLP
    torch.manual_seed(0)
    moe = FMoETransformerMLP(num_expert=4, d_model=64, d_hidden=128, top_k=2).cuda().to(torch.bfloat16)
    par = torch.nn.DataParallel(moe, device_ids=[0, 1])
    x = torch.randn(256, 64, device="cuda:0", dtype=torch.bfloat16)
    for _ in range(5):
        y = par(x)
    ref = moe(x)
    assert torch.allclose(y.float(), ref.float(), atol=3e-2, rtol=3e-2)
    from fastmoe_b200.ops import native
    assert native.get().read_status(0) == 0 and native.get().read_status(1) == 0
