r"""CPU tier, several ranks: gloo processes exercise the multi-rank host logic (count exchange,
variable all-to-all layouts, capacity gates, SWIPE, grouped DDP, slice group, rank failure)."""
import pytest

from dist_launch import run_ranks


@pytest.mark.parametrize("case", ["ep_matches_bruteforce", "capacity_gates", "swipe_gate",
                                  "grouped_ddp", "slice_group", "smart_schedule",
                                  "smart_sch_entry_points", "shadow_policy"])
@pytest.mark.parametrize("world", [2, 4])
def test_cpu_ranks(case, world):
    codes = run_ranks("dist_cpu_worker.py", case, world, timeout=240)
    assert codes == [0] * world, codes


def test_pipeline_times_expert_parallelism():
    r"""2 pipeline stages x 2 expert-parallel ranks over gloo."""
    codes = run_ranks("dist_cpu_worker.py", "pipeline_hybrid", 4, timeout=240)
    assert codes == [0] * 4, codes


def test_gpt_example_with_pipeline_stages():
    r"""The fmoefy-ed GPT example as 2 pipeline stages x 2 expert-parallel ranks (gloo, tiny)."""
    import os
    script = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                          "examples", "gpt", "pretrain.py")
    argv = ["--fmoefy", "--num-experts", "2", "--top-k", "2", "--balance-strategy", "gshard",
            "--num-layers", "2", "--hidden-size", "32", "--num-attention-heads", "2",
            "--seq-length", "16", "--vocab-size", "64", "--micro-batch-size", "2", "--train-iters", "2",
            "--log-interval", "1", "--pipeline-model-parallel-size", "2", "--num-microbatches", "3",
            "--dtype", "fp32"]
    codes = run_ranks(script, None, 4, timeout=240, args=argv)
    assert codes == [0] * 4, codes


def test_hybrid_data_and_expert_parallelism():
    codes = run_ranks("dist_cpu_worker.py", "hybrid_dp_ep", 4, timeout=240)
    assert codes == [0] * 4, codes


def test_megatron_tensor_parallel_experts():
    codes = run_ranks("dist_cpu_worker.py", "tensor_parallel", 2, timeout=240)
    assert codes == [0, 0], codes


def test_rank_failure_is_detected():
    r"""Rank 1 exits before the collective; rank 0 must come back with an error, not hang."""
    codes = run_ranks("dist_cpu_worker.py", "rank_failure", 2, timeout=120, stop_on_failure=False)
    assert codes[1] == 3
    assert codes[0] == 0, codes


@pytest.mark.parametrize("case", ["megatron_checkpoint", "generic_checkpoint"])
def test_checkpoints_under_expert_parallelism(case, tmp_path):
    codes = run_ranks("dist_cpu_worker.py", case, 2, timeout=240,
                      extra_env={"FMOE_TEST_TMP": str(tmp_path)})
    assert codes == [0, 0], codes
