"""DualPipeV engine on CPU ranks (gloo): schedule, p2p, expert exchange, deferred weight grads."""
import pytest

from utilities import launch
import dualpipev_worker


@pytest.mark.parametrize("pp,ep", [(1, 1), (2, 1), (1, 2), (2, 2)])
def test_qwen3_ladder(pp, ep):
    launch(pp * ep, dualpipev_worker.run, "qwen3", pp, ep, 2 * pp + 1)


@pytest.mark.parametrize("model", ["deepseek", "gpt_oss", "qwen35"])
def test_other_models_pp2_ep2(model):
    launch(4, dualpipev_worker.run, model, 2, 2, 5)


def test_qwen3_no_overlap_pp2():
    launch(2, dualpipev_worker.run, "qwen3", 2, 1, 6, False)


def test_qwen3_packed_sequences_pp2_ep2():
    """Two documents per micro-batch (cu_seqlens travel down the pipeline): same loss and gradients as the oracle."""
    launch(4, dualpipev_worker.run, "qwen3", 2, 2, 5, True, "cpu", "nccl", True, False)


def test_qwen3_forward_only_returns_oracle_logits():
    """``step`` under no_grad with return_outputs: the inference path of the pipeline."""
    launch(2, dualpipev_worker.run, "qwen3", 2, 1, 4, True, "cpu", "nccl", False, True)
