"""DualPipeV engine on real GPUs (NCCL): same protocol as the CPU test, bf16 on the sm_100a kernels."""
import pytest
import torch

from utilities import launch
import dualpipev_worker

pytestmark = pytest.mark.gpu


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


@pytest.mark.parametrize("pp,ep", [(1, 2), (2, 1)])
def test_qwen3_two_gpus(pp, ep):
    _need(2)
    launch(2, dualpipev_worker.run, "qwen3_gpu", pp, ep, 2 * pp + 1, True, "cuda", backend="nccl")


def test_qwen3_pp2_ep2_four_gpus():
    _need(4)
    launch(4, dualpipev_worker.run, "qwen3_gpu", 2, 2, 5, True, "cuda", backend="nccl")
