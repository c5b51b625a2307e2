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


@pytest.mark.parametrize("m,H,E,k", [(256, 512, 8, 2), (1000, 256, 16, 4)])
def test_fused_exchange_matches_all_to_all(m, H, E, k):
    _need(2)
    import ep_fused_worker

    launch(2, ep_fused_worker.run, m, H, E, k, backend="nccl")


def test_qwen3_ep2_fused_transport():
    _need(2)
    launch(2, dualpipev_worker.run, "qwen3_gpu", 1, 2, 3, True, "cuda", "fused", backend="nccl")


def test_qwen3_pp2_ep2_fused_transport_four_gpus():
    _need(4)
    launch(4, dualpipev_worker.run, "qwen3_gpu", 2, 2, 5, True, "cuda", "fused", backend="nccl")


def test_bounds_checking_build_catches_a_corrupted_send_plan():
    """The -DPT_BOUNDS_CHECK build of the library (pithtrain_b200/_lib/libpithb200_checked.so)."""
    from pathlib import Path

    _need(2)
    import ep_fused_worker

    if not (Path(__file__).resolve().parents[1] / "pithtrain_b200" / "_lib" / "libpithb200_checked.so").exists():
        pytest.skip("bounds-checking build not present: python -m pithtrain_b200.build --bounds-check")
    launch(2, ep_fused_worker.run_checked, 256, 512, 8, 2, backend="nccl")
