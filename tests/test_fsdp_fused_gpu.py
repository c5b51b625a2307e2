"""Reduce-scatter / parameter publication through peer memory against the NCCL collectives (2+ GPUs)."""
import pytest
import torch

from utilities import launch

import fsdp_fused_worker

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("grad_dtype", ["bf16", "fp32"])
def test_fused_shard_collectives_match_nccl(grad_dtype):
    n = min(torch.cuda.device_count(), 4)
    if n < 2:
        pytest.skip("needs 2 GPUs")
    launch(n, fsdp_fused_worker.run, grad_dtype, backend="nccl")
