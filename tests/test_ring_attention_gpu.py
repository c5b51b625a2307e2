"""Ring attention on GPUs: the payload travels through symmetric peer memory (publish / pull / gradient push)."""
import pytest
import torch

from utilities import launch

import ring_worker

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", ["gqa", "window_sink", "mla"])
def test_ring_attention_peer_pull(case):
    n = 4 if torch.cuda.device_count() >= 4 else 2
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    launch(n, ring_worker.run, case, "cuda", 4, backend="nccl")


def test_ring_attention_reads_peer_blocks_in_place():
    """bf16, head dim 128, no window: forward steps hand the attention kernel the address of the peer's published K/V
    (ops/ring_attention.py: IN_PLACE_REMOTE_BLOCKS), so its TMA loads fetch the block over NVLink while it computes."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    launch(2, ring_worker.run, "gqa_d128_bf16", "cuda", 3, backend="nccl")
