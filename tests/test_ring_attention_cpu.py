"""Context-parallel ring attention on CPU ranks: every rank checks its zigzag slice against dense
attention over the whole sequence, gradients included (protocol of the reference's
tests/operators/test_ring_attention.py)."""
import pytest

from utilities import launch
import ring_worker


@pytest.mark.parametrize("cp,case", [(2, "mha"), (2, "gqa"), (4, "gqa"), (2, "window_sink"), (4, "window_sink"),
                                     (2, "mla"), (4, "mla"), (2, "gqa_d128_bf16")])
def test_ring_attention(cp, case):
    launch(cp, ring_worker.run, case)
