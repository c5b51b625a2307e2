"""A small attention case for Nsight Compute: two forward + backward passes of causal GQA attention
(1 x 4096 tokens, 16 query / 2 key-value heads of 128: 100 MB of operands, past L2 together with the fp32 accumulators).

    python benchmarks/operators/ncu_attention_case.py
    ncu --set full --clock-control none -k regex:attn_bwd_kernel -s 1 -c 1 -o prof_attn_bwd python benchmarks/operators/ncu_attention_case.py
"""

import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from pithtrain_b200 import _native  # noqa: E402
from pithtrain_b200.ops import attention_native as N  # noqa: E402

B, S, Hq, Hkv, D = 1, 4096, 16, 2, 128
qkv = torch.randn(B, S, (Hq + 2 * Hkv) * D, device="cuda").bfloat16()
q = qkv[..., :Hq * D].view(B, S, Hq, D)
k = qkv[..., Hq * D:(Hq + Hkv) * D].view(B, S, Hkv, D)
v = qkv[..., (Hq + Hkv) * D:].view(B, S, Hkv, D)
for _ in range(2):
    out, lse = N.forward(q, k, v, D ** -0.5, True, 0, None, None)
    do = torch.randn_like(out)
    N.backward(do, q, k, v, out, lse, D ** -0.5, True, 0, None)
torch.cuda.synchronize()
_native.check_status()
print("ok")
