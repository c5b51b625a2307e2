"""Attention forward / backward: the tcgen05 kernels of this package against the library's flash attention.

    python benchmarks/operators/bench_attention.py [--shapes qwen3,gpt-oss,long] [--iters 10]

Causal self-attention in the models' layouts (token-major q/k/v sliced out of one fused projection output). Each
figure is the median of ``--iters`` launches timed with CUDA events, with a 256 MB buffer written between launches so
that no operand is served from L2. FLOPs are counted as 4*S^2*Hq*D/2 for the forward and 2.5x that for the backward.
The library line (``torch`` SDPA on the cuDNN backend) is the comparison baseline only; nothing in the package calls it.
"""

import argparse
import sys
from pathlib import Path

import torch
import torch.nn.functional as F

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from pithtrain_b200 import _native  # noqa: E402
from pithtrain_b200.ops import attention_native as N  # noqa: E402

SHAPES = {
    "qwen3": (1, 4096, 32, 4, 128),      # Qwen3-30B-A3B layer at the benchmark's sequence length
    "long": (1, 8192, 32, 4, 128),
    "gpt-oss": (1, 4096, 64, 8, 64),     # GPT-OSS head geometry (full-attention layer)
}


def timeit(fn, iters, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    ts = []
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="qwen3,long,gpt-oss")
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    for name in a.shapes.split(","):
        B, S, Hq, Hkv, D = SHAPES[name]
        qkv = torch.randn(B, S, (Hq + 2 * Hkv) * D, device="cuda").bfloat16()
        q = qkv[..., :Hq * D].view(B, S, Hq, D)
        k = qkv[..., Hq * D:(Hq + Hkv) * D].view(B, S, Hkv, D)
        v = qkv[..., (Hq + Hkv) * D:].view(B, S, Hkv, D)
        fl = 4 * B * S * S * Hq * D / 2
        sc = D ** -0.5
        t = timeit(lambda: N.forward(q, k, v, sc, True, 0, None, None), a.iters)
        print(f"{name:8s} S={S} H={Hq}/{Hkv} D={D}  own forward   {t * 1e3:8.1f} us  {fl / t / 1e9:6.0f} TFLOP/s", flush=True)
        out, lse = N.forward(q, k, v, sc, True, 0, None, None)
        do = torch.randn_like(out)
        t = timeit(lambda: N.backward(do, q, k, v, out, lse, sc, True, 0, None), a.iters)
        print(f"{name:8s} S={S} H={Hq}/{Hkv} D={D}  own backward  {t * 1e3:8.1f} us  {2.5 * fl / t / 1e9:6.0f} TFLOP/s"
              "  (pre + main + post kernels and the accumulator memset)", flush=True)
        _native.check_status()
        qt, kt, vt = (x.transpose(1, 2) for x in (q, k, v))
        with torch.nn.attention.sdpa_kernel(torch.nn.attention.SDPBackend.CUDNN_ATTENTION):
            t = timeit(lambda: F.scaled_dot_product_attention(qt, kt, vt, is_causal=True, enable_gqa=True), a.iters)
            print(f"{name:8s} library forward   {t * 1e3:8.1f} us  {fl / t / 1e9:6.0f} TFLOP/s", flush=True)
            q2, k2, v2 = (x.detach().clone().requires_grad_() for x in (q, k, v))
            o = F.scaled_dot_product_attention(q2.transpose(1, 2), k2.transpose(1, 2), v2.transpose(1, 2), is_causal=True,
                                               enable_gqa=True)
            go = torch.randn_like(o)
            t = timeit(lambda: torch.autograd.grad(o, [q2, k2, v2], go, retain_graph=True), a.iters)
            print(f"{name:8s} library backward  {t * 1e3:8.1f} us  {2.5 * fl / t / 1e9:6.0f} TFLOP/s", flush=True)


if __name__ == "__main__":
    main()
