"""Small single-kernel cases sized for a profiler capture (a few launches, under 2 GB on the device, inputs
larger than the 126 MB L2 where the kernel is bandwidth-sensitive).

    python benchmarks/operators/ncu_case.py <case>          # plain run first; it must exit 0
    ncu --set full --clock-control none -k regex:<kernel> -s 3 -c 1 -o prof python benchmarks/operators/ncu_case.py <case>

Cases: gemm_dense (8192x8192x4096 bf16), gemm_grouped (128 experts x 256 rows, 1536x2048), wgrad_grouped
(K-grouped with TMA reduce-add), gemm_fp8 (8192x8192x4096 e4m3), gemm_fp8_grouped, quant_rows, rmsnorm, swiglu,
cross_entropy, gather_rows, combine, route_sort, router_topk, qk_norm_rope. Each case prints its CUDA-event time so the capture can be matched to an unprofiled number.
"""

import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from benchmarks.operators.utilities import rand_bf16  # noqa: E402
from pithtrain_b200 import _native  # noqa: E402
from pithtrain_b200.ops import gemm as G  # noqa: E402
from pithtrain_b200.ops import quant as Q  # noqa: E402


def case_gemm_dense():
    x, w = rand_bf16(8192, 4096), rand_bf16(8192, 4096)
    return (lambda: G.gemm_nt(x, w)), 2 * 8192 * 8192 * 4096, 0


def case_gemm_grouped():
    E, rows, H, N = 128, 256, 2048, 1536
    offs = torch.arange(0, E * rows + 1, rows, dtype=torch.int32, device="cuda")
    xs, w = rand_bf16(E * rows, H), rand_bf16(E, N, H)
    out = torch.empty(E * rows, N, device="cuda", dtype=torch.bfloat16)
    return (lambda: G.grouped_gemm_nt(xs, w, offs, out=out)), 2 * E * rows * H * N, 0


def case_wgrad_grouped():
    E, rows, H, N = 128, 256, 2048, 1536
    offs = torch.arange(0, E * rows + 1, rows, dtype=torch.int32, device="cuda")
    xs, dy = rand_bf16(E * rows, H), rand_bf16(E * rows, N)
    gw = torch.zeros(E, N, H, device="cuda", dtype=torch.bfloat16)
    return (lambda: G.grouped_gemm_tn(dy, xs, offs, gw)), 2 * E * rows * H * N, 0


def case_gemm_fp8():
    x, w = rand_bf16(8192, 4096), rand_bf16(8192, 4096)
    xq, xs = Q.quant_rows(x)
    wq, ws, _, _ = Q.quant_blocks(w, transposed=False)
    return (lambda: Q.gemm_fp8_nt(xq, xs, wq, ws)), 2 * 8192 * 8192 * 4096, 0


def case_gemm_fp8_grouped():
    E, rows, H, N = 128, 256, 2048, 1536
    offs = torch.arange(0, E * rows + 1, rows, dtype=torch.int32, device="cuda")
    xq, xs = Q.quant_rows(rand_bf16(E * rows, H))
    wq, ws, _, _ = Q.quant_blocks(rand_bf16(E, N, H), transposed=False)
    out = torch.empty(E * rows, N, device="cuda", dtype=torch.bfloat16)
    return (lambda: Q.gemm_fp8_nt(xq, xs, wq, ws, offs=offs, out=out)), 2 * E * rows * H * N, 0


def case_quant_rows():
    x = rand_bf16(65536, 2048)
    return (lambda: Q.quant_rows(x)), 0, 65536 * 2048 * 3


def case_rmsnorm():
    from pithtrain_b200.ops.norm import rmsnorm

    x, w = rand_bf16(65536, 2048), torch.ones(2048, device="cuda", dtype=torch.bfloat16)
    return (lambda: rmsnorm(x, w, 1e-6)), 0, 65536 * 2048 * 4


def case_swiglu():
    from pithtrain_b200.ops.moe import swiglu_fwd

    gu = rand_bf16(65536, 1536)
    return (lambda: swiglu_fwd(gu)), 0, 65536 * (1536 + 768) * 2


def case_cross_entropy():
    from pithtrain_b200.ops.cross_entropy import cross_entropy

    logits = rand_bf16(4096, 151936)
    labels = torch.randint(0, 151936, (4096,), device="cuda")
    return (lambda: cross_entropy(logits, labels)), 0, 4096 * 151936 * 2 * 3


def case_gather_rows():
    from pithtrain_b200.ops.moe import gather_rows

    x = rand_bf16(8192, 2048)
    idx = torch.randint(0, 8192 * 8, (65536,), device="cuda", dtype=torch.int32)
    return (lambda: gather_rows(x, idx, div=8)), 0, 65536 * 2048 * 2 * 2


def case_combine():
    from pithtrain_b200.ops.moe import combine_rows

    y = rand_bf16(65536, 2048)
    ros = torch.randperm(65536, device="cuda").int()
    w = torch.rand(8192, 8, device="cuda")
    return (lambda: combine_rows(y, ros, 8, w=w)), 0, (65536 + 8192) * 2048 * 2


def case_route_sort():
    from pithtrain_b200.ops.moe import route_sort

    eids = torch.randint(0, 128, (65536, 8), device="cuda", dtype=torch.int32)
    return (lambda: route_sort(eids, 128)), 0, 65536 * 8 * 4 * 4


def case_router_topk():
    from pithtrain_b200.ops.router import router_topk

    logits = rand_bf16(65536, 128)
    return (lambda: router_topk(logits, 8, "softmax_topk", True)), 0, 65536 * 128 * 2 + 65536 * (128 * 4 + 8 * 8)


def case_qk_norm_rope():
    from pithtrain_b200.ops.rope import qk_norm_rope

    n, Hq, Hkv, D = 32768, 32, 4, 128
    qkv = rand_bf16(n, (Hq + 2 * Hkv) * D)
    qw, kw = torch.ones(D, device="cuda", dtype=torch.bfloat16), torch.ones(D, device="cuda", dtype=torch.bfloat16)
    cos, sin = rand_bf16(4096, D), rand_bf16(4096, D)
    return (lambda: qk_norm_rope(qkv, qw, kw, cos, sin, Hq, Hkv, D, 1e-6, S=4096)), 0, n * (Hq + 2 * Hkv) * D * 2 * 2


def main():
    name = sys.argv[1] if len(sys.argv) > 1 else "gemm_dense"
    fn, flops, nbytes = globals()["case_" + name]()
    with torch.no_grad():
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(3):
            fn()
        b.record()
        torch.cuda.synchronize()
    _native.check_status()
    ms = a.elapsed_time(b) / 3
    extra = f"{flops / ms / 1e9:.0f} TFLOP/s" if flops else f"{nbytes / ms / 1e6:.0f} GB/s (algorithmic bytes)"
    print(f"{name}: {ms * 1e3:.1f} us per launch, {extra}")


if __name__ == "__main__":
    main()
