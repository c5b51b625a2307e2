"""tcgen05 GEMM family against the library GEMMs (cuBLAS ``matmul``, ``F.grouped_mm``) on the model shape grid.

    python benchmarks/operators/bench_gemm.py [--quick]

Covers forward (NT), input gradient (NN) and weight gradient (TN, accumulating) of dense projections and of
the expert-grouped GEMMs at Qwen3-30B-A3B, DeepSeek-V2-Lite and GPT-OSS expert shapes; the reference's operator
bench walks the same kind of grid for its DeepGEMM path (benchmarks/operators/fp8/test_deepgemm.py:46-78 of the
reference). Prints one line per case: microseconds, TFLOP/s, fraction of the measured cuBLAS bf16 peak.
"""

import argparse
import sys
from pathlib import Path

import torch
import torch.nn.functional as F

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from benchmarks.operators.utilities import bench, peaks, rand_bf16  # noqa: E402
from pithtrain_b200 import _native  # noqa: E402
from pithtrain_b200.ops import gemm as G  # noqa: E402

PEAK = peaks()["bf16_tflops"]


def line(tag, flops, ms):
    tf = flops / ms / 1e9
    print(f"{tag:<58s}{ms * 1e3:10.1f} us{tf:9.0f} TF{tf / PEAK:7.2f} of measured", flush=True)


def dense(M, N, K):
    x, w, dy = rand_bf16(M, K), rand_bf16(N, K), rand_bf16(M, N)
    gw = torch.zeros(N, K, device="cuda", dtype=torch.bfloat16)
    fl = 2 * M * N * K
    line(f"dense fwd  NT {M}x{N}x{K} tcgen05 (CTA pairs, default)", fl, bench(lambda: G.gemm_nt(x, w)))
    G.USE_2CTA = False
    line(f"dense fwd  NT {M}x{N}x{K} tcgen05 (single CTA)", fl, bench(lambda: G.gemm_nt(x, w)))
    G.USE_2CTA = True
    line(f"dense fwd  NT {M}x{N}x{K} cuBLAS", fl, bench(lambda: torch.matmul(x, w.t())))
    line(f"dense dgrad NN {M}x{N}x{K} tcgen05", fl, bench(lambda: G.gemm_nn(dy, w)))
    line(f"dense dgrad NN {M}x{N}x{K} cuBLAS", fl, bench(lambda: torch.matmul(dy, w)))
    line(f"dense wgrad TN+acc {M}x{N}x{K} tcgen05", fl, bench(lambda: G.gemm_tn(dy, x, out=gw, accumulate=True)))
    line(f"dense wgrad TN+acc {M}x{N}x{K} cuBLAS addmm_", fl, bench(lambda: gw.addmm_(dy.t(), x)))
    _native.check_status()


def grouped(E, rows, H, I2):
    R = E * rows
    offs = torch.arange(0, R + 1, rows, dtype=torch.int32, device="cuda")
    xs, w, dy = rand_bf16(R, H), rand_bf16(E, I2, H), rand_bf16(R, I2)
    out, dx = torch.empty(R, I2, device="cuda", dtype=torch.bfloat16), torch.empty(R, H, device="cuda", dtype=torch.bfloat16)
    gw = torch.zeros(E, I2, H, device="cuda", dtype=torch.bfloat16)
    fl = 2 * R * H * I2
    tag = f"E={E} rows={rows} [{I2}x{H}]"
    line(f"grouped fwd   {tag} tcgen05", fl, bench(lambda: G.grouped_gemm_nt(xs, w, offs, out=out)))
    if hasattr(F, "grouped_mm"):
        line(f"grouped fwd   {tag} F.grouped_mm", fl, bench(lambda: F.grouped_mm(xs, w.transpose(1, 2), offs=offs[1:])))
    line(f"grouped dgrad {tag} tcgen05", fl, bench(lambda: G.grouped_gemm_nn(dy, w, offs, out=dx)))
    line(f"grouped wgrad {tag} tcgen05 (TMA reduce-add)", fl, bench(lambda: G.grouped_gemm_tn(dy, xs, offs, gw)))
    gw32 = torch.zeros(E, I2, H, device="cuda", dtype=torch.float32)
    line(f"grouped wgrad {tag} fp32 accumulators, two launches", 2 * fl,
         bench(lambda: (G.grouped_gemm_tn(dy, xs, offs, gw32, accumulate=True), G.grouped_gemm_tn(dy, xs, offs, gw32, accumulate=True))))
    line(f"grouped wgrad {tag} fp32 accumulators, paired launch", 2 * fl,
         bench(lambda: G.grouped_gemm_tn_pair(dy, xs, offs, dy, xs, offs, gw32)))
    if hasattr(F, "grouped_mm"):
        def lib_wgrad():
            gw.add_(F.grouped_mm(dy.t(), xs, offs=offs[1:]))
        line(f"grouped wgrad {tag} F.grouped_mm + add_", fl, bench(lib_wgrad))
    _native.check_status()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true")
    a = ap.parse_args()
    print(f"roofline denominator: {PEAK:.0f} TFLOP/s bf16 (cuBLAS burst, measured on this pool)")
    dense_grid = [(4096, 5120, 2048), (4096, 2048, 4096)] if a.quick else \
        [(4096, 5120, 2048), (4096, 2048, 4096), (4096, 4096, 2048), (8192, 8192, 8192), (4096, 151936, 2048)]
    for s in dense_grid:
        dense(*s)
    grouped_grid = [(128, 256, 2048, 1536)] if a.quick else \
        [(128, 256, 2048, 1536), (128, 256, 768, 2048), (32, 1024, 2048, 1536), (16, 2048, 2048, 1536),
         (64, 384, 2048, 2816), (32, 512, 2880, 5760)]
    for s in grouped_grid:
        grouped(*s)


if __name__ == "__main__":
    main()
