"""Run one throughput recipe:  torchrun --nproc-per-node 8 benchmarks/pretraining/run.py qwen3-30b-a3b b200-1n8g/pp2-dp1-cp1-ep4-seq4096-bf16-gbs256

``--list`` prints every model and mesh. The trainer's rank-0 log carries tokens-per-second and peak memory per step.
"""

import argparse
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from benchmarks.pretraining.recipes import MODELS, make_cfg, parse_mesh  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("model", nargs="?")
    ap.add_argument("mesh", nargs="?")
    ap.add_argument("--list", action="store_true")
    ap.add_argument("--max-steps", type=int, default=25)
    ap.add_argument("--layers", type=int, default=None,
                    help="debug only: truncate the model to this many layers (a run with it is no benchmark number)")
    a = ap.parse_args()
    if a.list or not a.model:
        for name, r in MODELS.items():
            for mesh in r.meshes:
                print(f"{name:<18s}{mesh:<52s}{parse_mesh(mesh)['gpus']:4d} GPUs")
        return
    mesh = a.mesh or MODELS[a.model].meshes[0]
    cfg = make_cfg(a.model, mesh)
    cfg.training.max_steps = a.max_steps
    if a.layers is not None:
        cfg.training.num_hidden_layers_override = a.layers
    from pithtrain_b200.tasks.pretrain_lm import launch

    launch(cfg)


if __name__ == "__main__":
    main()
