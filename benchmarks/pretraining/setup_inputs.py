"""Prepare the inputs of a throughput recipe from files that are already on disk (no downloads).

    python benchmarks/pretraining/setup_inputs.py qwen3-30b-a3b

1. raw DCLM shards under ``workspace/datasets/dclm-baseline/rawtxt`` (``.jsonl`` / ``.jsonl.zst``) are tokenized into
   ``workspace/datasets/dclm-baseline/toktxt/<tokenizer dir>`` unless every shard already has its ``.bin``;
2. a Hugging Face release under ``workspace/checkpoints/<model>/hf-import`` is converted to the step-0 checkpoint
   ``workspace/checkpoints/<model>/torch-dcp/step-00000000`` unless that exists.
Either part is skipped with a message when its source is absent; the recipes then run on the synthetic token stream
and the seeded random initialisation. (The reference's setup step also fetches the shard and the release from the
hub, .agents/skills/setup-benchmark-inputs/scripts/setup.py; this machine class has no network.)
"""

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from benchmarks.pretraining.recipes import MODELS  # noqa: E402


def main() -> int:
    if len(sys.argv) != 2 or sys.argv[1] not in MODELS:
        print("usage: setup_inputs.py <" + "|".join(MODELS) + ">")
        return 2
    model = sys.argv[1]
    recipe = MODELS[model]
    ws = Path("workspace")
    raw = ws / "datasets" / "dclm-baseline" / "rawtxt"
    tok = ws / "datasets" / "dclm-baseline" / "toktxt" / recipe.tokens
    hf = ws / "checkpoints" / model / "hf-import"
    shards = [p for p in raw.rglob("*") if p.name.endswith((".jsonl", ".jsonl.zst"))] if raw.exists() else []
    if not shards:
        print(f"no raw shards under {raw}: the recipes will use the synthetic token stream")
    elif not hf.exists():
        print(f"no tokenizer under {hf}: cannot tokenize, the recipes will use the synthetic token stream")
    else:
        done = sum(1 for _ in tok.rglob("*.bin")) if tok.exists() else 0
        if done < len(shards) or any(tok.rglob("*.lock")):
            from pithtrain_b200.tasks.tokenize_corpus import TokenizeCorpusCfg, launch

            cfg = TokenizeCorpusCfg()
            cfg.tokenizer_name, cfg.source_path, cfg.output_path = str(hf), raw, tok
            launch(cfg)
        else:
            print(f"{done} tokenized shards already under {tok}")
    dcp = ws / "checkpoints" / model / "torch-dcp" / "step-00000000"
    if dcp.exists():
        print(f"step-0 checkpoint already at {dcp}")
    elif not any(hf.glob("*.safetensors")) if hf.exists() else True:
        print(f"no safetensors under {hf}: the recipes will start from the seeded random initialisation")
    else:
        from pithtrain_b200.tasks.convert_checkpoint import ConvertCheckpointCfg, launch as convert

        cfg = ConvertCheckpointCfg()
        cfg.operation, cfg.load_path, cfg.save_path = "hf2dcp", hf, dcp
        convert(cfg)
    return 0


if __name__ == "__main__":
    sys.exit(main())
