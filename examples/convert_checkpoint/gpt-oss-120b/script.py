"""Import the Hugging Face release of openai/gpt-oss-120b into a step-0 training checkpoint, or export one back.

    python examples/convert_checkpoint/gpt-oss-120b/script.py            # HF -> DCP (default)
    python examples/convert_checkpoint/gpt-oss-120b/script.py dcp2hf     # DCP -> HF

The Hugging Face files are expected under ``workspace/checkpoints/gpt-oss-120b/hf-import`` (fetch them with
``huggingface-cli download openai/gpt-oss-120b --local-dir workspace/checkpoints/gpt-oss-120b/hf-import`` on a machine with network access).
"""

import sys
from pathlib import Path

from pithtrain_b200.tasks.convert_checkpoint import ConvertCheckpointCfg, launch

BASE = Path("workspace/checkpoints/gpt-oss-120b")


def make_cfg(operation: str = "hf2dcp") -> ConvertCheckpointCfg:
    cfg = ConvertCheckpointCfg()
    cfg.operation = operation
    if operation == "hf2dcp":
        cfg.load_path = BASE / "hf-import"
        cfg.save_path = BASE / "torch-dcp" / "step-00000000"
    else:
        cfg.load_path = BASE / "torch-dcp" / "step-00000000"
        cfg.save_path = BASE / "hf-export"
    return cfg


if __name__ == "__main__":
    launch(make_cfg(sys.argv[1] if len(sys.argv) > 1 else "hf2dcp"))
