"""Import the Hugging Face release of deepseek-ai/DeepSeek-V2-Lite into a step-0 training checkpoint, or export one back.

    python examples/convert_checkpoint/deepseek-v2-lite/script.py            # HF -> DCP (default)
    python examples/convert_checkpoint/deepseek-v2-lite/script.py dcp2hf     # DCP -> HF

The Hugging Face files are expected under ``workspace/checkpoints/deepseek-v2-lite/hf-import`` (fetch them with
``huggingface-cli download deepseek-ai/DeepSeek-V2-Lite --local-dir workspace/checkpoints/deepseek-v2-lite/hf-import`` on a machine with network access).
"""

import sys
from pathlib import Path

from pithtrain_b200.tasks.convert_checkpoint import ConvertCheckpointCfg, launch

BASE = Path("workspace/checkpoints/deepseek-v2-lite")


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
