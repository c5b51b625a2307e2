"""Tokenize DCLM-baseline shards with the Qwen/Qwen3.5-35B-A3B tokenizer into flat ``.bin`` token files.

Raw ``.jsonl`` / ``.jsonl.zst`` shards are read from ``workspace/datasets/dclm-baseline/rawtxt`` (any sub-tree of
``mlfoundations/dclm-baseline-1.0`` copied there); the tokenizer is loaded from the local Hugging Face cache or from
a directory path.
"""

from pathlib import Path

from pithtrain_b200.tasks.tokenize_corpus import TokenizeCorpusCfg, launch


def make_cfg() -> TokenizeCorpusCfg:
    cfg = TokenizeCorpusCfg()
    cfg.tokenizer_name = "Qwen/Qwen3.5-35B-A3B"
    cfg.source_path = Path("workspace/datasets/dclm-baseline/rawtxt")
    cfg.output_path = Path("workspace/datasets/dclm-baseline/toktxt/qwen3.5")
    return cfg


if __name__ == "__main__":
    launch(make_cfg())
