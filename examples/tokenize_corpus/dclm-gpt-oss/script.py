"""Tokenize DCLM-baseline shards with the openai/gpt-oss-20b tokenizer into flat ``.bin`` token files.

Raw ``.jsonl`` / ``.jsonl.zst`` shards are read from ``workspace/datasets/dclm-baseline/rawtxt`` (any sub-tree of
``mlfoundations/dclm-baseline-1.0`` copied there); the tokenizer is loaded from the local Hugging Face cache or from
a directory path.
"""

from pathlib import Path

from pithtrain_b200.tasks.tokenize_corpus import TokenizeCorpusCfg, launch


def make_cfg() -> TokenizeCorpusCfg:
    cfg = TokenizeCorpusCfg()
    cfg.tokenizer_name = "openai/gpt-oss-20b"
    cfg.source_path = Path("workspace/datasets/dclm-baseline/rawtxt")
    cfg.output_path = Path("workspace/datasets/dclm-baseline/toktxt/gpt-oss")
    return cfg


if __name__ == "__main__":
    launch(make_cfg())
