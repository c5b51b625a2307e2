"""Corpus tokenizer: shard format, EOS per document, dtype choice, resumability, dataset reading."""
import json

import numpy as np

import fake_tokenizer
from pithtrain_b200.modules.dataset import MemmapDataset
from pithtrain_b200.tasks.tokenize_corpus import TokenizeCorpusCfg, best_dtype, launch, output_name


def _cfg(src, out, workers=1):
    c = TokenizeCorpusCfg()
    c.tokenizer_name, c.source_path, c.output_path, c.num_workers = "bytes", src, out, workers
    c.tokenizer_factory = fake_tokenizer.factory
    return c


def _write(path, docs):
    path.parent.mkdir(parents=True, exist_ok=True)
    with open(path, "w") as f:
        for d in docs:
            f.write(json.dumps({"text": d}) + "\n")


def test_best_dtype():
    assert best_dtype(200) == np.uint8 and best_dtype(50000) == np.uint16 and best_dtype(151936) == np.uint32


def test_tokenize_and_resume(tmp_path):
    src, out = tmp_path / "raw", tmp_path / "tok"
    _write(src / "a" / "x.jsonl", ["hello", "wor ld"])
    _write(src / "y.jsonl", ["abc"] * 5)
    done = launch(_cfg(src, out))
    assert len(done) == 2
    with open(output_name(src / "a" / "x.jsonl", src, out), "rb") as f:
        tokens, splits = np.load(f), np.load(f)
    assert tokens.dtype == np.uint16
    assert tokens.tolist() == list(b"hello") + [256] + list(b"wor ld") + [256]
    assert splits.tolist() == [6, 13]
    assert launch(_cfg(src, out)) == []  # everything already done
    (out / "y.lock").touch()  # an interrupted shard is redone
    assert len(launch(_cfg(src, out))) == 1
    ds = MemmapDataset(out / "y.bin", sequence_length=4)
    tok, lab = ds[0]
    assert tok.tolist() == [97, 98, 99, 256] and lab.tolist() == [98, 99, 256, 97]


def test_parallel_leaders(tmp_path):
    src, out = tmp_path / "raw", tmp_path / "tok"
    for i in range(3):
        _write(src / f"f{i}.jsonl", [f"doc {i} {j}" for j in range(20)])
    done = launch(_cfg(src, out, workers=4))
    assert sorted(d[2] for d in done) == [20, 20, 20]
