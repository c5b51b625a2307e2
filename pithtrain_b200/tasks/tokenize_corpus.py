"""Tokenize a corpus of ``.jsonl`` / ``.jsonl.zst`` files into packed ``.bin`` shards.

Each source file becomes ``<output_path>/<relative name>.bin`` holding two concatenated ``.npy``
arrays: the token ids of all documents (EOS appended to each) in the smallest unsigned dtype that
fits the vocabulary, then the cumulative document end offsets (uint64). Work is spread over a
two-level process tree: a few *leader* processes pull files largest-first from a shared queue and
each drives its own pool of encoder workers, so one huge file does not serialise the run. A
``<file>.lock`` sentinel marks work in progress; finished shards are skipped on restart. Same
on-disk format and resumability as pithtrain/tasks/tokenize_corpus.py:43-225.
"""

from __future__ import annotations

import json
import multiprocessing as mp
import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Iterator, List, Optional, Tuple

import numpy as np

from ..config import SlottedDefault
from ..contexts import logging
from ..modules.logging import LoggingCfg, setup_logging

SUFFIXES = (".jsonl", ".jsonl.zst", ".jsonl.zstd")


@dataclass(init=False, slots=True)
class TokenizeCorpusCfg(SlottedDefault):
    tokenizer_name: str
    """Local path (or cached hub id) of a Hugging Face tokenizer."""
    source_path: Path
    output_path: Path
    num_workers: int = max(1, (os.cpu_count() or 2) // 2)
    num_leaders: int = 0
    """Leader processes (0 = pick from ``num_workers``)."""
    tokenizer_factory: Optional[Callable[[str], object]] = None
    """Override for tests: ``factory(name)`` returns an object with ``encode``, ``vocab_size``, ``eos_token_id``."""
    logging: LoggingCfg = field(default_factory=LoggingCfg)


def read_file(path: Path) -> Iterator[str]:
    """Yield the ``"text"`` field of every JSON line."""
    suffix = "".join(path.suffixes[-2:]) if path.suffix in (".zst", ".zstd") else path.suffix
    if suffix in (".jsonl.zst", ".jsonl.zstd"):
        try:
            import zstandard as zstd
        except ImportError as e:  # pragma: no cover - optional dependency
            raise RuntimeError("reading .zst shards needs the `zstandard` package") from e
        with zstd.open(path, mode="rt") as f:
            for line in f:
                yield json.loads(line)["text"]
    elif suffix == ".jsonl":
        with open(path) as f:
            for line in f:
                if line.strip():
                    yield json.loads(line)["text"]
    else:
        raise ValueError("unsupported format: %s" % suffix)


def best_dtype(vocab_size: int):
    for dt in (np.uint8, np.uint16, np.uint32):
        if vocab_size < np.iinfo(dt).max:
            return dt
    return np.uint64


def load_tokenizer(name: str, factory=None):
    if factory is not None:
        return factory(name)
    os.environ["TOKENIZERS_PARALLELISM"] = "false"
    from transformers import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(name, local_files_only=True)
    tok.model_max_length = int(np.iinfo(np.int64).max)
    return tok


class _Encoder:
    """Per-process tokenizer state for pool workers."""

    tok = None
    dtype = None

    @classmethod
    def init(cls, name: str, factory) -> None:
        cls.tok = load_tokenizer(name, factory)
        cls.dtype = best_dtype(int(cls.tok.vocab_size))

    @classmethod
    def encode(cls, text: str) -> np.ndarray:
        ids = list(cls.tok.encode(text))
        ids.append(int(cls.tok.eos_token_id))
        return np.asarray(ids, dtype=cls.dtype)


def write_shard(path: Path, docs: List[np.ndarray], dtype) -> Tuple[int, int]:
    tokens = np.concatenate(docs, axis=0) if docs else np.zeros(0, dtype=dtype)
    splits = np.cumsum([d.shape[0] for d in docs], dtype=np.uint64) if docs else np.zeros(0, dtype=np.uint64)
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_suffix(path.suffix + ".tmp")
    with open(tmp, "wb") as f:
        np.save(f, tokens)
        np.save(f, splits)
    os.replace(tmp, path)
    return int(tokens.shape[0]), len(docs)


def output_name(src: Path, source_root: Path, output_root: Path) -> Path:
    rel = src.relative_to(source_root)
    name = rel.name
    for s in sorted(SUFFIXES, key=len, reverse=True):
        if name.endswith(s):
            name = name[: -len(s)]
            break
    return output_root / rel.parent / (name + ".bin")


def pending_files(cfg: TokenizeCorpusCfg) -> List[Path]:
    src = Path(cfg.source_path)
    files = [p for p in src.rglob("*") if p.is_file() and p.name.endswith(SUFFIXES)]
    todo = []
    for p in files:
        out = output_name(p, src, Path(cfg.output_path))
        lock = out.with_suffix(".lock")
        if out.exists() and not lock.exists():
            continue
        todo.append(p)
    return sorted(todo, key=lambda p: p.stat().st_size, reverse=True)


def _leader(cfg_items: dict, queue, workers: int, results) -> None:
    name, factory = cfg_items["tokenizer_name"], cfg_items["tokenizer_factory"]
    src_root, out_root = Path(cfg_items["source_path"]), Path(cfg_items["output_path"])
    pool = mp.get_context("spawn").Pool(workers, initializer=_Encoder.init, initargs=(name, factory)) if workers > 1 else None
    if pool is None:
        _Encoder.init(name, factory)
    try:
        while True:
            item = queue.get()
            if item is None:
                break
            src = Path(item)
            out = output_name(src, src_root, out_root)
            lock = out.with_suffix(".lock")
            lock.parent.mkdir(parents=True, exist_ok=True)
            lock.touch()
            texts = read_file(src)
            docs = list(pool.imap(_Encoder.encode, texts, chunksize=64)) if pool else [_Encoder.encode(t) for t in texts]
            dtype = docs[0].dtype if docs else np.uint32
            n_tok, n_doc = write_shard(out, docs, dtype)
            lock.unlink(missing_ok=True)
            results.put((str(src), n_tok, n_doc))
    finally:
        if pool is not None:
            pool.close()
            pool.join()


def launch(cfg: TokenizeCorpusCfg) -> List[Tuple[str, int, int]]:
    """Tokenize every pending source file; returns ``(file, tokens, documents)`` per shard written."""
    setup_logging(cfg)
    out = logging.stdout
    files = pending_files(cfg)
    out.info("tokenize_corpus: %d file(s) to process" % len(files))
    if not files:
        return []
    workers = max(1, int(cfg.num_workers))
    leaders = int(cfg.num_leaders) or max(1, min(len(files), workers // 4 or 1))
    per_leader = max(1, workers // leaders)
    items = dict(tokenizer_name=cfg.tokenizer_name, tokenizer_factory=cfg.tokenizer_factory,
                 source_path=str(cfg.source_path), output_path=str(cfg.output_path))
    ctx = mp.get_context("spawn")
    queue, results = ctx.Queue(), ctx.Queue()
    for f in files:
        queue.put(str(f))
    for _ in range(leaders):
        queue.put(None)
    if leaders == 1 and per_leader == 1:
        _leader(items, queue, 1, results)
    else:
        procs = [ctx.Process(target=_leader, args=(items, queue, per_leader, results)) for _ in range(leaders)]
        for p in procs:
            p.start()
        for p in procs:
            p.join()
        if any(p.exitcode != 0 for p in procs):
            raise RuntimeError("a tokenizer leader process failed")
    done = []
    for _ in range(len(files)):
        try:
            done.append(results.get(timeout=10))
        except Exception:
            break
    for src, n_tok, n_doc in done:
        out.info("tokenized %s: %s tokens in %d documents" % (src, format(n_tok, ","), n_doc))
    return done
