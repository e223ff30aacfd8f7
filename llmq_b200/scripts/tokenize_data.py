"""``pyllmq-tokenize``: turns text / chat datasets into ``BIN.TOK`` files (train-*.bin / eval-*.bin).

Role of the reference's scripts/tokenize_data.py: documents are tokenised with the model's tokenizer, joined with EOS,
written as int32 tokens; fine-tuning sets (prompt/response pairs) get a training mask that covers the response only
and may be padded to a fixed sequence length.  Sources: a local text / jsonl file, or a Hugging Face dataset when the
``datasets`` package and a local cache are available (nothing is downloaded by this tool itself).
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Iterable, Optional, Tuple

import numpy as np

from ..training.dataloader import TokenFileWriter


def _load_tokenizer(model: str):
    from transformers import AutoTokenizer
    return AutoTokenizer.from_pretrained(model)


def iter_documents(path: str, text_key: str = "text") -> Iterable[dict]:
    """Yields {"text": ...} or {"prompt": ..., "response": ...} records from .txt (blank-line separated) or .jsonl."""
    if path.endswith(".jsonl"):
        with open(path) as f:
            for line in f:
                if line.strip():
                    yield json.loads(line)
    else:
        with open(path) as f:
            buf = []
            for line in f:
                if line.strip():
                    buf.append(line)
                elif buf:
                    yield {text_key: "".join(buf)}
                    buf = []
            if buf:
                yield {text_key: "".join(buf)}


def encode_record(tok, rec: dict, text_key: str, seq_len: Optional[int]) -> Tuple[np.ndarray, Optional[np.ndarray]]:
    eos = tok.eos_token_id
    if "prompt" in rec and "response" in rec:
        p = tok(rec["prompt"], add_special_tokens=False)["input_ids"]
        if tok.bos_token_id is not None:
            p = [tok.bos_token_id] + p
        r = tok(rec["response"], add_special_tokens=False)["input_ids"]
        tokens = np.array(p + r + [eos], dtype=np.int32)
        mask = np.concatenate([np.zeros(len(p)), np.ones(len(r) + 1)]).astype(bool)
        if seq_len:
            if len(tokens) > seq_len:
                tokens, mask = tokens[:seq_len], mask[:seq_len]
            pad = seq_len - len(tokens)
            tokens, mask = np.pad(tokens, (0, pad)), np.pad(mask, (0, pad))
        return tokens, mask
    ids = tok(rec[text_key], add_special_tokens=False)["input_ids"]
    return np.array(ids + [eos], dtype=np.int32), None


def default_workers() -> int:
    """Half the cores, at most 8 (the reference's pool size)."""
    return max(1, min((os.cpu_count() or 2) // 2, 8))


def _encode_stream(records: Iterable[dict], tok, text_key: str, seq_len: Optional[int], workers: int):
    """Encoded records in input order.  With several workers the tokenizer runs in a thread pool (the Rust tokenizers
    release the interpreter lock) with a bounded window of documents in flight, so a streamed dataset is never read
    ahead as a whole."""
    if workers <= 1:
        for rec in records:
            yield encode_record(tok, rec, text_key, seq_len)
        return
    import collections
    from concurrent.futures import ThreadPoolExecutor
    window = collections.deque()
    with ThreadPoolExecutor(max_workers=workers) as pool:
        for rec in records:
            window.append(pool.submit(encode_record, tok, rec, text_key, seq_len))
            if len(window) >= 8 * workers:
                yield window.popleft().result()
        while window:
            yield window.popleft().result()


def tokenize_records(records: Iterable[dict], out_prefix: str, tok, vocab_size: int, text_key="text", seq_len=None,
                     max_tokens_per_file=100_000_000, masking=False, single_file: bool = False, max_tokens: Optional[int] = None,
                     first_file: Optional[Tuple[str, int]] = None, workers: int = 1) -> list:
    """Writes the records to ``{out_prefix}-000.bin``, ``-001.bin``, ... (or ``{out_prefix}.bin`` with ``single_file``).

    ``first_file`` = (path, tokens): the first that many tokens go to a file of their own (an eval set cut off the
    head of a stream); ``max_tokens`` stops after about that many tokens in total."""
    os.makedirs(os.path.dirname(os.path.abspath(out_prefix)), exist_ok=True)
    files, idx, w, total = [], 0, None, 0
    limit = first_file[1] if first_file else max_tokens_per_file

    def open_next():
        nonlocal idx, w, limit
        if first_file and not files:
            name = first_file[0]
        else:
            name = f"{out_prefix}.bin" if single_file else f"{out_prefix}-{idx:03d}.bin"
            idx += 1
            limit = max_tokens_per_file
        files.append(name)
        w = TokenFileWriter(name, vocab_size, masking=masking)
        w.__enter__()

    open_next()
    for t, m in _encode_stream(records, tok, text_key, seq_len, workers):
        if not single_file and w.n_tokens + len(t) > limit and w.n_tokens > 0:
            w.__exit__(None, None, None)
            open_next()
        w.add_document(t, m if masking else None)
        total += len(t)
        if max_tokens and total >= max_tokens:
            break
    w.__exit__(None, None, None)
    return files


def tokenize_files(inputs, out_prefix: str, tok, vocab_size: int, text_key="text", seq_len=None, max_tokens_per_file=100_000_000,
                   masking=False, workers: int = 1) -> list:
    recs = (rec for path in inputs for rec in iter_documents(path, text_key))
    return tokenize_records(recs, out_prefix, tok, vocab_size, text_key, seq_len, max_tokens_per_file, masking, workers=workers)


# Named datasets of the reference's tool (scripts/tokenize_data.py:255-300 there): hub id, configuration, how a record
# becomes text or a (prompt, response) pair, where the eval set comes from (a split name, or the first N tokens of the
# stream), how many tokens to keep, whether the files are single small ones, and the fine-tuning defaults.
CLIMB_CLUSTERS = [86, 121, 145, 386, 189, 1778, 1673, 117, 81, 734, 156, 2568, 90, 28, 23, 728, 702, 227, 116, 51]    # relative sizes of clusters 1-20
DATASETS = {
    "tiny-shakespeare": dict(hub=("Trelis/tiny-shakespeare",), key="Text", eval="test", tiny=True),
    "tiny-stories": dict(hub=("roneneldan/TinyStories",), key="text", eval="validation"),
    "gsm8k": dict(hub=("openai/gsm8k", "main"), pair=("question", "answer"), eval="test", tiny=True, masking=True, seq_len=512),
    "limo": dict(hub=("GAIR/LIMO",), pair=("question", "solution"), eval="test", tiny=True, masking=True, seq_len=16383, holdout=40),
    "fineweb-1b": dict(hub=("HuggingFaceFW/fineweb", "sample-10BT"), key="text", eval=10_000_000, subsample=1_000_000_000, streaming=True),
    "fineweb-10b": dict(hub=("HuggingFaceFW/fineweb", "sample-10BT"), key="text", eval=10_000_000, streaming=True),
    "climb-1b": dict(hub=("gvlassis/ClimbMix",), clusters=CLIMB_CLUSTERS, key="text", eval=10_000_000, subsample=1_000_000_000, streaming=True),
    "climb-10b": dict(hub=("gvlassis/ClimbMix",), clusters=CLIMB_CLUSTERS, key="text", eval=10_000_000, subsample=10_000_000_000, streaming=True),
    "climb-20b": dict(hub=("gvlassis/ClimbMix",), clusters=CLIMB_CLUSTERS, key="text", eval=20_000_000, subsample=20_000_000_000, streaming=True),
}
TOKENIZERS = {"qwen": "Qwen/Qwen2.5-0.5B", "llama": "unsloth/llama-2-7b"}


def _load_named(spec, load_dataset):
    """The dataset as a {split: iterable} mapping.  ClimbMix is an interleaving of its 20 clusters in proportion to
    their sizes (seed 42, until all are exhausted); LIMO has no test split, so a fixed number of examples is held out."""
    if "clusters" in spec:
        from datasets import interleave_datasets
        total = float(sum(spec["clusters"]))
        parts = [load_dataset(spec["hub"][0], f"cluster_id={i + 1}", split="train", streaming=True) for i in range(len(spec["clusters"]))]
        return {"train": interleave_datasets(parts, probabilities=[c / total for c in spec["clusters"]], seed=42, stopping_strategy="all_exhausted")}
    d = load_dataset(*spec["hub"], **({"streaming": True} if spec.get("streaming") else {}))
    if "holdout" in spec:
        return d["train"].train_test_split(test_size=spec["holdout"], seed=42)
    return d


def _records(split, spec):
    if "pair" in spec:
        q, r = spec["pair"]
        return ({"prompt": ex[q], "response": ex[r]} for ex in split)
    return ({"text": ex[spec["key"]]} for ex in split)


def generate_tokenized_dataset(dataset: str, model: str, out_dir: str = "data", seq_len: Optional[int] = None, *, load_dataset=None,
                               tokenizer=None, workers: int = 1) -> list:
    """``--dataset NAME --model qwen|llama``: tokenises a named hub dataset into ``{out_dir}/{NAME}-{model}/``
    (``train.bin`` / ``train-000.bin``... and ``eval.bin``).  ``load_dataset`` / ``tokenizer`` can be passed in
    (tests do); by default they come from the ``datasets`` and ``transformers`` packages and their local caches."""
    if dataset not in DATASETS:
        raise ValueError(f"unknown dataset {dataset}; known: {', '.join(DATASETS)}")
    spec = DATASETS[dataset]
    short = model.lower()
    tok = tokenizer if tokenizer is not None else _load_tokenizer(TOKENIZERS.get(short, model))
    if load_dataset is None:
        try:
            from datasets import load_dataset
        except ImportError as e:
            raise RuntimeError("--dataset needs the `datasets` package; tokenise local .txt / .jsonl files instead") from e
    d = _load_named(spec, load_dataset)
    dst = os.path.join(out_dir, f"{dataset}-{short if short in TOKENIZERS else os.path.basename(model.rstrip('/'))}")
    masking = bool(spec.get("masking"))
    if seq_len is None:
        seq_len = spec.get("seq_len")
    elif seq_len <= 0:
        seq_len = None
    vocab, tiny = len(tok), bool(spec.get("tiny"))
    common = dict(text_key="text", seq_len=seq_len, masking=masking, workers=workers)
    if isinstance(spec["eval"], int):
        return tokenize_records(_records(d["train"], spec), os.path.join(dst, "train"), tok, vocab, max_tokens=spec.get("subsample"),
                                first_file=(os.path.join(dst, "eval.bin"), spec["eval"]), **common)
    files = tokenize_records(_records(d["train"], spec), os.path.join(dst, "train"), tok, vocab, single_file=tiny,
                             max_tokens=spec.get("subsample"), **common)
    return files + tokenize_records(_records(d[spec["eval"]], spec), os.path.join(dst, "eval"), tok, vocab, single_file=True, **common)


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description="Tokenise text / jsonl files, or a named hub dataset, into BIN.TOK files")
    p.add_argument("inputs", nargs="*", help=".txt or .jsonl files ({text} or {prompt, response} records)")
    p.add_argument("--dataset", default=None, help="named dataset instead of files: " + ", ".join(DATASETS))
    p.add_argument("--model", required=True, help="tokenizer to use: qwen, llama, a local directory or a cached HF name")
    p.add_argument("--out-dir", default="data")
    p.add_argument("--split", default="train")
    p.add_argument("--text-key", default="text")
    p.add_argument("--seq-len", type=int, default=None,
                   help="pad / cut prompt-response pairs to this many tokens (-1: no padding; default: the dataset's own)")
    p.add_argument("--masking", action="store_true", help="write a training mask (response tokens only)")
    p.add_argument("--max-tokens-per-file", type=int, default=100_000_000)
    p.add_argument("--workers", type=int, default=default_workers(), help="tokenizer threads")
    a = p.parse_args(argv)
    if a.dataset:
        print("wrote", *generate_tokenized_dataset(a.dataset, a.model, a.out_dir, a.seq_len, workers=a.workers))
        return 0
    if not a.inputs:
        p.error("give input files or --dataset")
    tok = _load_tokenizer(TOKENIZERS.get(a.model.lower(), a.model))
    files = tokenize_files(a.inputs, os.path.join(a.out_dir, a.split), tok, len(tok), a.text_key,
                           a.seq_len if a.seq_len and a.seq_len > 0 else None, a.max_tokens_per_file, a.masking, workers=a.workers)
    print("wrote", *files)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
