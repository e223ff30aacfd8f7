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


def tokenize_files(inputs, out_prefix: str, tok, vocab_size: int, text_key="text", seq_len=None, max_tokens_per_file=100_000_000,
                   masking=False) -> list:
    os.makedirs(os.path.dirname(os.path.abspath(out_prefix)), exist_ok=True)
    files, idx, w = [], 0, None

    def open_next():
        nonlocal idx, w
        name = f"{out_prefix}-{idx:03d}.bin"
        idx += 1
        files.append(name)
        w = TokenFileWriter(name, vocab_size, masking=masking)
        w.__enter__()

    open_next()
    for path in inputs:
        for rec in iter_documents(path, text_key):
            t, m = encode_record(tok, rec, text_key, seq_len)
            if w.n_tokens + len(t) > max_tokens_per_file and w.n_tokens > 0:
                w.__exit__(None, None, None)
                open_next()
            w.add_document(t, m if masking else None)
    w.__exit__(None, None, None)
    return files


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description="Tokenise text / jsonl files into BIN.TOK files")
    p.add_argument("inputs", nargs="+", help=".txt or .jsonl files ({text} or {prompt, response} records)")
    p.add_argument("--model", required=True, help="tokenizer to use (local directory or cached HF name)")
    p.add_argument("--out-dir", default="data")
    p.add_argument("--split", default="train")
    p.add_argument("--text-key", default="text")
    p.add_argument("--seq-len", type=int, default=None, help="pad / cut prompt-response pairs to this many tokens")
    p.add_argument("--masking", action="store_true", help="write a training mask (response tokens only)")
    p.add_argument("--max-tokens-per-file", type=int, default=100_000_000)
    a = p.parse_args(argv)
    tok = _load_tokenizer(a.model)
    files = tokenize_files(a.inputs, os.path.join(a.out_dir, a.split), tok, len(tok), a.text_key, a.seq_len, a.max_tokens_per_file, a.masking)
    print("wrote", *files)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
