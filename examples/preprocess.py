"""Tokenize a text corpus into the binary format ``DatasetForCausalLM`` reads.

    python examples/preprocess.py --input corpus.jsonl --json-key text --output data/corpus
    python examples/preprocess.py --input notes.txt --output data/notes --tokenizer path/to/hf_tokenizer
    python examples/preprocess.py --input-dir corpora/ --output data/ --small-first      # every .jsonl / .txt below corpora/

Writes ``<output>.bin`` and ``<output>.idx`` (reference: oslo/data/preprocess/preprocessor.py:94-129). Without
``--tokenizer`` documents are encoded as UTF-8 bytes (ids 0-255, end of document 256), which needs no vocabulary
files; with it, any tokenizer directory that ``transformers.AutoTokenizer`` can open is used.

``--input-dir`` converts a whole tree (the role of the reference's ``tests/utils/test_dataset_preprocessor.py``):
every ``.jsonl`` / ``.txt`` file below it becomes ``<output>/<relative path without extension>.bin/.idx``; finished
files are appended to ``<output>/done.txt``, so an interrupted batch continues with the files that are left.
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from oslo_b200.data import DatasetPreprocessor  # noqa: E402


class ByteTokenizer:
    """UTF-8 bytes as tokens: vocabulary 0-255 plus ``eos_token_id`` 256 (use ``vocab_size >= 257``)."""

    eos_token_id = 256
    vocab_size = 257

    def encode(self, text: str):
        return list(text.encode("utf-8"))

    def decode(self, ids) -> str:
        return bytes(int(i) for i in ids if 0 <= int(i) < 256).decode("utf-8", errors="replace")


def documents(path: str, json_key: str):
    if path.endswith(".jsonl"):
        yield from DatasetPreprocessor.open_jsonl(path, json_key)
    else:                       # plain text: blank lines separate documents
        with open(path, "r", encoding="utf-8") as f:
            doc = []
            for line in f:
                if line.strip():
                    doc.append(line)
                elif doc:
                    yield "".join(doc)
                    doc = []
            if doc:
                yield "".join(doc)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--input", help=".jsonl (one object per line) or plain text")
    ap.add_argument("--input-dir", help="convert every .jsonl / .txt file below this directory; --output is a directory")
    ap.add_argument("--small-first", action="store_true", help="--input-dir: smallest files first")
    ap.add_argument("--json-key", default="text")
    ap.add_argument("--output", required=True, help="prefix of the .bin / .idx pair")
    ap.add_argument("--tokenizer", help="directory of a Hugging Face tokenizer (default: UTF-8 bytes)")
    ap.add_argument("--impl", default="mmap", choices=["mmap", "lazy", "cached"])
    ap.add_argument("--workers", type=int, default=0, help="encoder processes (0: in this process)")
    args = ap.parse_args()
    if args.tokenizer:
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(args.tokenizer)
    else:
        tok = ByteTokenizer()
    pre = DatasetPreprocessor(tok, binarization_impl=args.impl, append_eod=True)
    if bool(args.input) == bool(args.input_dir):
        raise SystemExit("give exactly one of --input and --input-dir")
    if args.input:
        stats = pre.preprocess(documents(args.input, args.json_key), args.output, num_workers=args.workers)
        print(f"{args.output}.bin/.idx: {stats['documents']} documents, {stats['docs_per_s']:.0f} docs/s")
        return
    files = sorted(os.path.join(d, f) for d, _, fs in os.walk(args.input_dir) for f in fs if f.endswith((".jsonl", ".txt")))
    if args.small_first:
        files.sort(key=os.path.getsize)
    os.makedirs(args.output, exist_ok=True)
    record = os.path.join(args.output, "done.txt")
    done = set(open(record).read().split("\n")) if os.path.exists(record) else set()
    for path in files:
        rel = os.path.relpath(path, args.input_dir)
        if rel in done:
            print(f"{rel}: already converted")
            continue
        prefix = os.path.join(args.output, os.path.splitext(rel)[0])
        stats = pre.preprocess(documents(path, args.json_key), prefix, num_workers=args.workers)
        with open(record, "a") as f:                   # only after both files of the pair are complete
            f.write(rel + "\n")
        print(f"{prefix}.bin/.idx: {stats['documents']} documents, {stats['docs_per_s']:.0f} docs/s")


if __name__ == "__main__":
    main()
