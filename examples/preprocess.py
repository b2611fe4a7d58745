"""Tokenize a text corpus into the binary format ``DatasetForCausalLM`` reads.

    python examples/preprocess.py --input corpus.jsonl --json-key text --output data/corpus
    python examples/preprocess.py --input notes.txt --output data/notes --tokenizer path/to/hf_tokenizer

Writes ``<output>.bin`` and ``<output>.idx`` (reference: oslo/data/preprocess/preprocessor.py:94-129). Without
``--tokenizer`` documents are encoded as UTF-8 bytes (ids 0-255, end of document 256), which needs no vocabulary
files; with it, any tokenizer directory that ``transformers.AutoTokenizer`` can open is used.
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
    ap.add_argument("--input", required=True, help=".jsonl (one object per line) or plain text")
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
    stats = pre.preprocess(documents(args.input, args.json_key), args.output, num_workers=args.workers)
    print(f"{args.output}.bin/.idx: {stats['documents']} documents, {stats['docs_per_s']:.0f} docs/s")


if __name__ == "__main__":
    main()
