"""Tokenise text in worker processes and write an indexed token store.

``DatasetPreprocessor.preprocess(iterable_of_documents, "prefix")`` writes ``prefix.bin`` and ``prefix.idx``
(reference: oslo/data/preprocess/preprocessor.py:94-129, binarizer.py:73-102, encoder.py:41-53).
"""
from __future__ import annotations

import json
import logging
import os
import time
from concurrent.futures import ProcessPoolExecutor
from functools import lru_cache
from typing import Iterable, Iterator, Optional

import numpy as np

from .indexing import data_path, index_path, make_builder

logger = logging.getLogger(__name__)


class DatasetEncoder:
    """Callable that turns one document into token ids (+ end-of-document id)."""

    def __init__(self, tokenizer, append_eod: bool = True, eod_token_id: Optional[int] = None) -> None:
        self.tokenizer = tokenizer
        self.append_eod = append_eod
        self.eod_token_id = eod_token_id if eod_token_id is not None else getattr(tokenizer, "eos_token_id", None)
        if append_eod and self.eod_token_id is None:
            raise ValueError("append_eod=True needs eod_token_id or a tokenizer with eos_token_id")

    @lru_cache(maxsize=4096)
    def encode(self, text: str):
        text = text.strip()
        tok = self.tokenizer
        if hasattr(tok, "convert_tokens_to_ids") and hasattr(tok, "tokenize"):
            ids = tok.convert_tokens_to_ids(tok.tokenize(text))
        else:
            ids = list(tok.encode(text))
        if self.append_eod and ids:
            ids.append(self.eod_token_id)
        return ids, len(text)

    __call__ = encode


class DatasetBinarizer:
    def __init__(self, impl: str = "mmap", log_interval: int = 10000) -> None:
        self.impl, self.log_interval = impl, log_interval

    def create_builder(self, path: str):
        """``(index file path, builder writing <path>.bin)`` for this binarizer's format
        (reference: oslo/data/preprocess/binarizer.py:58-70)."""
        return index_path(path), make_builder(data_path(path), self.impl, np.int32)

    def binarize(self, encoded: Iterable, save_file_name: str) -> dict:
        builder = make_builder(data_path(save_file_name), self.impl, np.int32)
        t0 = time.time()
        docs = nbytes = 0
        for ids, n_chars in encoded:
            if not ids:
                continue
            builder.add_item(np.asarray(ids, dtype=np.int32))
            builder.end_document()
            docs += 1
            nbytes += n_chars
            if docs % self.log_interval == 0:
                dt = max(time.time() - t0, 1e-9)
                logger.info("binarized %d documents (%.1f docs/s, %.2f MiB/s)", docs, docs / dt, nbytes / dt / 2 ** 20)
        builder.finalize(index_path(save_file_name))
        dt = max(time.time() - t0, 1e-9)
        return {"documents": docs, "docs_per_s": docs / dt, "mib_per_s": nbytes / dt / 2 ** 20}


class DatasetPreprocessor:
    def __init__(self, tokenizer, chunksize: int = 1024, binarization_impl: str = "mmap", append_eod: bool = True,
                 eod_token_id: Optional[int] = None) -> None:
        if binarization_impl not in ("mmap", "lazy", "cached"):
            raise ValueError("binarization_impl must be one of 'mmap', 'lazy', 'cached'")
        self.encoder = DatasetEncoder(tokenizer, append_eod, eod_token_id)
        self.binarizer = DatasetBinarizer(binarization_impl)
        self.chunksize = chunksize

    def preprocess(self, data: Iterable[str], save_file_name: str, num_workers: Optional[int] = None,
                   log_interval: int = 10000) -> dict:
        """Encode ``data`` (an iterable of document strings) and write ``save_file_name.{bin,idx}``."""
        self.binarizer.log_interval = log_interval
        d = os.path.dirname(save_file_name)
        if d:
            os.makedirs(d, exist_ok=True)
        if num_workers == 0:
            return self.binarizer.binarize(map(self.encoder.encode, data), save_file_name)
        with ProcessPoolExecutor(max_workers=num_workers) as pool:
            encoded = pool.map(self.encoder.encode, data, chunksize=self.chunksize)
            return self.binarizer.binarize(encoded, save_file_name)

    @staticmethod
    def open_jsonl(file: str, json_key: str = "text") -> Iterator[str]:
        """Yield ``obj[json_key]`` for every line of a ``.jsonl`` file."""
        with open(file, "r", encoding="utf-8") as f:
            for line in f:
                line = line.strip()
                if line:
                    yield json.loads(line)[json_key]
