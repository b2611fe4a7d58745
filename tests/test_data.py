"""Data utilities: byte-exact index files, packed causal-LM samples, C++ builders against NumPy oracles."""
import os
import struct

import numpy as np
import pytest
import torch

from oslo_b200 import data as D
from oslo_b200.data import cpp_builders
from oslo_b200.data.blending import build_blending_indices_numpy
from oslo_b200.data.datasets import build_sample_idx_numpy


class ToyTokenizer:
    eos_token_id = 1

    def encode(self, text):
        return [2 + (ord(c) % 50) for c in text]


DOCS = ["hello world " * 3, "the quick brown fox", "a", "pack my box with five dozen liquor jugs " * 4, "zz top"] * 7


@pytest.fixture(scope="module", autouse=True)
def built():
    from oslo_b200 import build
    build.build_data(verbose=False)
    assert cpp_builders.load() is not None


@pytest.mark.parametrize("impl", ["mmap", "lazy", "cached"])
def test_preprocess_and_read(tmp_path, impl):
    prefix = str(tmp_path / "toy")
    pre = D.DatasetPreprocessor(ToyTokenizer(), binarization_impl=impl)
    stats = pre.preprocess(DOCS, prefix, num_workers=0)
    assert stats["documents"] == len(DOCS)
    enc = [ToyTokenizer().encode(t.strip()) + [1] for t in DOCS]
    from oslo_b200.data.indexing import make_dataset
    ds = make_dataset(prefix, impl)
    assert len(ds) == len(DOCS)
    for i in (0, 3, len(DOCS) - 1):
        assert ds[i].tolist() == enc[i]
        assert ds.get(i, 2, 3).tolist() == enc[i][2:5]
    raw = open(prefix + ".idx", "rb").read()
    if impl == "mmap":
        assert raw[:9] == b"MMIDIDX\x00\x00" and struct.unpack("<Q", raw[9:17])[0] == 1 and raw[17] == 4
        n, ndoc = struct.unpack("<QQ", raw[18:34])
        assert n == len(DOCS) and ndoc == len(DOCS) + 1
        sizes = np.frombuffer(raw, dtype=np.int32, count=n, offset=34)
        ptrs = np.frombuffer(raw, dtype=np.int64, count=n, offset=34 + 4 * n)
        assert sizes.tolist() == [len(e) for e in enc]
        assert ptrs.tolist() == [4 * sum(len(e) for e in enc[:i]) for i in range(n)]
    else:
        assert raw[:8] == b"TNTIDX\x00\x00"
        code, esize = struct.unpack("<QQ", raw[16:32])
        assert (code, esize) == (4, 4)


@pytest.mark.parametrize("impl", ["mmap", "lazy"])
def test_causal_lm_dataset(tmp_path, impl):
    prefix = str(tmp_path / "toy")
    D.DatasetPreprocessor(ToyTokenizer(), binarization_impl=impl).preprocess(DOCS, prefix, num_workers=0)
    ds = D.DatasetForCausalLM(prefix, max_seq_length=16, binarization_impl=impl, seed=3)
    stream = []
    from oslo_b200.data.indexing import make_dataset
    store = make_dataset(prefix, impl)
    for d in ds.doc_idx:
        stream.extend(store[int(d)].tolist())
    assert len(ds) == (len(stream) - 1) // 15
    order = np.argsort(np.asarray(ds.shuffle_idx))
    for pos in (0, 1, len(ds) - 1):
        item = ds[int(order[pos])]  # sample number `pos` of the un-shuffled stream
        assert item["input_ids"].shape == (16,)
        assert item["input_ids"].tolist() == stream[pos * 15: pos * 15 + 16]
    again = D.DatasetForCausalLM(prefix, max_seq_length=16, binarization_impl=impl, seed=3)
    assert np.array_equal(np.asarray(again.shuffle_idx), np.asarray(ds.shuffle_idx))
    assert os.path.isfile(f"{prefix}_train_samples={len(DOCS)}_length=16_seed=3_sample_idx.npy")


def test_cpp_builders_match_numpy():
    cpp = cpp_builders.load()
    rng = np.random.RandomState(0)
    sizes = rng.randint(1, 40, size=200).astype(np.int32)
    doc_idx = rng.permutation(200).astype(np.int32)
    tokens = int(sizes.sum())
    for seq in (7, 16, 33):
        a = cpp.build_sample_idx(sizes, doc_idx, seq, 1, tokens)
        b = build_sample_idx_numpy(sizes, doc_idx, seq, 1, tokens)
        assert np.array_equal(a, b)
    w = np.array([0.5, 0.3, 0.2])
    di, si = np.zeros(1000, np.uint8), np.zeros(1000, np.int64)
    dj, sj = np.zeros(1000, np.uint8), np.zeros(1000, np.int64)
    cpp.build_blending_indices(di, si, w, 3, 1000)
    build_blending_indices_numpy(dj, sj, w, 3, 1000)
    assert np.array_equal(di, dj) and np.array_equal(si, sj)
    assert abs((di == 0).mean() - 0.5) < 0.01
    docs = np.array([0, 3, 4, 9, 12], dtype=np.int64)
    sent = rng.randint(3, 20, size=12).astype(np.int32)
    m = cpp.build_mapping(docs, sent, 2, 100, 32, 0.1, 5)
    assert m.shape[1] == 3 and len(m) > 0 and (m[:, 1] > m[:, 0]).all()
    assert np.array_equal(m, cpp.build_mapping(docs, sent, 2, 100, 32, 0.1, 5))
    blk = cpp.build_blocks_mapping(docs, sent, np.array([2, 2, 2, 2], np.int32), 1, 100, 32, 5)
    assert blk.shape[1] == 4 and (blk[:, 1] > blk[:, 0]).all() and set(blk[:, 2]) <= {0, 2, 3}


def test_blender_sampler_loader():
    class R(torch.utils.data.Dataset):
        def __init__(self, n, tag):
            self.n, self.tag = n, tag

        def __len__(self):
            return self.n

        def __getitem__(self, i):
            return (self.tag, i)

    b = D.DatasetBlender([R(30, "a"), R(10, "b")], weights=[0.5, 0.5])
    tags = [b[i][0] for i in range(len(b))]
    assert len(b) == 40 and abs(tags.count("a") - 20) <= 1
    base = torch.utils.data.SequentialSampler(range(10))
    parts = [list(D.DistributedProxySampler(base, num_replicas=2, rank=r, shuffle=False)) for r in range(2)]
    assert sorted(parts[0] + parts[1]) == list(range(10)) and not set(parts[0]) & set(parts[1])
    loader = D.InfiniteDataLoader(torch.utils.data.DataLoader(R(3, "x"), batch_size=2))
    seen = [next(loader) for _ in range(5)]
    assert len(seen) == 5 and loader.epoch == 2


@pytest.mark.parametrize("impl", ["mmap", "lazy"])
def test_builder_handles_and_index_helpers_of_the_reference_names(tmp_path, impl):
    """``DatasetBinarizer.create_builder``, ``PathUtils``, ``NumpyUtils``, ``MMapIndexedDataset.dtype`` and the public
    ``read_index`` / ``read_data`` of the lazy reader (oslo/data/indexing/__init__.py, lazy_indexing.py:165-264)."""
    prefix = str(tmp_path / "hand")
    idx, builder = D.DatasetBinarizer(impl).create_builder(prefix)
    assert idx == D.PathUtils.idx_path(prefix) == prefix + ".idx" and D.PathUtils.data_path(prefix) == prefix + ".bin"
    docs = [[5, 6, 7], [8], [9, 10]]
    for d in docs:
        builder.add_item(np.asarray(d, dtype=np.int32))
        builder.end_document()
    builder.finalize(idx)
    if impl == "mmap":
        ds = D.MMapIndexedDataset(prefix)
        assert ds.dtype == np.int32 and D.MmapIndex is D.MMapIndex
    else:
        ds = D.IndexedDataset(prefix)
        ds.read_index(prefix)
        ds.read_data(prefix)
        assert ds.data_file is not None and ds.num_tokens(2) == 2
    assert [ds[i].tolist() for i in range(3)] == docs
    assert D.NumpyUtils.dtypes_by_code[4] is np.int32 and D.NumpyUtils.cody_by_dtypes[np.uint16] == 8
    path = tmp_path / "arr.bin"
    with open(path, "wb") as f:
        D.NumpyUtils.write_file_from_array(f, [3, 1, 4, 1, 5])
    with open(path, "rb") as f:
        assert D.NumpyUtils.create_array_from_file(f, 5).tolist() == [3, 1, 4, 1, 5]
    with open(path, "rb") as f, pytest.raises(EOFError):
        D.NumpyUtils.create_array_from_file(f, 6)
