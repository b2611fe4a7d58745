"""Smaller reference features: TensorFlow checkpoint names, the ONNX export description of GPT-2, ZeRO-stage
detection under pipeline parallelism, and the two sentence-mapping index builders against NumPy statements."""
import sys
import types

import numpy as np
import pytest
import torch

import oslo_b200 as ob
from tests.dist_utils import run_distributed


def _tiny_gpt2():
    torch.manual_seed(0)
    return ob.GPT2LMHeadModel(ob.GPT2Config(vocab_size=61, n_positions=32, n_embd=16, n_layer=2, n_head=2))


def test_tf_variable_names_map_to_state_dict_keys():
    from oslo_b200.models.gpt2 import tf_name_to_key
    assert tf_name_to_key("model/wte") == "transformer.wte.weight"
    assert tf_name_to_key("model/wpe") == "transformer.wpe.weight"
    assert tf_name_to_key("model/h11/attn/c_attn/w") == "transformer.h.11.attn.c_attn.weight"
    assert tf_name_to_key("model/h0/mlp/c_proj/b") == "transformer.h.0.mlp.c_proj.bias"
    assert tf_name_to_key("model/h3/ln_2/g") == "transformer.h.3.ln_2.weight"
    assert tf_name_to_key("model/ln_f/b") == "transformer.ln_f.bias"
    assert tf_name_to_key("global_step") is None
    keys = set(_tiny_gpt2().state_dict())
    for name in ("model/h1/attn/c_proj/w", "model/h1/mlp/c_fc/b", "model/h0/ln_1/g", "model/wte"):
        assert tf_name_to_key(name) in keys


def test_tf_checkpoint_loader_fills_every_weight(monkeypatch):
    """A stand-in ``tensorflow.train`` serves the variables of an OpenAI-style checkpoint (projection weights stored
    with a leading 1-sized axis); after loading, the model computes what the source weights compute."""
    from oslo_b200.models.gpt2 import load_tf_weights_in_gpt2
    src = _tiny_gpt2().eval()
    store = {}
    for key, p in src.named_parameters():
        parts = key.replace("transformer.", "").split(".")
        arr = p.detach().numpy().copy()
        if parts[0] in ("wte", "wpe"):
            store["model/" + parts[0]] = arr
            continue
        leaf = {"weight": "g" if "ln_" in key else "w", "bias": "b"}[parts[-1]]
        mid = parts[:-1]
        if mid[0] == "h":
            mid = ["h" + mid[1]] + mid[2:]
        store["model/" + "/".join(mid + [leaf])] = arr[None] if arr.ndim == 2 else arr     # projections: [1, in, out]
    store["global_step"] = np.zeros(())
    fake = types.ModuleType("tensorflow")
    fake.train = types.SimpleNamespace(list_variables=lambda path: [(k, list(v.shape)) for k, v in store.items()],
                                       load_variable=lambda path, name: store[name])
    monkeypatch.setitem(sys.modules, "tensorflow", fake)
    torch.manual_seed(123)
    dst = ob.GPT2LMHeadModel(src.config).eval()
    ids = torch.randint(0, 61, (2, 8))
    assert not torch.allclose(dst(input_ids=ids).logits, src(input_ids=ids).logits)
    load_tf_weights_in_gpt2(dst, dst.config, "/nonexistent/model.ckpt")
    assert torch.allclose(dst(input_ids=ids).logits, src(input_ids=ids).logits, atol=1e-6)


def test_tf_checkpoint_loader_needs_tensorflow(monkeypatch):
    from oslo_b200.models.gpt2 import load_tf_weights_in_gpt2
    monkeypatch.setitem(sys.modules, "tensorflow", None)
    with pytest.raises(ImportError):
        load_tf_weights_in_gpt2(_tiny_gpt2(), None, "x")


def test_gpt2_onnx_config_describes_inputs_outputs_and_dummy_inputs():
    cfg = _tiny_gpt2().config
    oc = ob.GPT2OnnxConfig(cfg)
    assert list(oc.inputs) == ["input_ids", "attention_mask"] and list(oc.outputs) == ["last_hidden_state"]
    dummy = oc.generate_dummy_inputs(batch_size=3, seq_length=5)
    assert dummy["input_ids"].shape == (3, 5) and dummy["attention_mask"].shape == (3, 5)
    past = ob.GPT2OnnxConfig.with_past(cfg, task="causal-lm")
    assert list(past.outputs)[0] == "logits" and len(past.inputs) == 2 + 2 * cfg.n_layer
    d = past.generate_dummy_inputs()
    assert len(d["past_key_values"]) == cfg.n_layer and list(d) == ["input_ids", "past_key_values", "attention_mask"]
    k = d["past_key_values"][0][0]
    assert k.shape == (2, cfg.n_head, 10, cfg.n_embd // cfg.n_head) and d["attention_mask"].shape == (2, 18)
    # the dummy inputs run through the model
    model = _tiny_gpt2().eval()
    out = model(input_ids=d["input_ids"], past_key_values=d["past_key_values"], attention_mask=d["attention_mask"])
    assert out.logits.shape == (2, 8, cfg.vocab_size)


def _tiny_neo():
    torch.manual_seed(0)
    return ob.GPTNeoForCausalLM(ob.GPTNeoConfig(vocab_size=61, max_position_embeddings=32, hidden_size=16, num_layers=2,
                                                num_heads=2, window_size=4, attention_types=[[["global", "local"], 1]]))


def test_gpt_neo_tf_checkpoint_loader(monkeypatch):
    """Mesh-tensorflow variable names of the GPT-Neo release (projection matrices stored [in, out], a vocabulary padded
    beyond ``vocab_size``, optimizer slots beside the weights) against a stand-in ``tensorflow.train``."""
    from oslo_b200.models.gpt_neo.convert_tf import load_tf_weights_in_gpt_neo, tf_name_to_key
    assert tf_name_to_key("gpt2/h11/attn/q") == ("transformer.h.11.attn.attention.q_proj.weight", True)
    assert tf_name_to_key("gpt2/h0/attn/compute_output_bias/o_b") == ("transformer.h.0.attn.attention.out_proj.bias", False)
    assert tf_name_to_key("gpt2/h2/mlp/conv1d_main/c_proj/kernel") == ("transformer.h.2.mlp.c_proj.weight", True)
    assert tf_name_to_key("gpt2/h2/norm_2/g") == ("transformer.h.2.ln_2.weight", False)
    assert tf_name_to_key("gpt2/ln_f/b") == ("transformer.ln_f.bias", False)
    assert tf_name_to_key("gpt2/h2/attn/q/adam_m") is None and tf_name_to_key("global_step") is None
    src = _tiny_neo().eval()
    store = {}
    rev = {"q_proj": "q", "k_proj": "k", "v_proj": "v", "out_proj": "o"}
    for key, p in src.named_parameters():
        if key.startswith("lm_head"):
            continue
        parts = key.replace("transformer.", "").split(".")
        arr = p.detach().numpy().copy()
        if parts[0] in ("wte", "wpe"):
            if parts[0] == "wte":
                arr = np.concatenate([arr, np.zeros((3, arr.shape[1]), arr.dtype)])       # padded vocabulary
            store["gpt2/" + parts[0]] = arr
        elif parts[0] == "ln_f":
            store["gpt2/ln_f/" + ("g" if parts[-1] == "weight" else "b")] = arr
        else:
            h, rest = "gpt2/h" + parts[1], parts[2:]
            if rest[0] in ("ln_1", "ln_2"):
                store[f"{h}/norm_{rest[0][-1]}/" + ("g" if rest[-1] == "weight" else "b")] = arr
            elif rest[0] == "attn":
                if rest[-1] == "bias":
                    store[f"{h}/attn/compute_output_bias/o_b"] = arr
                else:
                    store[f"{h}/attn/{rev[rest[2]]}"] = arr.T.copy()
                    store[f"{h}/attn/{rev[rest[2]]}/adam_v"] = np.ones_like(arr)
            else:
                store[f"{h}/mlp/conv1d_main/{rest[1]}/" + ("kernel" if rest[-1] == "weight" else "bias")] = \
                    arr.T.copy() if rest[-1] == "weight" else arr
    store["global_step"] = np.zeros(())
    fake = types.ModuleType("tensorflow")
    fake.train = types.SimpleNamespace(list_variables=lambda path: [(k, list(v.shape)) for k, v in store.items()],
                                       load_variable=lambda path, name: store[name])
    monkeypatch.setitem(sys.modules, "tensorflow", fake)
    torch.manual_seed(5)
    dst = ob.GPTNeoForCausalLM(src.config).eval()
    ids = torch.randint(0, 61, (2, 8))
    assert not torch.allclose(dst(input_ids=ids).logits, src(input_ids=ids).logits)
    ob.load_tf_weights_in_gpt_neo(dst, dst.config, "/nonexistent/model.ckpt")
    assert torch.allclose(dst(input_ids=ids).logits, src(input_ids=ids).logits, atol=1e-6)
    assert dst.lm_head.weight.data_ptr() == dst.transformer.wte.weight.data_ptr()


def test_gpt_neo_onnx_config():
    cfg = _tiny_neo().config
    oc = ob.GPTNeoOnnxConfig.with_past(cfg, task="causal-lm")
    assert oc.num_layers == 2 and oc.num_attention_heads == 2
    assert list(oc.outputs)[0] == "logits" and len(oc.inputs) == 2 + 2 * 2
    d = oc.generate_dummy_inputs()
    assert d["past_key_values"][1][1].shape == (2, 2, 10, 8) and d["attention_mask"].shape == (2, 18)
    out = _tiny_neo().eval()(input_ids=d["input_ids"], past_key_values=d["past_key_values"],
                             attention_mask=d["attention_mask"])
    assert out.logits.shape == (2, 8, cfg.vocab_size)


class DeepSpeedEngine:          # recognised by class name when DeepSpeed itself is not installed
    def __init__(self, module, stage):
        self.module, self.stage = module, stage

    def zero_optimization(self):
        return self.stage > 0

    def zero_optimization_stage(self):
        return self.stage

    def __call__(self, **kw):
        engine = self            # noqa: F841 - DeepSpeed's own forward keeps the engine in a local of the calling frame
        return self.module(**kw)


def _zero_stage_ranks(rank, world):
    torch.manual_seed(0)
    cfg = ob.GPT2Config(vocab_size=61, n_positions=16, n_embd=16, n_layer=2, n_head=2)
    ids = torch.randint(0, 61, (2, 8))
    for stage, ok in ((1, True), (2, False), (3, False)):
        model = ob.parallelize(ob.GPT2LMHeadModel(cfg), pipeline_parallel_size=2, micro_batch_size=1)
        engine = DeepSpeedEngine(model.gpu_modules(), stage)
        if ok:
            for out in engine(input_ids=ids, labels=ids):
                out.loss.backward()
            assert model._pipe_engine.zero_stage == 1
        else:
            with pytest.raises(RuntimeError, match="ZeRO-2 and ZeRO-3"):
                engine(input_ids=ids, labels=ids)
    del engine                  # the lookup walks the callers' local variables: no engine may be left in this frame
    plain = ob.parallelize(ob.GPT2LMHeadModel(cfg), pipeline_parallel_size=2, micro_batch_size=1)
    for out in plain(input_ids=ids, labels=ids):
        out.loss.backward()
    assert plain._pipe_engine.zero_stage == 0


def test_pipeline_engine_refuses_zero_stage_2_and_3():
    """Reference behaviour (oslo/parallelism/engine_pipeline.py:270-278, :457-480): the stage of a DeepSpeed engine
    found in the calling frames decides; 0 / 1 run, 2 / 3 raise."""
    run_distributed(_zero_stage_ranks, 2)


# ---------------------------------------------------------------------------------------------------------------
# sentence-span index builders (C++: csrc/data_builders.cpp) against plain-Python statements of the same rules

def _py_mapping(docs, sizes, num_epochs, max_num_samples, max_seq_length, min_num_sent=2):
    """Greedy packing of whole sentences into samples of about ``max_seq_length`` tokens, document by document:
    a sample closes when it has reached the target and more than one sentence of the document is left, or when the
    document ends; documents with fewer than ``min_num_sent`` sentences or a sentence above 512 tokens are skipped.
    Rows: (first sentence, one past the last sentence, target length)."""
    rows = []
    for _epoch in range(num_epochs):
        for d in range(len(docs) - 1):
            first, last = int(docs[d]), int(docs[d + 1])
            remain = last - first
            if remain < min_num_sent or any(sizes[s] > 512 for s in range(first, last)):
                continue
            start, seq_len, num_sent = first, 0, 0
            for s in range(first, last):
                seq_len += int(sizes[s])
                num_sent += 1
                remain -= 1
                if (seq_len >= max_seq_length and remain > 1 and num_sent >= min_num_sent) or remain == 0:
                    if num_sent >= min_num_sent:
                        rows.append((start, s + 1, max_seq_length))
                        if len(rows) >= max_num_samples:
                            return rows
                    start, seq_len, num_sent = s + 1, 0, 0
    return rows


def _py_blocks(docs, sizes, titles, num_epochs, max_num_samples, max_seq_length, one_sent):
    """Blocks of whole sentences whose token budget is ``max_seq_length`` minus the document's title length.
    Rows: (first sentence, one past the last, document, running block id within the epoch)."""
    rows, min_sent = [], (1 if one_sent else 2)
    for _epoch in range(num_epochs):
        block_id = 0
        for d in range(len(docs) - 1):
            first, last = int(docs[d]), int(docs[d + 1])
            remain, budget = last - first, max_seq_length - int(titles[d])
            if remain < min_sent or any(sizes[s] > 512 for s in range(first, last)):
                continue
            start, seq_len, num_sent = first, 0, 0
            for s in range(first, last):
                seq_len += int(sizes[s])
                num_sent += 1
                remain -= 1
                if (seq_len >= budget and remain >= min_sent and num_sent >= min_sent) or remain == 0:
                    rows.append((start, s + 1, d, block_id))
                    block_id += 1
                    if len(rows) >= max_num_samples:
                        return rows
                    start, seq_len, num_sent = s + 1, 0, 0
    return rows


def _corpus(seed):
    rng = np.random.default_rng(seed)
    sent_per_doc = rng.integers(1, 12, size=40)
    docs = np.concatenate([[0], np.cumsum(sent_per_doc)]).astype(np.int64)
    sizes = rng.integers(3, 90, size=int(docs[-1])).astype(np.int32)
    sizes[rng.integers(0, len(sizes), size=2)] = 600          # two documents carry an over-long sentence
    titles = rng.integers(2, 12, size=len(docs) - 1).astype(np.int32)
    return docs, sizes, titles


@pytest.mark.parametrize("seed", [0, 1])
def test_build_mapping_matches_the_python_statement(seed):
    from oslo_b200.data import cpp_builders
    lib = cpp_builders.load()
    if lib is None:
        pytest.skip("_data_C.so is not built")
    docs, sizes, _ = _corpus(seed)
    for epochs, cap, max_len in ((1, 10 ** 6, 128), (2, 10 ** 6, 64), (3, 37, 100)):
        want = _py_mapping(docs, sizes, epochs, cap, max_len)
        got = lib.build_mapping(docs, sizes, epochs, cap, max_len, 0.0, 1234)
        assert got.shape == (len(want), 3)
        assert sorted(map(tuple, got.tolist())) == sorted(want)            # same samples; the order is shuffled
        again = lib.build_mapping(docs, sizes, epochs, cap, max_len, 0.0, 1234)
        assert np.array_equal(got, again), "the shuffle must be deterministic in the seed"
        other = lib.build_mapping(docs, sizes, epochs, cap, max_len, 0.0, 99)
        assert len(want) < 8 or not np.array_equal(got, other)
    # short sequences: every target stays within [2, max], spans still tile each document without gaps
    short = lib.build_mapping(docs, sizes, 1, 10 ** 6, 128, 0.5, 7)
    assert short[:, 2].min() >= 2 and short[:, 2].max() <= 128 and (short[:, 2] < 128).any()
    assert (short[:, 1] > short[:, 0]).all()


@pytest.mark.parametrize("one_sent", [False, True])
def test_build_blocks_mapping_matches_the_python_statement(one_sent):
    from oslo_b200.data import cpp_builders
    lib = cpp_builders.load()
    if lib is None:
        pytest.skip("_data_C.so is not built")
    docs, sizes, titles = _corpus(3)
    for epochs, cap, max_len in ((1, 10 ** 6, 128), (2, 10 ** 6, 72), (2, 25, 128)):
        want = _py_blocks(docs, sizes, titles, epochs, cap, max_len, one_sent)
        got = lib.build_blocks_mapping(docs, sizes, titles, epochs, cap, max_len, 5, use_one_sent_blocks=one_sent)
        assert got.shape == (len(want), 4)
        assert sorted(map(tuple, got.tolist())) == sorted(want)


def test_gptj_rotary_helper_functions_agree_with_the_model_path():
    """``fixed_pos_embedding`` / ``rotate_every_two`` / ``apply_rotary_pos_emb`` (the reference's module-level helpers,
    oslo/models/gptj/modeling_gptj.py:49-77) against the rotary op the model uses, with a position offset."""
    from oslo_b200 import ops
    x = torch.randn(2, 7, 3, 16)
    assert torch.equal(ob.rotate_every_two(torch.tensor([[[[1.0, 2.0, 3.0, 4.0]]]])), torch.tensor([[[[-2.0, 1.0, -4.0, 3.0]]]]))
    sincos = ob.fixed_pos_embedding(x[..., :8], 1, seq_len=12)
    assert sincos[0].shape == (12, 4) and sincos[1].dtype == torch.float32
    got = torch.cat((ob.apply_rotary_pos_emb(x[..., :8], sincos, offset=5), x[..., 8:]), -1)
    assert torch.allclose(got, ops.reference.rotary_interleaved(x, torch.arange(5, 12), 8), atol=1e-6)
    full = ob.apply_rotary_pos_emb(x, ob.fixed_pos_embedding(x))
    assert torch.allclose(full, ops.reference.rotary_interleaved(x, torch.arange(7), 16), atol=1e-6)


def test_fused_op_wrappers_take_the_reference_call_signatures():
    """``Fused*.apply`` and the function-style entry points with the reference's argument orders
    (oslo/fused_kernels_utils.py:260-479), against plain PyTorch statements."""
    import os
    import torch.nn.functional as F
    from oslo_b200 import fused_kernels_utils as fk
    torch.manual_seed(0)
    x, bias, res = torch.randn(4, 6, 8), torch.randn(8), torch.randn(4, 6, 8)
    assert torch.allclose(fk.FusedBiasDropout.apply(x, bias, False, 0.3), x + bias)
    assert torch.allclose(fk.FusedBiasDropoutResidual.apply(x, bias, res, False, 0.3), x + bias + res)
    assert torch.allclose(fk.bias_dropout_residual_inference(x, bias, res, 0.5), x + bias + res)
    dropped = fk.bias_dropout_train(torch.ones(64, 64), None, 0.5)
    assert 0.3 < float((dropped == 0).float().mean()) < 0.7 and float(dropped.max()) == 2.0
    want = F.gelu(x + bias, approximate="tanh")
    assert torch.allclose(fk.FusedBiasActivation.apply(x, bias, "gelu_new"), want, atol=1e-6)
    assert torch.allclose(fk.FusedBiasGeLU.apply(x, bias), want, atol=1e-6)
    assert torch.allclose(fk.bias_gelu_fwb(x, bias), want, atol=1e-6)
    xg = x.clone().requires_grad_(True)
    F.gelu(xg + bias, approximate="tanh").backward(res)
    assert torch.allclose(fk.bias_gelu_bwd(res, x, bias), xg.grad, atol=1e-5)
    # softmax: causal with an additive padding mask (the reference's convention) and with a boolean one; masked form
    s = torch.randn(2, 3, 5, 5)
    causal = torch.ones(5, 5, dtype=torch.bool).tril()
    ref = torch.softmax((s * 0.5).masked_fill(~causal, float("-inf")), -1)
    assert torch.allclose(fk.FusedScaleMaskSoftmax.apply(s, None, 0.5, True), ref, atol=1e-6)
    assert torch.allclose(fk.ScaledUpperTriangMaskedSoftmaxFunction.apply(s.view(6, 5, 5), 0.5).view(2, 3, 5, 5), ref, atol=1e-6)
    pad = torch.zeros(2, 1, 1, 5, dtype=torch.bool)
    pad[0, ..., 0] = True
    ref_pad = torch.softmax((s * 0.5).masked_fill(~causal | pad, float("-inf")), -1)
    got = fk.FusedScaleMaskSoftmax.apply(s, pad, 0.5, True)
    assert torch.allclose(got[1], ref_pad[1], atol=1e-6) and torch.allclose(got[0, :, 1:], ref_pad[0, :, 1:], atol=1e-4)
    add = torch.zeros(2, 1, 1, 5).masked_fill(pad, -1e4)
    assert torch.allclose(fk.FusedScaleMaskSoftmax.apply(s, add, 0.5, True)[0, :, 1:], ref_pad[0, :, 1:], atol=1e-4)
    sq = torch.randn(2, 3, 4, 5)
    ref_m = torch.softmax((sq * 2.0).masked_fill(pad, float("-inf")), -1)
    assert torch.allclose(fk.FusedScaleMaskSoftmax.apply(sq, pad, 2.0, False), ref_m, atol=1e-4)
    assert torch.allclose(fk.ScaledMaskedSoftmaxFunction.apply(sq, pad, 2.0), ref_m, atol=1e-4)
    assert torch.allclose(fk.FusedScaleMaskSoftmax.apply(sq, None, None, False), torch.softmax(sq, -1), atol=1e-6)
    assert fk.FusedScaleMaskSoftmax.is_available(torch.float16, 2, 3, 5, 5, True)
    assert not fk.FusedScaleMaskSoftmax.is_available(torch.float16, 2, 3, 4, 5, True)
    assert fk.FusedScaleMaskSoftmax.is_available(torch.bfloat16, 2, 3, 4, 5, False)
    assert not fk.FusedScaleMaskSoftmax.is_available(torch.int8, 2, 3, 4, 5, False)
    # n-gram blocking: after "7 8 7" the bigram (7, 8) bans 8
    tokens = torch.tensor([[7, 8, 7], [1, 2, 3]])
    lp = torch.zeros(2, 10)
    out = fk.NGramRepeatBlockFunction.apply(tokens, lp, 2, 2, 1, 2)
    assert out[0, 8] == float("-inf") and torch.isfinite(out[1]).all() and int(torch.isinf(out[0]).sum()) == 1
    # builder handles
    kb, db = fk.KernelBuilder(), fk.DatasetsBuilder()
    assert all(os.path.isfile(f) for f in kb.sources() + db.sources()) and os.path.isdir(kb.includes()[0])
    assert "-gencode" in kb.nvcc_args() and "-maxrregcount=64" in kb.nvcc_args(64)
    assert db.load() is not None and hasattr(db.load(), "build_sample_idx")
