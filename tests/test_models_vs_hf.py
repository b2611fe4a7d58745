"""Single-process model numerics against the Hugging Face implementations (same weights, CPU fp32)."""
import os

import pytest
import torch

import oslo_b200 as ob

transformers = pytest.importorskip("transformers")


def _pair(kind):
    torch.manual_seed(0)
    if kind == "gpt2":
        cfg = ob.GPT2Config(vocab_size=97, n_positions=32, n_embd=48, n_layer=2, n_head=4,
                            resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
        ours = ob.GPT2LMHeadModel(cfg)
        hf_cfg = transformers.GPT2Config(vocab_size=97, n_positions=32, n_embd=48, n_layer=2, n_head=4,
                                         resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
        hf = transformers.GPT2LMHeadModel(hf_cfg)
    elif kind == "gpt_neo":
        cfg = ob.GPTNeoConfig(vocab_size=97, max_position_embeddings=32, hidden_size=48, num_layers=2, num_heads=4,
                              window_size=4, attention_types=[[["global", "local"], 1]])
        ours = ob.GPTNeoForCausalLM(cfg)
        hf_cfg = transformers.GPTNeoConfig(vocab_size=97, max_position_embeddings=32, hidden_size=48, num_layers=2,
                                           num_heads=4, window_size=4, attention_types=[[["global", "local"], 1]])
        hf = transformers.GPTNeoForCausalLM(hf_cfg)
    else:
        cfg = ob.GPTJConfig(vocab_size=97, n_positions=32, n_embd=48, n_layer=2, n_head=4, rotary_dim=8)
        ours = ob.GPTJForCausalLM(cfg)
        hf_cfg = transformers.GPTJConfig(vocab_size=97, n_positions=32, n_embd=48, n_layer=2, n_head=4, rotary_dim=8,
                                         resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
        hf = transformers.GPTJForCausalLM(hf_cfg)
    missing, unexpected = hf.load_state_dict(ours.state_dict(), strict=False)
    missing = [k for k in missing if not k.endswith((".attn.bias", ".attn.masked_bias", "attention.bias", "attention.masked_bias"))]
    assert not missing and not unexpected, (missing, unexpected)
    return ours.eval(), hf.eval()


@pytest.mark.parametrize("kind", ["gpt2", "gpt_neo", "gptj"])
def test_logits_and_loss_match_hf(kind):
    ours, hf = _pair(kind)
    x = torch.randint(0, 97, (2, 12))
    with torch.no_grad():
        a = ours(input_ids=x, labels=x)
        b = hf(input_ids=x, labels=x)
    assert torch.allclose(a.logits, b.logits, atol=2e-4, rtol=1e-4)
    assert torch.allclose(a.loss, b.loss, atol=1e-5)


@pytest.mark.parametrize("kind", ["gpt2", "gpt_neo", "gptj"])
def test_greedy_generate_matches_hf(kind):
    ours, hf = _pair(kind)
    x = torch.randint(0, 97, (2, 5))
    a = ours.generate(x, max_length=14, eos_token_id=None, pad_token_id=0)
    b = hf.generate(x, max_length=14, do_sample=False, eos_token_id=None, pad_token_id=0)
    assert torch.equal(a, b)


@pytest.mark.parametrize("kind", ["gpt2", "gptj"])
def test_fused_loss_without_logits(kind):
    ours, _ = _pair(kind)
    x = torch.randint(0, 97, (2, 12))
    with torch.no_grad():
        a = ours(input_ids=x, labels=x)
        ours.fuse()
        b = ours(input_ids=x, labels=x, output_logits=False)
    assert b.logits is None
    assert torch.allclose(a.loss, b.loss, atol=1e-5)


@pytest.mark.parametrize("kw", [
    dict(num_beams=3),
    dict(num_beams=4, no_repeat_ngram_size=2),
    dict(num_beams=1, repetition_penalty=1.3, no_repeat_ngram_size=2),
    dict(num_beams=3, length_penalty=0.6, early_stopping=True, eos_token_id=7, pad_token_id=0),
    dict(num_beams=2, min_length=10, eos_token_id=7, pad_token_id=0),
    dict(num_beams=4, num_return_sequences=3),
    dict(num_beams=1, bad_words_ids=[[5], [9, 11]]),
], ids=["beams", "beams_ngram", "penalty_ngram", "length_penalty_eos", "min_length", "return_sequences", "bad_words"])
def test_beam_search_and_logits_processors_match_hf(kw):
    """Beam search bookkeeping and the logits processors against Hugging Face's generate on the same weights."""
    ours, hf = _pair("gpt2")
    x = torch.randint(0, 97, (2, 5), generator=torch.Generator().manual_seed(3))
    args = dict(max_length=16, do_sample=False, eos_token_id=None, pad_token_id=0)
    args.update(kw)
    a = ours.generate(x, **args)
    b = hf.generate(x, **args)
    assert a.shape == b.shape and torch.equal(a, b)


def _load_into_hf(ours, hf):
    missing, unexpected = hf.load_state_dict(ours.state_dict(), strict=False)
    missing = [k for k in missing if not k.endswith((".attn.bias", ".attn.masked_bias", "attention.bias", "attention.masked_bias"))]
    assert not missing and not unexpected, (missing, unexpected)
    return ours.eval(), hf.eval()


@pytest.mark.parametrize("kind", ["gpt2", "gpt_neo", "gptj"])
def test_sequence_classification_heads_match_hf(kind):
    torch.manual_seed(0)
    common = dict(num_labels=3, pad_token_id=0)
    if kind == "gpt2":
        kw = dict(vocab_size=97, n_positions=32, n_embd=48, n_layer=2, n_head=4, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
        ours, hf = ob.GPT2ForSequenceClassification(ob.GPT2Config(**kw, **common)), \
            transformers.GPT2ForSequenceClassification(transformers.GPT2Config(**kw, **common))
    elif kind == "gpt_neo":
        kw = dict(vocab_size=97, max_position_embeddings=32, hidden_size=48, num_layers=2, num_heads=4, window_size=4,
                  attention_types=[[["global", "local"], 1]])
        ours, hf = ob.GPTNeoForSequenceClassification(ob.GPTNeoConfig(**kw, **common)), \
            transformers.GPTNeoForSequenceClassification(transformers.GPTNeoConfig(**kw, **common))
    else:
        kw = dict(vocab_size=97, n_positions=32, n_embd=48, n_layer=2, n_head=4, rotary_dim=8)
        ours, hf = ob.GPTJForSequenceClassification(ob.GPTJConfig(**kw, **common)), \
            transformers.GPTJForSequenceClassification(transformers.GPTJConfig(**kw, resid_pdrop=0.0, embd_pdrop=0.0,
                                                                               attn_pdrop=0.0, **common))
    ours, hf = _load_into_hf(ours, hf)
    x = torch.randint(1, 97, (3, 9))
    x[1, 6:] = 0                                   # right padding: the pooled position is the last non-pad token
    labels = torch.tensor([0, 2, 1])
    with torch.no_grad():
        a, b = ours(input_ids=x, labels=labels), hf(input_ids=x, labels=labels)
    assert torch.allclose(a.logits, b.logits, atol=2e-4, rtol=1e-4)
    assert torch.allclose(a.loss, b.loss, atol=1e-5)


def test_cache_modes_generate_the_same_tokens():
    """Static in-place cache (default), grow-by-cat tuple cache (the reference's) and no cache at all agree."""
    torch.manual_seed(0)
    model = ob.GPTJForCausalLM(ob.GPTJConfig(vocab_size=97, n_positions=64, n_embd=48, n_layer=2, n_head=4, rotary_dim=8)).eval()
    x = torch.randint(0, 97, (3, 5))
    want = model.generate(x, max_length=20, do_sample=False)
    assert torch.equal(want, model.generate(x, max_length=20, do_sample=False, use_static_cache=False))
    assert torch.equal(want, model.generate(x, max_length=20, do_sample=False, use_cache=False))


@pytest.mark.parametrize("kind", ["gpt2", "gpt_neo", "gptj"])
def test_checkpoints_interchange_with_hf(kind, tmp_path):
    """A directory written by Hugging Face (config.json + model.safetensors) loads here, and a directory written here
    (config.json + pytorch_model.bin) loads in Hugging Face, with identical logits."""
    torch.manual_seed(0)
    if kind == "gpt2":
        hf = transformers.GPT2LMHeadModel(transformers.GPT2Config(vocab_size=97, n_positions=32, n_embd=48, n_layer=2, n_head=4))
        cls = ob.GPT2LMHeadModel
    elif kind == "gpt_neo":
        hf = transformers.GPTNeoForCausalLM(transformers.GPTNeoConfig(
            vocab_size=97, max_position_embeddings=32, hidden_size=48, num_layers=2, num_heads=4, window_size=4,
            attention_types=[[["global", "local"], 1]]))
        cls = ob.GPTNeoForCausalLM
    else:
        hf = transformers.GPTJForCausalLM(transformers.GPTJConfig(vocab_size=97, n_positions=32, n_embd=48, n_layer=2,
                                                                  n_head=4, rotary_dim=8))
        cls = ob.GPTJForCausalLM
    hf.eval()
    x = torch.randint(0, 97, (2, 9))
    hf.save_pretrained(tmp_path / "hf")
    ours = cls.from_pretrained(str(tmp_path / "hf")).eval()
    with torch.no_grad():
        want = hf(input_ids=x).logits
        assert torch.allclose(ours(input_ids=x).logits, want, atol=2e-4, rtol=1e-4)
    ours.save_pretrained(str(tmp_path / "ours"))
    back = type(hf).from_pretrained(tmp_path / "ours").eval()
    with torch.no_grad():
        assert torch.allclose(back(input_ids=x).logits, want, atol=2e-4, rtol=1e-4)


def test_sharded_hf_checkpoints_load(tmp_path):
    """Multi-file checkpoints (`*.index.json` + shard files), as large models are published: the safetensors shards
    Hugging Face writes, and legacy `pytorch_model-0000x-of-0000y.bin` shards."""
    import json
    torch.manual_seed(0)
    hf = transformers.GPTJForCausalLM(transformers.GPTJConfig(vocab_size=97, n_positions=32, n_embd=48, n_layer=2,
                                                              n_head=4, rotary_dim=8)).eval()
    x = torch.randint(0, 97, (2, 9))
    with torch.no_grad():
        want = hf(input_ids=x).logits
    hf.save_pretrained(tmp_path / "st", max_shard_size="60KB")
    assert (tmp_path / "st" / "model.safetensors.index.json").is_file() and not (tmp_path / "st" / "model.safetensors").exists()
    ours = ob.GPTJForCausalLM.from_pretrained(str(tmp_path / "st")).eval()
    with torch.no_grad():
        assert torch.allclose(ours(input_ids=x).logits, want, atol=2e-4, rtol=1e-4)

    ours.save_pretrained(str(tmp_path / "one"))                     # re-cut our single file into two .bin shards
    state = torch.load(tmp_path / "one" / "pytorch_model.bin", weights_only=True)
    keys = sorted(state)
    shards = {"pytorch_model-00001-of-00002.bin": keys[: len(keys) // 2], "pytorch_model-00002-of-00002.bin": keys[len(keys) // 2:]}
    (tmp_path / "bins").mkdir()
    for name, ks in shards.items():
        torch.save({k: state[k] for k in ks}, tmp_path / "bins" / name)
    json.dump({"metadata": {}, "weight_map": {k: n for n, ks in shards.items() for k in ks}},
              open(tmp_path / "bins" / "pytorch_model.bin.index.json", "w"))
    (tmp_path / "bins" / "config.json").write_text((tmp_path / "one" / "config.json").read_text())
    again = ob.GPTJForCausalLM.from_pretrained(str(tmp_path / "bins")).eval()
    with torch.no_grad():
        assert torch.allclose(again(input_ids=x).logits, want, atol=2e-4, rtol=1e-4)
    os.remove(tmp_path / "bins" / "pytorch_model-00002-of-00002.bin")
    with pytest.raises(FileNotFoundError, match="missing"):
        ob.GPTJForCausalLM.from_pretrained(str(tmp_path / "bins"))


def test_logits_processors_match_hf():
    """Each logits processor / warper against Hugging Face's on random scores (bad-words, forced tokens included)."""
    import transformers.generation.logits_process as hlp
    from oslo_b200.generation import logits_process as lp
    torch.manual_seed(0)
    ids = torch.randint(0, 50, (4, 9))
    scores = torch.randn(4, 50)
    pairs = [
        (lp.TemperatureLogitsWarper(0.7), hlp.TemperatureLogitsWarper(0.7)),
        (lp.TopKLogitsWarper(5), hlp.TopKLogitsWarper(5)),
        (lp.TopKLogitsWarper(3, min_tokens_to_keep=4), hlp.TopKLogitsWarper(3, min_tokens_to_keep=4)),
        (lp.TopPLogitsWarper(0.8), hlp.TopPLogitsWarper(0.8)),
        (lp.TopPLogitsWarper(0.3, min_tokens_to_keep=2), hlp.TopPLogitsWarper(0.3, min_tokens_to_keep=2)),
        (lp.RepetitionPenaltyLogitsProcessor(1.4), hlp.RepetitionPenaltyLogitsProcessor(1.4)),
        (lp.NoRepeatNGramLogitsProcessor(2), hlp.NoRepeatNGramLogitsProcessor(2)),
        (lp.NoRepeatNGramLogitsProcessor(3), hlp.NoRepeatNGramLogitsProcessor(3)),
        (lp.MinLengthLogitsProcessor(12, 3), hlp.MinLengthLogitsProcessor(12, 3)),
        (lp.InfNanRemoveLogitsProcessor(), hlp.InfNanRemoveLogitsProcessor()),
    ]
    for ours, theirs in pairs:
        a, b = ours(ids, scores.clone()), theirs(ids, scores.clone())
        assert torch.allclose(a, b, equal_nan=True), type(ours).__name__


def test_gpt2_double_heads_matches_hf():
    torch.manual_seed(0)
    kw = dict(vocab_size=97, n_positions=32, n_embd=48, n_layer=2, n_head=4, resid_pdrop=0.0, embd_pdrop=0.0,
              attn_pdrop=0.0, summary_first_dropout=0.0, num_labels=1)
    ours, hf = _load_into_hf(ob.GPT2DoubleHeadsModel(ob.GPT2Config(**kw)),
                             transformers.GPT2DoubleHeadsModel(transformers.GPT2Config(**kw)))
    x = torch.randint(0, 97, (2, 3, 9))
    mc, mc_labels = torch.tensor([[8, 5, 7], [2, 8, 4]]), torch.tensor([1, 2])
    with torch.no_grad():
        a = ours(input_ids=x, mc_token_ids=mc, labels=x, mc_labels=mc_labels)
        b = hf(input_ids=x, mc_token_ids=mc, labels=x, mc_labels=mc_labels)
    assert torch.allclose(a.logits, b.logits, atol=2e-4, rtol=1e-4) and torch.allclose(a.mc_logits, b.mc_logits, atol=2e-4)
    assert torch.allclose(a.loss, b.loss, atol=1e-5) and torch.allclose(a.mc_loss, b.mc_loss, atol=1e-5)


@pytest.mark.parametrize("kind", ["gpt2", "gpt_neo", "gptj"])
def test_masks_attentions_hidden_states_and_embeds_match_hf(kind):
    """Left padding through ``attention_mask``, ``output_attentions``, ``output_hidden_states`` and ``inputs_embeds``."""
    ours, hf = _pair(kind)
    x = torch.randint(1, 97, (2, 10))
    am = torch.ones(2, 10, dtype=torch.long)
    am[0, :3] = 0
    keep = am.bool()
    with torch.no_grad():
        a = ours(input_ids=x, attention_mask=am, output_attentions=True, output_hidden_states=True)
        b = hf(input_ids=x, attention_mask=am, output_attentions=True, output_hidden_states=True)
    assert torch.allclose(a.logits[keep], b.logits[keep], atol=3e-4)
    assert len(a.hidden_states) == len(b.hidden_states)
    for p, q in zip(a.hidden_states, b.hidden_states):
        assert torch.allclose(p[keep], q[keep], atol=3e-4)
    assert len(a.attentions) == len(a.hidden_states) - 1
    for p in a.attentions:                                     # causal rows of probabilities
        assert torch.allclose(p[1].sum(-1), torch.ones_like(p[1].sum(-1)), atol=1e-4)
        assert float(p[1].triu(1).abs().max()) == 0.0
    for p, q in zip(a.attentions, b.attentions):               # empty when HF runs its fused attention path
        assert torch.allclose(p[1], q[1], atol=3e-4)           # the row without padding
    emb = hf.get_input_embeddings()(x)
    with torch.no_grad():
        assert torch.allclose(ours(inputs_embeds=emb).logits, hf(inputs_embeds=emb).logits, atol=3e-4)


def test_low_cpu_mem_usage_skips_redundant_initialisation(tmp_path):
    """`low_cpu_mem_usage=True`: same weights and logits, no random fill of tensors the checkpoint overwrites, and
    tensors the checkpoint lacks (a new classification head) still get their proper initialisation."""
    import torch.nn.init as init
    torch.manual_seed(0)
    cfg = ob.GPTJConfig(vocab_size=97, n_positions=32, n_embd=48, n_layer=2, n_head=4, rotary_dim=8)
    model = ob.GPTJForCausalLM(cfg).eval()
    model.save_pretrained(str(tmp_path))
    x = torch.randint(0, 97, (2, 9))
    calls = []
    real = init.kaiming_uniform_
    init.kaiming_uniform_ = lambda t, *a, **k: (calls.append(1), real(t, *a, **k))[1]
    try:
        slow = ob.GPTJForCausalLM.from_pretrained(str(tmp_path))
        n_slow = len(calls)
        fast = ob.GPTJForCausalLM.from_pretrained(str(tmp_path), low_cpu_mem_usage=True)
        assert n_slow > 0 and len(calls) == n_slow          # no constructor fill on the fast path
    finally:
        init.kaiming_uniform_ = real
    assert init.normal_.__name__ == "normal_"               # the patches are gone afterwards
    with torch.no_grad():
        want = model(input_ids=x).logits
        assert torch.equal(fast(input_ids=x).logits, want) and torch.equal(slow(input_ids=x).logits, want)
    cls_cfg = ob.GPTJConfig(vocab_size=97, n_positions=32, n_embd=48, n_layer=2, n_head=4, rotary_dim=8, num_labels=3,
                            pad_token_id=0)
    cls_cfg.save_pretrained(str(tmp_path))
    head = ob.GPTJForSequenceClassification.from_pretrained(str(tmp_path), low_cpu_mem_usage=True)
    w = head.score.weight.detach()
    assert torch.isfinite(w).all() and 0.005 < float(w.std()) < 0.05    # initializer_range 0.02, not raw memory
    fresh = ob.GPTJForCausalLM(cfg)
    assert float(fresh.lm_head.weight.std()) > 0.005                     # ordinary construction still initialises


@pytest.mark.parametrize("kind,beams", [("gpt2", 1), ("gptj", 1), ("gpt_neo", 2)])
def test_generate_returns_attentions_and_hidden_states_like_hf(kind, beams):
    """``generate(..., output_attentions=True, output_hidden_states=True, return_dict_in_generate=True)``: one entry
    per generated token, each a tuple over the layers, as in HF (the first entry covers the prompt). The arguments of
    encoder-decoder models are accepted and change nothing."""
    ours, hf = _pair(kind)
    x = torch.randint(1, 97, (2, 6))
    kw = dict(max_new_tokens=4, num_beams=beams, eos_token_id=None, pad_token_id=0, output_attentions=True,
              output_hidden_states=True, output_scores=True, return_dict_in_generate=True)
    a = ours.generate(x, use_static_cache=False, encoder_no_repeat_ngram_size=3, decoder_start_token_id=1, **kw)
    b = hf.generate(x, do_sample=False, **kw)
    assert torch.equal(a.sequences, b.sequences)
    assert len(a.hidden_states) == len(b.hidden_states) == 4 and len(a.attentions) == 4
    for step, (p, q) in enumerate(zip(a.hidden_states, b.hidden_states)):
        assert len(p) == len(q) == 3                           # embeddings + 2 layers
        for u, v in zip(p, q):
            assert u.shape == v.shape and u.shape[1] == (6 if step == 0 else 1)
            assert torch.allclose(u, v, atol=3e-4)
    for step, (p, q) in enumerate(zip(a.attentions, b.attentions)):
        assert len(p) == 2
        for u in p:
            assert u.shape[0] == 2 * beams and u.shape[-2] == (6 if step == 0 else 1) and u.shape[-1] == 6 + step
            assert torch.allclose(u.sum(-1), torch.ones_like(u.sum(-1)), atol=1e-4)
        for u, v in zip(p, q):                                 # empty when HF runs its fused attention path
            if v is not None:
                assert torch.allclose(u, v, atol=3e-4)
    # the default static cache gives the same tokens and states; without return_dict_in_generate nothing is collected
    c = ours.generate(x, **kw)
    assert torch.equal(c.sequences, a.sequences) and len(c.attentions) == 4
    for p, q in zip(c.hidden_states, a.hidden_states):
        for u, v in zip(p, q):
            assert torch.allclose(u, v, atol=1e-5)
    plain = ours.generate(x, max_new_tokens=4, eos_token_id=None, pad_token_id=0, output_attentions=True)
    assert torch.is_tensor(plain) and plain.shape == (2, 10)
