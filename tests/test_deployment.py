"""Deployment launcher on CPU workers (gloo): proxied generate / forward and dead-worker detection."""
import os

import pytest
import torch

import oslo_b200 as ob
from oslo_b200.parallel.engine_deployment import DeploymentError


def _model():
    torch.manual_seed(5)
    cfg = ob.GPT2Config(vocab_size=61, n_positions=32, n_embd=32, n_layer=2, n_head=4, resid_pdrop=0.0,
                        embd_pdrop=0.0, attn_pdrop=0.0)
    return ob.GPT2LMHeadModel(cfg).eval()


@pytest.fixture()
def gloo_env(monkeypatch):
    monkeypatch.setenv("OSLO_B200_BACKEND", "gloo")


@pytest.mark.parametrize("tp,pp", [(2, 1), (2, 2)])
def test_deployment_generate_and_forward(gloo_env, tp, pp):
    ref = _model()
    ids = torch.randint(0, 61, (2, 5), generator=torch.Generator().manual_seed(1))
    want = ref.generate(ids, max_length=12, num_beams=3, eos_token_id=None, pad_token_id=0)
    with torch.no_grad():
        want_logits = ref(input_ids=ids).logits
    model = ob.parallelize(_model(), tensor_parallel_size=tp, pipeline_parallel_size=pp, deployment=True,
                           startup_timeout_s=120, request_timeout_s=120)
    try:
        got = model.generate(ids, max_length=12, num_beams=3, eos_token_id=None, pad_token_id=0)
        assert torch.equal(got, want)
        out = model(input_ids=ids)
        assert torch.allclose(out.logits, want_logits, atol=1e-4)
    finally:
        model.cpu()  # shuts the workers down
    assert not model._deployment_engine.procs


def test_dead_worker_is_detected(gloo_env):
    model = ob.parallelize(_model(), tensor_parallel_size=2, deployment=True, startup_timeout_s=120,
                           request_timeout_s=30)
    eng = model._deployment_engine
    eng.procs[1].kill()
    eng.procs[1].join(5)
    with pytest.raises(DeploymentError):
        model.generate(torch.zeros(1, 3, dtype=torch.long), max_length=6, eos_token_id=None, pad_token_id=0)
    assert not eng.procs


def test_deployment_from_config_builds_the_model_inside_the_workers(gloo_env):
    """``from_config_with_parallel(..., deployment=True, init_on_device=True)``: the parent keeps a weightless handle,
    every worker draws the same random weights from the shared seed; the result equals a single-process model built
    from the same seed."""
    cfg = ob.GPT2Config(vocab_size=61, n_positions=32, n_embd=32, n_layer=2, n_head=4, resid_pdrop=0.0,
                        embd_pdrop=0.0, attn_pdrop=0.0)
    ids = torch.randint(0, 61, (2, 5), generator=torch.Generator().manual_seed(1))
    from oslo_b200.parallelism_utils import set_seed
    set_seed(77)
    want = ob.GPT2LMHeadModel(cfg).eval().generate(ids, max_length=12, eos_token_id=None, pad_token_id=0)
    model = ob.GPT2LMHeadModel.from_config_with_parallel(cfg, tensor_parallel_size=2, seed=77, deployment=True,
                                                         init_on_device=True)
    try:
        assert all(p.device.type == "meta" for p in model.parameters())
        assert model.fuse() is model                    # proxied: every worker fuses its copy
        got = model.generate(ids, max_length=12, eos_token_id=None, pad_token_id=0)
        assert torch.equal(got, want)
    finally:
        model.cpu()
    assert not model._deployment_engine.procs
