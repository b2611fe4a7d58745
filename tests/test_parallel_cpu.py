"""Tensor / pipeline / 3D parallel equivalence against a single-process fp32 oracle, on gloo CPU ranks."""
import os
import tempfile

import pytest
import torch

import oslo_b200 as ob
from tests.dist_utils import run_distributed


def tiny_config(kind):
    if kind == "gpt2":
        return ob.GPT2Config(vocab_size=101, n_positions=32, n_embd=32, n_layer=4, n_head=4,
                             resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    if kind == "gpt_neo":
        return ob.GPTNeoConfig(vocab_size=101, max_position_embeddings=32, hidden_size=32, num_layers=4, num_heads=4,
                               window_size=4)
    return ob.GPTJConfig(vocab_size=104, n_positions=32, n_embd=32, n_layer=4, n_head=4, rotary_dim=4)


MODEL = {"gpt2": "GPT2LMHeadModel", "gpt_neo": "GPTNeoForCausalLM", "gptj": "GPTJForCausalLM"}


def build(kind, seed=7):
    torch.manual_seed(seed)
    return getattr(ob, MODEL[kind])(tiny_config(kind))


def batch(seed=3, bsz=4, seq=16, vocab=101):
    g = torch.Generator().manual_seed(seed)
    x = torch.randint(0, vocab, (bsz, seq), generator=g)
    return dict(input_ids=x, labels=x.clone())


def oracle_steps(kind, steps, micro=None, lr=1e-2, loss_scale=1.0):
    """Single-process training: returns losses per step and the final state dict. ``loss_scale`` multiplies every
    micro-batch loss before ``backward`` (1 / replicas reproduces gradient averaging over data-parallel replicas)."""
    model = build(kind).train()
    opt = torch.optim.AdamW(model.parameters(), lr=lr)
    losses = []
    for s in range(steps):
        b = batch(seed=3 + s)
        opt.zero_grad()
        if micro is None:
            out = model(**b)
            out.loss.backward()
            losses.append(float(out.loss))
        else:
            tot = 0.0
            for i in range(0, b["input_ids"].size(0), micro):
                out = model(input_ids=b["input_ids"][i:i + micro], labels=b["labels"][i:i + micro])
                (out.loss * loss_scale).backward()
                tot += float(out.loss)
            losses.append(tot)
        opt.step()
    return losses, {k: v.detach().clone() for k, v in model.state_dict().items()}


def _train_parallel(rank, world, kind, tp, pp, steps, micro, expected_losses, tmpdir, fuse, out_logits, seq_par=False):
    from oslo_b200.optim import sync_sequence_parallel_grads
    model = build(kind).train()
    model = ob.parallelize(model, tensor_parallel_size=tp, pipeline_parallel_size=pp,
                           micro_batch_size=micro or 1, sequence_parallel=seq_par)
    if fuse:
        model.fuse()
    mpu = model.mpu
    params = [p for p in model.gpu_parameters() if p.requires_grad]
    opt = torch.optim.AdamW(params, lr=1e-2)
    dp, dpr = mpu.get_data_parallel_world_size(), mpu.get_data_parallel_rank()
    for s in range(steps):
        b = batch(seed=3 + s)
        if dp > 1:  # each data-parallel replica takes a slice; grads are averaged by hand below
            n = b["input_ids"].size(0) // dp
            b = {k: v[dpr * n:(dpr + 1) * n] for k, v in b.items()}
        opt.zero_grad()
        if pp > 1:
            tot = 0.0
            for out in model(**b, output_logits=out_logits):
                out.loss.backward()
                tot += float(out.loss)
            loss = tot
        else:
            out = model(**b, output_logits=out_logits)
            out.loss.backward()
            loss = float(out.loss)
        sync_sequence_parallel_grads(model)
        if dp > 1:
            import torch.distributed as dist
            for p in params:
                if p.grad is not None:
                    dist.all_reduce(p.grad, group=mpu.get_data_parallel_group())
                    p.grad /= dp
        else:
            assert abs(loss - expected_losses[s]) < 2e-4, (s, loss, expected_losses[s])
        opt.step()
    model.save_pretrained_with_parallel(os.path.join(tmpdir, "merged"), save_with_merging=True)
    model.save_pretrained_with_parallel(os.path.join(tmpdir, "split"))


def _check_merged(tmpdir, ref_state, atol):
    merged = torch.load(os.path.join(tmpdir, "merged", "pytorch_model.bin"), weights_only=True)
    for k, v in ref_state.items():
        if k not in merged:
            assert k == "lm_head.weight", k
            continue
        assert merged[k].shape == v.shape, (k, merged[k].shape, v.shape)
        assert torch.allclose(merged[k], v, atol=atol), (k, (merged[k] - v).abs().max())


@pytest.mark.parametrize("kind", ["gpt2", "gpt_neo", "gptj"])
@pytest.mark.parametrize("fuse,out_logits", [(False, True), (True, False)])
def test_tensor_parallel_training_matches_oracle(kind, fuse, out_logits):
    losses, state = oracle_steps(kind, steps=3)
    with tempfile.TemporaryDirectory() as d:
        run_distributed(_train_parallel, 2, kind, 2, 1, 3, None, losses, d, fuse, out_logits)
        _check_merged(d, state, 1e-3)
        names = sorted(f for f in os.listdir(os.path.join(d, "split")) if f.endswith(".bin"))
        assert names == ["pytorch_model_tp=0_pp=0.bin", "pytorch_model_tp=1_pp=0.bin"]


def test_tensor_parallel_shared_input_gradient_matches_oracle(monkeypatch):
    """GPT-J block with q / k / v / fc_in as one autograd node and a single all-reduce of the block's input gradient
    (``OSLO_B200_TP_SHARED_INPUT_GRAD=1``): same losses and merged weights as the single-process oracle."""
    monkeypatch.setenv("OSLO_B200_TP_SHARED_INPUT_GRAD", "1")
    losses, state = oracle_steps("gptj", steps=3)
    with tempfile.TemporaryDirectory() as d:
        run_distributed(_train_parallel, 2, "gptj", 2, 1, 3, None, losses, d, False, True)
        _check_merged(d, state, 1e-3)


@pytest.mark.parametrize("kind", ["gpt2", "gpt_neo", "gptj"])
def test_sequence_parallel_training_matches_oracle(kind):
    """Megatron-style sequence parallelism inside the TP group (absent in the reference): same losses, same weights."""
    losses, state = oracle_steps(kind, steps=3)
    with tempfile.TemporaryDirectory() as d:
        run_distributed(_train_parallel, 2, kind, 2, 1, 3, None, losses, d, False, True, True)
        _check_merged(d, state, 1e-3)


def test_sequence_parallel_with_pipeline():
    losses, state = oracle_steps("gptj", steps=2, micro=2)
    with tempfile.TemporaryDirectory() as d:
        run_distributed(_train_parallel, 4, "gptj", 2, 2, 2, 2, losses, d, False, True, True)
        _check_merged(d, state, 1e-3)


@pytest.mark.parametrize("kind", ["gpt2", "gptj"])
def test_pipeline_parallel_training_matches_oracle(kind):
    losses, state = oracle_steps(kind, steps=2, micro=1)
    with tempfile.TemporaryDirectory() as d:
        run_distributed(_train_parallel, 2, kind, 1, 2, 2, 1, losses, d, False, True)
        _check_merged(d, state, 1e-3)


def test_3d_parallel_training_gpt_neo():
    # tp=2 x pp=2 x dp=2 on 8 ranks would be the full layout; 4 ranks give tp=2 x pp=2 (dp=1)
    losses, state = oracle_steps("gpt_neo", steps=2, micro=2)
    with tempfile.TemporaryDirectory() as d:
        run_distributed(_train_parallel, 4, "gpt_neo", 2, 2, 2, 2, losses, d, False, True)
        _check_merged(d, state, 1e-3)


@pytest.mark.parametrize("kind,tp,pp,fuse", [("gpt_neo", 1, 2, True), ("gpt2", 2, 2, True), ("gptj", 2, 2, True),
                                             ("gpt2", 2, 2, False), ("gptj", 2, 2, False), ("gpt_neo", 2, 2, True),
                                             ("gptj", 4, 1, True), ("gpt2", 4, 1, False), ("gpt_neo", 4, 2, True)])
def test_training_matrix_over_families_and_layouts(kind, tp, pp, fuse):
    """The remaining cells of the reference's {tp, pp, 3d} x {training, training_with_fusion} matrix for the three
    families: losses of every step and the merged weights equal the single-process oracle."""
    micro = 2 if pp > 1 else None
    losses, state = oracle_steps(kind, steps=2, micro=micro)
    with tempfile.TemporaryDirectory() as d:
        run_distributed(_train_parallel, tp * pp, kind, tp, pp, 2, micro, losses, d, fuse, not fuse)
        _check_merged(d, state, 1e-3)


def _roundtrip(rank, world, kind, tmpdir):
    cls = getattr(ob, MODEL[kind])
    model = cls.from_pretrained_with_parallel(os.path.join(tmpdir, "split"), tensor_parallel_size=2)
    b = batch(seed=11)
    with torch.no_grad():
        out = model(**b)
    ref = torch.load(os.path.join(tmpdir, "ref.pt"), weights_only=True)
    assert torch.allclose(out.logits, ref["logits"], atol=2e-4), (out.logits - ref["logits"]).abs().max()
    gen = model.generate(b["input_ids"][:, :4], max_length=10, eos_token_id=None, pad_token_id=0)
    assert torch.equal(gen, ref["gen"])


def _save_split(rank, world, kind, tmpdir):
    cls = getattr(ob, MODEL[kind])
    model = cls.from_pretrained_with_parallel(os.path.join(tmpdir, "hf"), tensor_parallel_size=2)
    model.save_pretrained_with_parallel(os.path.join(tmpdir, "split"))


@pytest.mark.parametrize("kind", ["gpt2", "gptj"])
def test_split_checkpoint_roundtrip(kind):
    with tempfile.TemporaryDirectory() as d:
        model = build(kind).eval()
        model.save_pretrained(os.path.join(d, "hf"))
        b = batch(seed=11)
        with torch.no_grad():
            logits = model(**b).logits
        gen = model.generate(b["input_ids"][:, :4], max_length=10, eos_token_id=None, pad_token_id=0)
        torch.save({"logits": logits, "gen": gen}, os.path.join(d, "ref.pt"))
        run_distributed(_save_split, 2, kind, d)
        run_distributed(_roundtrip, 2, kind, d)
        with pytest.raises(AssertionError):  # wrong layout must be refused, not silently mis-loaded
            run_distributed(_bad_layout, 4, kind, d)


def _inference_matrix(rank, world, kind, tp, pp, fuse, tmpdir):
    """The reference's ``*_inference`` / ``*_inference_with_fusion`` / ``*_deparallelization`` scripts in one flow:
    merged checkpoint -> parallel model -> logits and beam search equal one process's -> split files -> reloaded in
    the same layout -> merged again -> one process reproduces the logits."""
    cls = getattr(ob, MODEL[kind])
    ref = torch.load(os.path.join(tmpdir, "ref.pt"), weights_only=True)
    b = batch(seed=11, vocab=104 if kind == "gptj" else 101)

    def check(model):
        model.eval()
        with torch.no_grad():
            out = model(input_ids=b["input_ids"])
            logits = torch.cat([o.logits for o in out]) if pp > 1 else out.logits     # one output per micro-batch
        assert torch.allclose(logits, ref["logits"], atol=3e-4), float((logits - ref["logits"]).abs().max())
        gen = model.generate(b["input_ids"][:, :4], max_length=9, num_beams=2, eos_token_id=None, pad_token_id=0)
        assert torch.equal(gen, ref["gen"])

    model = cls.from_pretrained_with_parallel(os.path.join(tmpdir, "hf"), tensor_parallel_size=tp,
                                              pipeline_parallel_size=pp, micro_batch_size=2)
    if fuse:
        model.fuse()
    check(model)
    model.save_pretrained_with_parallel(os.path.join(tmpdir, "split"))
    again = cls.from_pretrained_with_parallel(os.path.join(tmpdir, "split"), tensor_parallel_size=tp,
                                              pipeline_parallel_size=pp, micro_batch_size=2)
    check(again)
    again.save_pretrained_with_parallel(os.path.join(tmpdir, "merged"), save_with_merging=True)


@pytest.mark.parametrize("kind", ["gpt2", "gpt_neo", "gptj"])
@pytest.mark.parametrize("tp,pp,fuse", [(2, 1, False), (1, 2, True), (2, 2, False), (2, 2, True)])
def test_inference_and_deparallelization_matrix(kind, tp, pp, fuse):
    with tempfile.TemporaryDirectory() as d:
        model = build(kind).eval()
        model.save_pretrained(os.path.join(d, "hf"))
        b = batch(seed=11, vocab=104 if kind == "gptj" else 101)
        with torch.no_grad():
            logits = model(input_ids=b["input_ids"]).logits
        gen = model.generate(b["input_ids"][:, :4], max_length=9, num_beams=2, eos_token_id=None, pad_token_id=0)
        torch.save({"logits": logits, "gen": gen}, os.path.join(d, "ref.pt"))
        run_distributed(_inference_matrix, tp * pp, kind, tp, pp, fuse, d)
        single = getattr(ob, MODEL[kind]).from_pretrained(os.path.join(d, "merged")).eval()
        with torch.no_grad():
            assert torch.allclose(single(input_ids=b["input_ids"]).logits, logits, atol=3e-4)


def _bad_layout(rank, world, kind, tmpdir):
    cls = getattr(ob, MODEL[kind])
    try:
        cls.from_pretrained_with_parallel(os.path.join(tmpdir, "split"), tensor_parallel_size=4)
    except FileNotFoundError:
        raise


def _train_zero_ddp(rank, world, kind, steps, tmpdir, accumulate):
    """Data parallel over all ranks with the framework's own pieces: ZeRO-1 FusedAdamW on the flat buffers and the
    bucketed DistributedDataParallel wrapper (tiny buckets so that several reductions are in flight)."""
    import contextlib
    import torch.distributed as dist
    from oslo_b200.optim import FusedAdamW
    from oslo_b200.parallel.data_parallel import DistributedDataParallel
    model = build(kind).train()
    model = ob.parallelize(model, tensor_parallel_size=1)
    mpu = model.mpu
    opt = FusedAdamW(model.gpu_parameters(), lr=1e-2, weight_decay=0.01, shard_group=mpu.get_data_parallel_group())
    ddp = DistributedDataParallel(model, mpu, optimizer=opt, bucket_mb=0.01)
    for s in range(steps):
        b = batch(seed=3 + s, bsz=4 * world)
        n = b["input_ids"].size(0) // world
        mine = {k: v[rank * n:(rank + 1) * n] for k, v in b.items()}
        opt.zero_grad()
        if accumulate:   # two micro-batches, gradients reduced only after the second one
            half = n // 2
            for i in range(2):
                mb = {k: v[i * half:(i + 1) * half] for k, v in mine.items()}
                hold = ddp.no_sync() if i == 0 else contextlib.nullcontext()
                with hold:
                    (ddp(**mb).loss / 2).backward()
        else:
            ddp(**mine).loss.backward()
        opt.step()
    state = {k: v.detach().clone() for k, v in model.state_dict().items()}
    gathered = [None] * world
    dist.all_gather_object(gathered, {k: float(v.double().sum()) for k, v in state.items()})
    assert all(g == gathered[0] for g in gathered), "replicas diverged"
    if rank == 0:
        torch.save(state, os.path.join(tmpdir, "state.pt"))


@pytest.mark.parametrize("kind,accumulate", [("gptj", False), ("gptj", True), ("gpt2", True), ("gpt_neo", False)])
def test_zero1_and_bucketed_ddp_match_single_process(kind, accumulate):
    """2 data-parallel gloo ranks with ZeRO-1 + the bucketed DDP wrapper == one process on the whole batch."""
    steps, world = 3, 2
    torch.manual_seed(0)
    ref = build(kind).train()
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.01)
    for s in range(steps):
        b = batch(seed=3 + s, bsz=4 * world)
        opt.zero_grad()
        ref(**b).loss.backward()
        opt.step()
    with tempfile.TemporaryDirectory() as d:
        run_distributed(_train_zero_ddp, world, kind, steps, d, accumulate)
        got = torch.load(os.path.join(d, "state.pt"), weights_only=True)
    for k, v in ref.state_dict().items():
        assert torch.allclose(got[k], v, atol=2e-4), (k, (got[k] - v).abs().max())


def _train_wide_grads(rank, world, tmpdir):
    """bf16 parameters, fp32 gradient buffer, ZeRO-1 + bucketed wrapper on ``world`` ranks (one rank = the oracle)."""
    import contextlib
    import torch.distributed as dist
    from oslo_b200.optim import FusedAdamW
    from oslo_b200.parallel.data_parallel import DistributedDataParallel
    torch.manual_seed(7)
    model = ob.parallelize(ob.GPTJForCausalLM(tiny_config("gptj")).to(torch.bfloat16).train(), tensor_parallel_size=1)
    mpu = model.mpu
    opt = FusedAdamW(model.gpu_parameters(), lr=1e-2, grad_dtype=torch.float32, max_grad_norm=1.0,
                     shard_group=mpu.get_data_parallel_group() if world > 1 else None)
    call = DistributedDataParallel(model, mpu, optimizer=opt, bucket_mb=0.01) if world > 1 else model
    assert opt.buf.flat_g.dtype == torch.float32 and opt.buf.symm_g is None
    b = batch(seed=3, bsz=8, vocab=104)
    n = 8 // world
    mine = {k: v[rank * n:(rank + 1) * n] for k, v in b.items()}
    opt.zero_grad()
    for i in range(2):          # two micro-batches per step
        mb = {k: v[i * (n // 2):(i + 1) * (n // 2)] for k, v in mine.items()}
        hold = call.no_sync() if (world > 1 and i == 0) else contextlib.nullcontext()
        with hold:
            (call(**mb).loss / 2).backward()
    if world > 1:
        call.finish_gradient_sync()                     # buckets summed over the ranks, in fp32
    grad = opt.buf.flat_g[: opt.buf.numel].clone() / world
    if rank == 0:
        torch.save(grad, os.path.join(tmpdir, f"grad{world}.pt"))
    opt.step()
    flat = opt.buf.flat_p.float().clone()
    if world > 1:
        other = [torch.empty_like(flat) for _ in range(world)]
        dist.all_gather(other, flat)
        assert all(torch.equal(o, other[0]) for o in other), "replicas diverged"
        others_grad = [torch.empty_like(grad) for _ in range(world)]
        dist.all_gather(others_grad, grad)
        assert all(torch.equal(o, others_grad[0]) for o in others_grad), "summed gradients differ between the ranks"


def test_fp32_gradient_buffer_with_zero1_and_bucketed_ddp():
    """``grad_dtype=torch.float32`` under data parallelism: fp32 buckets through the all-reduce path, the owned shard
    stepped, bf16 parameters gathered. The averaged gradient of two ranks equals one process's on the whole batch up
    to the bf16 rounding of the individual micro-batch gradients (the micro-batches are cut differently)."""
    with tempfile.TemporaryDirectory() as d:
        run_distributed(_train_wide_grads, 1, d)
        run_distributed(_train_wide_grads, 2, d)
        one = torch.load(os.path.join(d, "grad1.pt"), weights_only=True)
        two = torch.load(os.path.join(d, "grad2.pt"), weights_only=True)
    assert one.dtype == two.dtype == torch.float32
    assert (one - two).norm() / one.norm() < 2e-2, float((one - two).norm() / one.norm())


def test_3d_parallel_with_data_parallel_replicas():
    """TP=2 x PP=2 x DP=2 on 8 gloo ranks (the GPT-Neo configuration of the benchmark list, in miniature): merged
    weights equal the single-process oracle whose two micro-batch gradients are averaged like the two replicas'."""
    losses, state = oracle_steps("gpt_neo", steps=2, micro=2, loss_scale=0.5)
    with tempfile.TemporaryDirectory() as d:
        run_distributed(_train_parallel, 8, "gpt_neo", 2, 2, 2, 2, losses, d, False, True)
        _check_merged(d, state, 1e-3)


def _zero_resume(rank, world, kind, tmpdir):
    """3 uninterrupted ZeRO-1 steps == 2 steps + (split checkpoint, per-rank sidecar) + fresh objects + 1 step."""
    from oslo_b200.optim import DynamicLossScaler, FusedAdamW
    cls = getattr(ob, MODEL[kind])

    def optimizer(model):
        return FusedAdamW(model.gpu_parameters(), lr=1e-2, shard_group=model.mpu.get_data_parallel_group(),
                          loss_scaler=DynamicLossScaler(init_scale=4.0))

    def step(model, opt, s):
        b = batch(seed=11 + s, bsz=2 * world)
        mine = {k: v[rank * 2:(rank + 1) * 2] for k, v in b.items()}
        opt.zero_grad()
        opt.loss_scaler.scale(model(**mine).loss).backward()
        assert opt.step()

    model = ob.parallelize(build(kind).train(), tensor_parallel_size=1)
    opt = optimizer(model)
    for s in range(2):
        step(model, opt, s)
    ckpt = os.path.join(tmpdir, "ckpt")
    model.save_pretrained_with_parallel(ckpt)
    path = model.save_training_state(ckpt, opt, step=2)
    assert path.endswith(f"oslo_state_tp=0_pp=0_dp={rank}.pt")
    step(model, opt, 2)
    want = {k: v.detach().clone() for k, v in model.state_dict().items()}

    again = cls.from_pretrained_with_parallel(ckpt, tensor_parallel_size=1).train()
    opt2 = optimizer(again)
    info = again.load_training_state(ckpt, opt2)
    assert info["step"] == 2 and opt2.step_count == 2
    assert torch.equal(opt2.master, opt.master) is False      # opt has moved on; the shard on disk is step 2's
    step(again, opt2, 2)
    for k, v in again.state_dict().items():
        assert torch.equal(v, want[k]), k
    assert torch.equal(opt2.master, opt.master) and torch.equal(opt2.exp_avg_sq, opt.exp_avg_sq)


def test_zero1_resume_from_per_rank_sidecars():
    with tempfile.TemporaryDirectory() as d:
        run_distributed(_zero_resume, 2, "gpt2", d)


def _elastic_dp(rank, world, tmpdir, phase):
    """Phase "save": ``world`` data-parallel ranks with ZeRO-1 train 2 steps, save, train a third step and leave its
    result behind. Phase "resume": another number of ranks loads that checkpoint (the optimizer shards are re-cut),
    trains the third step on the same global batch and compares."""
    import torch.distributed as dist
    from oslo_b200.optim import FusedAdamW
    cls = ob.GPTJForCausalLM
    ckpt = os.path.join(tmpdir, "ckpt")

    def step(model, opt, s):
        b = batch(seed=21 + s, bsz=8, vocab=104)
        n = 8 // world
        mine = {k: v[rank * n:(rank + 1) * n] for k, v in b.items()}
        opt.zero_grad()
        model(**mine).loss.backward()
        opt.step()

    def optimizer(model):
        return FusedAdamW(model.gpu_parameters(), lr=1e-2, shard_group=model.mpu.get_data_parallel_group() if world > 1 else None)

    if phase == "save":
        model = ob.parallelize(build("gptj").train(), tensor_parallel_size=1)
        opt = optimizer(model)
        for s in range(2):
            step(model, opt, s)
        model.save_pretrained_with_parallel(ckpt)
        model.save_training_state(ckpt, opt, step=2)
        full = [torch.empty_like(opt.master) for _ in range(world)]
        dist.all_gather(full, opt.master)
        step(model, opt, 2)
        if rank == 0:
            torch.save({"master": torch.cat(full)[: opt.buf.numel], "after": opt.buf.flat_p[: opt.buf.numel].clone()},
                       os.path.join(tmpdir, "want.pt"))
        return
    want = torch.load(os.path.join(tmpdir, "want.pt"), weights_only=True)
    model = cls.from_pretrained_with_parallel(ckpt, tensor_parallel_size=1).train()
    opt = optimizer(model)
    info = model.load_training_state(ckpt, opt)
    assert info["step"] == 2 and info["resharded_from"] == 2 and opt.step_count == 2
    lo, hi = opt._lo, min(opt._hi, opt.buf.numel)
    assert torch.equal(opt.master[: hi - lo], want["master"][lo:hi])           # the re-cut shard is the saved state
    assert float(opt.exp_avg_sq.abs().sum()) > 0
    step(model, opt, 2)
    got = opt.buf.flat_p[: opt.buf.numel]
    assert torch.allclose(got, want["after"], atol=1e-5), float((got - want["after"]).abs().max())


@pytest.mark.parametrize("new_world", [1, 4])
def test_zero1_state_is_recut_when_the_number_of_replicas_changes(new_world):
    """A job saved with 2 data-parallel replicas continues with 1 or with 4: every new rank builds its optimizer shard
    from the old ranks' sidecars, and the next step lands where the original job's next step landed."""
    with tempfile.TemporaryDirectory() as d:
        run_distributed(_elastic_dp, 2, d, "save")
        run_distributed(_elastic_dp, new_world, d, "resume")


def _every_unit_announces_itself(rank, world, kind, tp, pp):
    """Forward pre-hooks on every forward unit of the (stage's) model: a training forward must fire all of them, also
    for modules whose parameters are read without calling the module (the LM head inside the fused loss)."""
    from oslo_b200.parallel.data_parallel import forward_units
    model = build(kind).train()
    if world > 1:
        model = ob.parallelize(model, tensor_parallel_size=tp, pipeline_parallel_size=pp, micro_batch_size=2)
    gm = model.gpu_modules() if world > 1 else model
    units = forward_units(gm)
    covered = {id(p) for m in units for p in m.parameters()}
    assert all(id(p) in covered for p in gm.parameters())
    for out_logits in (False, True):
        fired = set()
        handles = [m.register_forward_pre_hook(lambda mod, args: fired.add(id(mod))) for m in units]
        b = batch(vocab=104 if kind == "gptj" else 101)
        out = model(**b, output_logits=out_logits)
        if pp > 1:
            for o in out:
                o.loss.backward()
        else:
            out.loss.backward()
        missing = [type(m).__name__ for m in units if id(m) not in fired]
        for h in handles:
            h.remove()
        assert not missing, (kind, tp, pp, out_logits, missing)


@pytest.mark.parametrize("kind,tp,pp", [("gpt2", 1, 1), ("gpt_neo", 1, 1), ("gptj", 1, 1), ("gptj", 2, 1), ("gptj", 1, 2),
                                        ("gpt2", 1, 2)])
def test_every_forward_unit_runs_its_pre_hooks(kind, tp, pp):
    """What the overlapped ZeRO-1 parameter all-gather relies on: it makes the compute stream wait for a unit's
    parameter buckets in that unit's forward pre-hook."""
    if tp * pp == 1:
        _every_unit_announces_itself(0, 1, kind, 1, 1)
    else:
        run_distributed(_every_unit_announces_itself, tp * pp, kind, tp, pp)


# ---------------------------------------------------------------------------- classification / multiple-choice heads
def _head_config(name):
    if name == "GPT2ForSequenceClassification":
        return ob.GPT2Config(vocab_size=101, n_positions=32, n_embd=32, n_layer=4, n_head=4, resid_pdrop=0.0,
                             embd_pdrop=0.0, attn_pdrop=0.0, num_labels=3, pad_token_id=0)
    if name == "GPT2DoubleHeadsModel":
        return ob.GPT2Config(vocab_size=101, n_positions=32, n_embd=32, n_layer=4, n_head=4, resid_pdrop=0.0,
                             embd_pdrop=0.0, attn_pdrop=0.0, summary_first_dropout=0.0, num_labels=1)
    if name == "GPTNeoForSequenceClassification":
        return ob.GPTNeoConfig(vocab_size=101, max_position_embeddings=32, hidden_size=32, num_layers=4, num_heads=4,
                               window_size=4, num_labels=3, pad_token_id=0)
    return ob.GPTJConfig(vocab_size=104, n_positions=32, n_embd=32, n_layer=4, n_head=4, rotary_dim=4, num_labels=3,
                         pad_token_id=0)


def _head_inputs(name):
    g = torch.Generator().manual_seed(1)
    if name == "GPT2DoubleHeadsModel":      # [batch, choices, seq] ids, one summary position per choice
        ids = torch.randint(1, 101, (4, 2, 16), generator=g)
        return dict(input_ids=ids, mc_token_ids=torch.randint(0, 16, (4, 2), generator=g), labels=ids.clone(),
                    mc_labels=torch.randint(0, 2, (4,), generator=g))
    ids = torch.randint(1, 101, (4, 16), generator=g)
    return dict(input_ids=ids, labels=torch.randint(0, 3, (4,), generator=g))


def _head_model(name):
    torch.manual_seed(5)
    return getattr(ob, name)(_head_config(name)).train()


def _head_ranks(rank, world, name, tp, pp, want):
    model = ob.parallelize(_head_model(name), tensor_parallel_size=tp, pipeline_parallel_size=pp, micro_batch_size=2)
    b = _head_inputs(name)
    if pp > 1:
        got = 0.0
        for out in model(**b):
            out.loss.backward()
            got += float(out.loss.detach()) / 2
    else:
        out = model(**b)
        out.loss.backward()
        got = float(out.loss.detach())
    assert abs(got - want) < 1e-4, (name, tp, pp, got, want)
    if name != "GPT2DoubleHeadsModel":     # (its `loss` is the LM loss alone, as in HF: the choice head gets no gradient)
        missing = [n for n, p in model.gpu_modules().named_parameters() if p.requires_grad and p.grad is None]
        assert not missing, (rank, missing)


@pytest.mark.parametrize("name,tp,pp", [("GPT2ForSequenceClassification", 2, 2), ("GPT2DoubleHeadsModel", 1, 2),
                                        ("GPT2DoubleHeadsModel", 2, 2), ("GPTNeoForSequenceClassification", 2, 2),
                                        ("GPTJForSequenceClassification", 2, 2)])
def test_classification_and_double_heads_models_under_tp_and_pp(name, tp, pp):
    """The non-LM heads go through the same engines: loss of the parallel model == single process (mean over the two
    micro-batches under pipeline parallelism, where the last stage must see the multiple-choice inputs too)."""
    model, b = _head_model(name), _head_inputs(name)
    if pp > 1:
        want = sum(float(model(**{k: v[i:i + 2] for k, v in b.items()}).loss.detach()) for i in (0, 2)) / 2
    else:
        want = float(model(**b).loss.detach())
    run_distributed(_head_ranks, tp * pp, name, tp, pp, want)


# ---------------------------------------------------------------------------- generation through the engines
def _gen_inputs():
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(1, 100, (2, 6), generator=g)
    mask = torch.ones_like(ids)
    mask[0, :2] = 0                      # row 0 is left-padded
    return ids, mask


def _generate(model, case):
    ids, mask = _gen_inputs()
    ids, mask = ids.to(model.device), mask.to(model.device)
    if case == "greedy":
        return model.generate(ids, attention_mask=mask, max_new_tokens=6, do_sample=False, pad_token_id=0)
    if case == "beam":
        return model.generate(ids, attention_mask=mask, max_new_tokens=6, num_beams=3, no_repeat_ngram_size=2,
                              pad_token_id=0)
    torch.manual_seed(11)
    return model.generate(ids, attention_mask=mask, max_new_tokens=6, do_sample=True, top_k=5, pad_token_id=0)


def _generate_ranks(rank, world, kind, tp, pp, case, want):
    model = ob.parallelize(build(kind).eval(), tensor_parallel_size=tp, pipeline_parallel_size=pp, micro_batch_size=1)
    got = _generate(model, case)
    assert torch.equal(got.cpu(), want), (kind, tp, pp, case, got, want)


@pytest.mark.parametrize("kind,tp,pp,case", [("gpt2", 1, 2, "beam"), ("gptj", 2, 2, "greedy"),
                                             ("gpt_neo", 2, 2, "sample"), ("gptj", 2, 1, "beam")])
def test_generate_through_tensor_and_pipeline_engines(kind, tp, pp, case):
    """`generate()` with a KV cache on a TP / PP / TP x PP model returns, on every rank, the tokens of the
    single-process model (every pipeline stage keeps and advances the cache of its own layers)."""
    want = _generate(build(kind).eval(), case)
    run_distributed(_generate_ranks, tp * pp, kind, tp, pp, case, want)


# ---------------------------------------------------------------------------- further flows through the engines
def _flow_ranks(rank, world, kind, tp, pp, sp, case, want):
    model = build(kind)
    model = model.train() if case == "checkpointing" else model.eval()
    model = ob.parallelize(model, tensor_parallel_size=tp, pipeline_parallel_size=pp, micro_batch_size=2,
                           sequence_parallel=sp)
    ids, mask = _gen_inputs()
    if case == "checkpointing":
        model.gradient_checkpointing_enable()
        b = batch(seed=3)
        if pp > 1:
            got = 0.0
            for out in model(**b):
                out.loss.backward()
                got += float(out.loss.detach()) / 2
        else:
            out = model(**b)
            out.loss.backward()
            got = float(out.loss.detach())
        got = torch.tensor(got)
    elif case == "generate":
        got = model.generate(ids, attention_mask=mask, max_new_tokens=5, do_sample=False, pad_token_id=0)
    elif case == "inputs_embeds":
        emb = build(kind).get_input_embeddings()(ids).detach()
        with torch.no_grad():     # without gradients every stage receives the last stage's tensors
            got = torch.cat([o.logits for o in model(inputs_embeds=emb, output_hidden_states=True)])
    else:
        from oslo_b200.generation import GraphedGreedyDecoder
        got = GraphedGreedyDecoder(model, max_len=32, use_graph=False).generate(ids, max_new_tokens=5)
    assert torch.allclose(got.float().cpu(), want.float(), atol=2e-4), (case, got, want)


@pytest.mark.parametrize("kind,tp,pp,sp,case", [("gptj", 2, 2, False, "checkpointing"), ("gpt2", 2, 1, True, "checkpointing"),
                                                ("gptj", 2, 1, True, "generate"), ("gpt2", 1, 2, False, "inputs_embeds"),
                                                ("gptj", 2, 1, False, "graph_decoder")])
def test_more_flows_through_the_engines(kind, tp, pp, sp, case):
    """Activation checkpointing under TP x PP and under sequence parallelism, generation on a sequence-parallel
    model, `inputs_embeds` through pipeline stages, the static-cache greedy decoder on a tensor-parallel model."""
    model = build(kind)
    ids, mask = _gen_inputs()
    if case == "checkpointing":
        model.train()
        b = batch(seed=3)
        if pp > 1:
            want = torch.tensor(sum(float(model(**{k: v[i:i + 2] for k, v in b.items()}).loss.detach()) for i in (0, 2)) / 2)
        else:
            want = model(**b).loss.detach()
    elif case == "generate":
        want = model.eval().generate(ids, attention_mask=mask, max_new_tokens=5, do_sample=False, pad_token_id=0)
    elif case == "inputs_embeds":
        want = model.eval()(input_ids=ids).logits.detach()
    else:
        want = model.eval().generate(ids, max_new_tokens=5, do_sample=False, pad_token_id=0)
    run_distributed(_flow_ranks, tp * pp, kind, tp, pp, sp, case, want)


def _torch_ddp_ranks(rank, world, kind, tp, pp):
    """The reference's data-parallel recipe: torch DDP around `gpu_modules()` over `mpu.get_data_parallel_group()`."""
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as TorchDDP
    model = ob.parallelize(build(kind).train(), tensor_parallel_size=tp, pipeline_parallel_size=pp, micro_batch_size=2)
    mpu = model.mpu
    ddp = TorchDDP(model.gpu_modules(), process_group=mpu.get_data_parallel_group())
    opt = torch.optim.Adam(model.gpu_parameters(), lr=1e-2)
    dp, dpr = mpu.get_data_parallel_world_size(), mpu.get_data_parallel_rank()
    for s in range(2):
        b = batch(seed=3 + s)
        n = b["input_ids"].size(0) // dp
        b = {k: v[dpr * n:(dpr + 1) * n] for k, v in b.items()}
        opt.zero_grad()
        if pp > 1:
            for out in ddp(**b):        # one micro-batch per step: torch DDP reduces during the only backward
                out.loss.backward()
        else:
            ddp(**b).loss.backward()
        opt.step()
    sums = {k: float(v.double().sum()) for k, v in model.state_dict().items() if v.is_floating_point()}
    gathered = [None] * dp
    dist.all_gather_object(gathered, sums, group=mpu.get_data_parallel_group())
    assert all(g == gathered[0] for g in gathered), "replicas diverged"


@pytest.mark.parametrize("kind,tp,pp", [("gptj", 2, 1), ("gpt2", 1, 2)])
def test_torch_ddp_around_gpu_modules(kind, tp, pp):
    run_distributed(_torch_ddp_ranks, 4, kind, tp, pp)


def _misuse_ranks(rank, world):
    model = ob.parallelize(build("gptj"), tensor_parallel_size=2)
    with pytest.raises(RuntimeError, match="already parallelized"):
        ob.parallelize(model, tensor_parallel_size=2)
    with pytest.raises(ValueError, match="exceeds world size"):
        ob.parallelize(build("gptj"), tensor_parallel_size=2, pipeline_parallel_size=2)
    with pytest.raises(ValueError, match="power of two"):
        ob.parallelize(build("gptj"), tensor_parallel_size=3)
    pp_model = ob.parallelize(build("gpt2"), pipeline_parallel_size=2)
    with pytest.raises(ValueError, match="keyword arguments only"):
        pp_model(batch()["input_ids"])
    from oslo_b200.generation import GraphedGreedyDecoder
    with pytest.raises(NotImplementedError, match="pipeline"):
        GraphedGreedyDecoder(pp_model, max_len=16)
    ids = batch()["input_ids"][:, :4]          # the flag falls back to the ordinary greedy loop under PP
    assert torch.equal(pp_model.generate(ids, max_new_tokens=3, cuda_graph=True, pad_token_id=0),
                       pp_model.generate(ids, max_new_tokens=3, pad_token_id=0))


def test_misuse_raises_clear_errors():
    run_distributed(_misuse_ranks, 2)


def _pp_split_roundtrip(rank, world, kind, tmpdir, phase):
    cls = getattr(ob, MODEL[kind])
    if phase == "save":
        model = cls.from_pretrained_with_parallel(os.path.join(tmpdir, "hf"), pipeline_parallel_size=2)
        model.save_pretrained_with_parallel(os.path.join(tmpdir, "split"))
        return
    # a different seed: whatever the files do not restore stays visibly wrong
    model = cls.from_pretrained_with_parallel(os.path.join(tmpdir, "split"), pipeline_parallel_size=2, seed=999,
                                              low_cpu_mem_usage=(kind == "gpt2"))
    b = batch(seed=11)
    with torch.no_grad():
        logits = torch.cat([o.logits for o in model(input_ids=b["input_ids"])])
    ref = torch.load(os.path.join(tmpdir, "ref.pt"), weights_only=True)
    assert torch.allclose(logits, ref["logits"], atol=2e-4), (logits - ref["logits"]).abs().max()


@pytest.mark.parametrize("kind", ["gpt_neo", "gpt2"])
def test_pipeline_split_checkpoint_restores_the_tied_head(kind):
    """Split files of a pipeline-parallel model with tied embeddings: the last stage gets its head back (its own
    copy is saved even where the model leaves `lm_head.weight` out of merged files, and the first stage's tensor
    is sent over after loading)."""
    with tempfile.TemporaryDirectory() as d:
        model = build(kind).eval()
        model.save_pretrained(os.path.join(d, "hf"))
        with torch.no_grad():
            torch.save({"logits": model(input_ids=batch(seed=11)["input_ids"]).logits}, os.path.join(d, "ref.pt"))
        run_distributed(_pp_split_roundtrip, 2, kind, d, "save")
        run_distributed(_pp_split_roundtrip, 2, kind, d, "load")


def _train_pp_zero_ddp(rank, world, kind, steps, tmpdir, direct=False):
    """Pipeline stages x data-parallel replicas with the framework's own wrapper and ZeRO-1 optimizer.
    ``direct``: call the model itself instead of the wrapper's ``forward`` (the wrapper then only learns from the
    pipeline engine which micro-batch is the last one)."""
    from oslo_b200.optim import FusedAdamW
    from oslo_b200.parallel.data_parallel import DistributedDataParallel
    model = ob.parallelize(build(kind).train(), pipeline_parallel_size=2, micro_batch_size=1)
    mpu = model.mpu
    opt = FusedAdamW(model.gpu_parameters(), lr=1e-2, weight_decay=0.01, shard_group=mpu.get_data_parallel_group(),
                     model_parallel_group=mpu.get_model_parallel_group())
    ddp = DistributedDataParallel(model, mpu, optimizer=opt, bucket_mb=0.01)
    dp, dpr = mpu.get_data_parallel_world_size(), mpu.get_data_parallel_rank()
    for s in range(steps):
        b = batch(seed=3 + s)
        n = b["input_ids"].size(0) // dp
        mine = {k: v[dpr * n:(dpr + 1) * n] for k, v in b.items()}
        opt.zero_grad()
        for out in (model if direct else ddp)(**mine):
            (out.loss / n).backward()
        opt.step()
    model.save_pretrained_with_parallel(os.path.join(tmpdir, "merged"), save_with_merging=True)


@pytest.mark.parametrize("kind", ["gpt_neo", "gptj"])
def test_pipeline_with_bucketed_ddp_and_zero1_matches_single_process(kind):
    """PP2 x DP2 through the bucketed wrapper: with a tied embedding (GPT-Neo) the first / last stage sum of its
    gradient and the data-parallel reduction of its bucket touch the same memory and must not overlap."""
    steps = 3
    torch.manual_seed(0)
    ref = build(kind).train()
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.01)
    for s in range(steps):
        opt.zero_grad()
        ref(**batch(seed=3 + s)).loss.backward()
        opt.step()
    with tempfile.TemporaryDirectory() as d:
        run_distributed(_train_pp_zero_ddp, 4, kind, steps, d)
        got = torch.load(os.path.join(d, "merged", "pytorch_model.bin"), weights_only=True)
    for k, v in ref.state_dict().items():
        if k in got:
            assert torch.allclose(got[k], v, atol=2e-4), (k, (got[k] - v).abs().max())


def _train_wrapper_layout(rank, world, kind, tp, pp, steps, tmpdir, seq_par, balanced=False):
    """Any tp x pp layout with data-parallel replicas over the remaining ranks: bucketed wrapper, ZeRO-1, clipping."""
    from oslo_b200.optim import FusedAdamW
    from oslo_b200.parallel.data_parallel import DistributedDataParallel
    from oslo_b200.parallel.engine_pipeline import balanced_partition
    model = ob.parallelize(build(kind).train(), tensor_parallel_size=tp, pipeline_parallel_size=pp, micro_batch_size=1,
                           sequence_parallel=seq_par, pipeline_partition=balanced_partition(4, pp) if balanced else None)
    mpu = model.mpu
    opt = FusedAdamW(model.gpu_parameters(), lr=1e-2, weight_decay=0.01, max_grad_norm=0.5, model=model,
                     shard_group=mpu.get_data_parallel_group(), model_parallel_group=mpu.get_model_parallel_group())
    ddp = DistributedDataParallel(model, mpu, optimizer=opt, bucket_mb=0.01)
    dp, dpr = mpu.get_data_parallel_world_size(), mpu.get_data_parallel_rank()
    for s in range(steps):
        b = batch(seed=3 + s, vocab=104 if kind == "gptj" else 101)
        n = b["input_ids"].size(0) // dp
        mine = {k: v[dpr * n:(dpr + 1) * n] for k, v in b.items()}
        opt.zero_grad()
        if pp > 1:
            for out in ddp(**mine, output_logits=not balanced):
                (out.loss / n).backward()
        else:
            ddp(**mine).loss.backward()
        opt.step()
    model.save_pretrained_with_parallel(os.path.join(tmpdir, "merged"), save_with_merging=True)


@pytest.mark.parametrize("kind,tp,pp,world,seq_par,balanced", [
    ("gptj", 2, 1, 4, False, False), ("gpt2", 2, 1, 4, True, False), ("gptj", 2, 2, 8, False, False),
    ("gpt2", 2, 2, 8, False, False),
    ("gpt_neo", 2, 2, 8, False, True)])     # the GPT-Neo benchmark layout: uneven vocabulary, 3 + 1 blocks, fused loss
def test_wrapper_zero1_and_clipping_under_tensor_and_pipeline_parallel_replicas(kind, tp, pp, world, seq_par, balanced):
    """Tensor (and pipeline) parallel replicas x 2 data-parallel replicas with this package's wrapper, ZeRO-1 and
    global-norm clipping: merged weights equal one process training on the whole batch with ``clip_grad_norm_``."""
    steps = 2
    torch.manual_seed(0)
    ref = build(kind).train()
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.01)
    for s in range(steps):
        opt.zero_grad()
        ref(**batch(seed=3 + s, vocab=104 if kind == "gptj" else 101)).loss.backward()
        torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.5)
        opt.step()
    with tempfile.TemporaryDirectory() as d:
        run_distributed(_train_wrapper_layout, world, kind, tp, pp, steps, d, seq_par, balanced)
        got = torch.load(os.path.join(d, "merged", "pytorch_model.bin"), weights_only=True)
    for k, v in ref.state_dict().items():
        if k in got:
            assert torch.allclose(got[k], v, atol=3e-4), (k, float((got[k] - v).abs().max()))


def test_pipeline_with_bucketed_ddp_when_the_model_is_called_directly():
    """PP2 x DP2 with two micro-batches per replica, driving ``model(...)`` and not the wrapper: the bucket reductions
    must still start during the LAST micro-batch's backward only (started during the first one, the later
    micro-batches' gradients would never be reduced)."""
    kind, steps = "gptj", 3
    torch.manual_seed(0)
    ref = build(kind).train()
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.01)
    for s in range(steps):
        opt.zero_grad()
        ref(**batch(seed=3 + s)).loss.backward()
        opt.step()
    with tempfile.TemporaryDirectory() as d:
        run_distributed(_train_pp_zero_ddp, 4, kind, steps, d, True)
        got = torch.load(os.path.join(d, "merged", "pytorch_model.bin"), weights_only=True)
    for k, v in ref.state_dict().items():
        if k in got:
            assert torch.allclose(got[k], v, atol=2e-4), (k, (got[k] - v).abs().max())


def _train_ddp_unsharded(rank, world, steps, tmpdir, clip):
    from oslo_b200.optim import FusedAdamW
    from oslo_b200.parallel.data_parallel import DistributedDataParallel
    model = ob.parallelize(build("gptj").train(), tensor_parallel_size=1)
    mpu = model.mpu
    opt = FusedAdamW(model.gpu_parameters(), lr=1e-2, weight_decay=0.01, max_grad_norm=clip)   # no shard_group
    ddp = DistributedDataParallel(model, mpu, optimizer=opt, bucket_mb=0.01)
    for s in range(steps):
        b = batch(seed=3 + s, bsz=4 * world)
        n = b["input_ids"].size(0) // world
        opt.zero_grad()
        ddp(**{k: v[rank * n:(rank + 1) * n] for k, v in b.items()}).loss.backward()
        opt.step()
    if rank == 0:
        torch.save({k: v.detach().clone() for k, v in model.state_dict().items()}, os.path.join(tmpdir, "state.pt"))


def test_bucketed_ddp_with_unsharded_fused_adamw_averages_and_clips_like_one_process():
    """Plain data parallelism (no ZeRO-1): the summed buckets become the mean inside the optimizer, so a clipping
    threshold that bites sees the same norm as a single process on the whole batch."""
    steps, world, clip = 3, 2, 1.0
    torch.manual_seed(0)
    ref = build("gptj").train()
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.01)
    norms = []
    for s in range(steps):
        opt.zero_grad()
        ref(**batch(seed=3 + s, bsz=4 * world)).loss.backward()
        norms.append(float(torch.nn.utils.clip_grad_norm_(ref.parameters(), clip)))
        opt.step()
    # a gradient left as the SUM over two replicas has twice the norm: it would be clipped in steps where the mean is not
    assert max(norms) > clip and any(clip / world < n < clip for n in norms), norms
    with tempfile.TemporaryDirectory() as d:
        run_distributed(_train_ddp_unsharded, world, steps, d, clip)
        got = torch.load(os.path.join(d, "state.pt"), weights_only=True)
    for k, v in ref.state_dict().items():
        assert torch.allclose(got[k], v, atol=2e-4), (k, (got[k] - v).abs().max())


def _scaler_ranks(rank, world):
    import torch.distributed as dist
    from oslo_b200.optim import DynamicLossScaler, FusedAdamW
    from oslo_b200.parallel.data_parallel import DistributedDataParallel
    model = ob.parallelize(build("gpt2").train(), pipeline_parallel_size=2, micro_batch_size=2)
    mpu = model.mpu
    opt = FusedAdamW(model.gpu_parameters(), lr=1e-2, shard_group=mpu.get_data_parallel_group(),
                     model_parallel_group=mpu.get_model_parallel_group(), loss_scaler=DynamicLossScaler(init_scale=8.0))
    ddp = DistributedDataParallel(model, mpu, optimizer=opt)
    stepped = []
    for s in range(3):
        opt.zero_grad()
        for out in ddp(**batch(seed=3 + s)):
            opt.loss_scaler.scale(out.loss / 2).backward()
        if s == 1 and rank == 0:
            opt.buf.flat_g[5] = float("nan")          # an overflow that ONE rank sees
        stepped.append(opt.step())
    seen = [None] * world
    dist.all_gather_object(seen, (stepped, opt.step_count, opt.loss_scaler.loss_scale))
    assert all(s == seen[0] for s in seen), seen
    assert stepped == [True, False, True] and opt.step_count == 2 and opt.loss_scaler.loss_scale == 4.0, seen[0]


def test_loss_scaler_skips_on_every_rank_when_one_rank_overflows():
    """PP2 x DP2: the overflow check rides on the gradient-norm reduction over the shard and model-parallel groups."""
    run_distributed(_scaler_ranks, 4)


def _clip_ranks(rank, world, kind, tp, pp, steps, tmpdir):
    from oslo_b200.optim import FusedAdamW
    from oslo_b200.parallel.data_parallel import DistributedDataParallel
    model = ob.parallelize(build(kind).train(), tensor_parallel_size=tp, pipeline_parallel_size=pp, micro_batch_size=1,
                           sequence_parallel=(tp > 1 and pp == 1))
    mpu = model.mpu
    opt = FusedAdamW(model.gpu_parameters(), lr=1e-2, weight_decay=0.01, max_grad_norm=0.5, model=model,
                     shard_group=mpu.get_data_parallel_group(), model_parallel_group=mpu.get_model_parallel_group())
    ddp = DistributedDataParallel(model, mpu, optimizer=opt, bucket_mb=0.01)
    dp, dpr = mpu.get_data_parallel_world_size(), mpu.get_data_parallel_rank()
    for s in range(steps):
        b = batch(seed=3 + s)
        n = b["input_ids"].size(0) // dp
        mine = {k: v[dpr * n:(dpr + 1) * n] for k, v in b.items()}
        opt.zero_grad()
        if pp > 1:
            for out in ddp(**mine):
                (out.loss / n).backward()
        else:
            ddp(**mine).loss.backward()
        opt.step()
    model.save_pretrained_with_parallel(os.path.join(tmpdir, "merged"), save_with_merging=True)


@pytest.mark.parametrize("kind,tp,pp", [("gptj", 2, 1), ("gpt2", 1, 2), ("gpt_neo", 2, 2)])
def test_gradient_clipping_counts_every_parameter_once(kind, tp, pp):
    """Global-norm clipping on model-parallel ranks == `clip_grad_norm_` of one process: tensors replicated over the
    tensor-parallel group and the last stage's copy of a tied embedding must not be counted twice."""
    steps, world = 3, tp * pp * 2 if tp * pp < 4 else 4
    torch.manual_seed(0)
    ref = build(kind).train()
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.01)
    for s in range(steps):
        opt.zero_grad()
        ref(**batch(seed=3 + s)).loss.backward()
        torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.5)
        opt.step()
    with tempfile.TemporaryDirectory() as d:
        run_distributed(_clip_ranks, world, kind, tp, pp, steps, d)
        got = torch.load(os.path.join(d, "merged", "pytorch_model.bin"), weights_only=True)
    for k, v in ref.state_dict().items():
        if k in got:
            assert torch.allclose(got[k], v, atol=3e-4), (k, float((got[k] - v).abs().max()))


def _decay_groups(model):
    """The usual split: matrices decay, biases and LayerNorm parameters do not."""
    decay = [p for p in model.parameters() if p.dim() >= 2]
    rest = [p for p in model.parameters() if p.dim() < 2]
    return [dict(params=decay, weight_decay=0.1), dict(params=rest, weight_decay=0.0, lr=2e-2)]


def _groups_ranks(rank, world, steps, tmpdir):
    from oslo_b200.optim import FusedAdamW
    from oslo_b200.parallel.data_parallel import DistributedDataParallel
    model = ob.parallelize(build("gptj").train(), tensor_parallel_size=1)
    mpu = model.mpu
    opt = FusedAdamW(_decay_groups(model), lr=1e-2, shard_group=mpu.get_data_parallel_group())
    assert [g["weight_decay"] for g in opt.param_groups] == [0.1, 0.0] and opt.param_groups[1]["lr"] == 2e-2
    ddp = DistributedDataParallel(model, mpu, optimizer=opt, bucket_mb=0.01)
    for s in range(steps):
        b = batch(seed=3 + s)
        n = b["input_ids"].size(0) // world
        opt.zero_grad()
        ddp(**{k: v[rank * n:(rank + 1) * n] for k, v in b.items()}).loss.backward()
        if s == 1:
            opt.param_groups[0]["lr"] = 5e-3          # what a learning-rate scheduler does
        opt.step()
    if rank == 0:
        torch.save({k: v.detach().clone() for k, v in model.state_dict().items()}, os.path.join(tmpdir, "state.pt"))


def test_parameter_groups_with_their_own_weight_decay_and_lr():
    """Torch-style groups on the one flat buffer (ZeRO-1 over 2 ranks: the group boundary falls inside a shard)."""
    steps = 3
    torch.manual_seed(0)
    ref = build("gptj").train()
    opt = torch.optim.AdamW(_decay_groups(ref), lr=1e-2)
    for s in range(steps):
        opt.zero_grad()
        ref(**batch(seed=3 + s)).loss.backward()
        if s == 1:
            opt.param_groups[0]["lr"] = 5e-3
        opt.step()
    with tempfile.TemporaryDirectory() as d:
        run_distributed(_groups_ranks, 2, steps, d)
        got = torch.load(os.path.join(d, "state.pt"), weights_only=True)
    for k, v in ref.state_dict().items():
        assert torch.allclose(got[k], v, atol=2e-4), (k, float((got[k] - v).abs().max()))


def _ddp_torch_optimizer_ranks(rank, world, steps, tmpdir):
    from oslo_b200.parallel.data_parallel import DistributedDataParallel
    model = ob.parallelize(build("gptj").train(), tensor_parallel_size=1)
    ddp = DistributedDataParallel(model, model.mpu, bucket_mb=0.01)         # no FusedAdamW: gradients are averaged
    opt = torch.optim.AdamW(model.gpu_parameters(), lr=1e-2, weight_decay=0.01)
    for s in range(steps):
        b = batch(seed=3 + s)
        n = b["input_ids"].size(0) // world
        mine = {k: v[rank * n:(rank + 1) * n] for k, v in b.items()}
        opt.zero_grad()                                # set_to_none=True: drops the views into the flat buffer
        for i in range(2):                             # two micro-batches, reduced once
            mb = {k: v[i:i + 1] for k, v in mine.items()}
            with (ddp.no_sync() if i == 0 else __import__("contextlib").nullcontext()):
                (ddp(**mb).loss / 2).backward()
        ddp.finish_gradient_sync()
        opt.step()
    if rank == 0:
        torch.save({k: v.detach().clone() for k, v in model.state_dict().items()}, os.path.join(tmpdir, "state.pt"))


def test_bucketed_ddp_with_a_torch_optimizer():
    """The wrapper without FusedAdamW: a torch optimizer whose zero_grad() sets gradients to None still gets averaged
    gradients (the hook puts fresh gradient tensors back into the flat buffer)."""
    steps = 3
    torch.manual_seed(0)
    ref = build("gptj").train()
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.01)
    for s in range(steps):
        opt.zero_grad()
        ref(**batch(seed=3 + s)).loss.backward()
        opt.step()
    with tempfile.TemporaryDirectory() as d:
        run_distributed(_ddp_torch_optimizer_ranks, 2, steps, d)
        got = torch.load(os.path.join(d, "state.pt"), weights_only=True)
    for k, v in ref.state_dict().items():
        assert torch.allclose(got[k], v, atol=2e-4), (k, float((got[k] - v).abs().max()))


def _train_custom_partition(rank, world, kind, partition, tp, steps, expected_losses, tmpdir):
    model = ob.parallelize(build(kind).train(), tensor_parallel_size=tp, pipeline_parallel_size=world // tp,
                           micro_batch_size=2, pipeline_partition=partition)
    eng = model._pipe_engine
    assert eng.block_range == (sum(partition[:eng.stage]), sum(partition[:eng.stage + 1]))
    assert model.initial_parameters["pipeline_partition"] == partition
    opt = torch.optim.AdamW([p for p in model.gpu_parameters() if p.requires_grad], lr=1e-2)
    for s in range(steps):
        opt.zero_grad()
        tot = 0.0
        for out in model(**batch(seed=3 + s)):
            out.loss.backward()
            tot += float(out.loss)
        assert abs(tot - expected_losses[s]) < 2e-4, (s, tot, expected_losses[s])
        opt.step()
    model.save_pretrained_with_parallel(os.path.join(tmpdir, "merged"), save_with_merging=True)
    model.save_pretrained_with_parallel(os.path.join(tmpdir, "split"))
    # a split checkpoint comes back with the partition it was written with
    again = getattr(ob, MODEL[kind]).from_pretrained_with_parallel(
        os.path.join(tmpdir, "split"), tensor_parallel_size=tp, pipeline_parallel_size=world // tp, micro_batch_size=2,
        pipeline_partition=partition)
    own, got = model.state_dict(), again.state_dict()
    for k, v in own.items():
        if v.numel():
            assert torch.equal(v, got[k]), k


@pytest.mark.parametrize("kind,partition,tp", [("gptj", [1, 3], 1), ("gpt_neo", [3, 1], 1), ("gptj", [1, 3], 2)])
def test_pipeline_stages_with_an_uneven_partition(kind, partition, tp):
    """``pipeline_partition=[blocks per stage]`` instead of the even split: same losses and merged weights as one
    process; the layout survives a split-checkpoint round trip."""
    steps = 2
    losses, state = oracle_steps(kind, steps, micro=2)
    with tempfile.TemporaryDirectory() as d:
        run_distributed(_train_custom_partition, 2 * tp, kind, partition, tp, steps, losses, d)
        _check_merged(d, state, atol=2e-4)


def test_pipeline_partition_is_validated():
    from oslo_b200.parallel.engine_pipeline import PipelineParallelEngine

    class _M:
        def num_blocks(self):
            return 4

    class _Mpu:
        device = torch.device("cpu")

        def get_pipeline_parallel_world_size(self):
            return 2

        def get_pipeline_parallel_rank(self):
            return 0

        @staticmethod
        def make_pipeline_partition(n, p):
            return [0, 2, 4]

    assert PipelineParallelEngine(_M(), _Mpu())._bounds() == [0, 2, 4]
    assert PipelineParallelEngine(_M(), _Mpu(), partition=[1, 3])._bounds() == [0, 1, 4]
    for bad in ([4], [1, 2], [0, 4], [2, 2, 0]):
        with pytest.raises(ValueError):
            PipelineParallelEngine(_M(), _Mpu(), partition=bad)._bounds()


def _bench_layout_in_miniature(rank, world, steps, expected_losses, tmpdir):
    """tp2 x pp4 on 8 ranks with the balanced split of 8 blocks (2-2-3-1), 4 micro-batches per step, the fused loss,
    ``FusedAdamW`` with global-norm clipping over the model-parallel group: the 8-GPU benchmark layout, small."""
    from oslo_b200.optim import FusedAdamW
    from oslo_b200.parallel.engine_pipeline import balanced_partition
    torch.manual_seed(7)
    cfg = ob.GPTJConfig(vocab_size=104, n_positions=32, n_embd=32, n_layer=8, n_head=4, rotary_dim=4)
    partition = balanced_partition(8, 4)
    assert partition == [2, 2, 3, 1]
    model = ob.parallelize(ob.GPTJForCausalLM(cfg).train(), tensor_parallel_size=2, pipeline_parallel_size=4,
                           micro_batch_size=2, pipeline_partition=partition)
    mpu = model.mpu
    opt = FusedAdamW(model.gpu_parameters(), lr=1e-2, weight_decay=0.01, max_grad_norm=0.5,
                     model_parallel_group=mpu.get_model_parallel_group())
    for s in range(steps):
        b = batch(seed=3 + s, bsz=8, vocab=104)
        opt.zero_grad()
        tot = 0.0
        for out in model(**b, output_logits=False):
            (out.loss / 4).backward()
            tot += float(out.loss.detach()) / 4
        assert abs(tot - expected_losses[s]) < 3e-4, (s, tot, expected_losses[s])
        opt.step()
    model.save_pretrained_with_parallel(os.path.join(tmpdir, "merged"), save_with_merging=True)


def test_the_eight_gpu_benchmark_layout_in_miniature():
    steps = 2
    torch.manual_seed(7)
    cfg = ob.GPTJConfig(vocab_size=104, n_positions=32, n_embd=32, n_layer=8, n_head=4, rotary_dim=4)
    ref = ob.GPTJForCausalLM(cfg).train()
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.01)
    losses = []
    for s in range(steps):
        b = batch(seed=3 + s, bsz=8, vocab=104)
        opt.zero_grad()
        loss = ref(**b).loss
        loss.backward()
        torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.5)
        opt.step()
        losses.append(float(loss.detach()))
    with tempfile.TemporaryDirectory() as d:
        run_distributed(_bench_layout_in_miniature, 8, steps, losses, d)
        got = torch.load(os.path.join(d, "merged", "pytorch_model.bin"), weights_only=True)
    for k, v in ref.state_dict().items():
        if k in got:
            assert torch.allclose(got[k], v, atol=3e-4), (k, float((got[k] - v).abs().max()))

