"""Auxiliary subsystems on the host: heartbeat failure detection, deadlines, timers, metrics, config."""
import json
import os
import time

import pytest
import torch
import torch.distributed as dist

from oslo_b200 import config as cfgmod
from oslo_b200.utils import (DeviceTimer, Heartbeat, MetricsLogger, RankFailure, StepDeadline, load_measured_peaks,
                             roofline_fraction)
from tests.dist_utils import run_distributed


def _hb(rank, world):
    dist.init_process_group("gloo", rank=rank, world_size=world)
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, period_s=0.1, misses=3).start()
    time.sleep(0.5)
    hb.check_peers()  # everyone alive
    dist.barrier()
    if rank == 1:
        hb.pause()  # rank 1 wedges: it stays in the job but stops beating
        time.sleep(2.0)
    else:
        deadline = time.time() + 5
        detected = None
        while time.time() < deadline and detected is None:
            time.sleep(0.1)
            try:
                hb.check_peers()
            except RankFailure as e:
                detected = e.dead
        assert detected == [1], detected
    hb.stop()


def test_heartbeat_detects_wedged_rank():
    run_distributed(_hb, 2)


def _short_pg_timeout(rank, world):
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=2))
    t = torch.ones(1)
    dist.all_reduce(t)
    if rank == 1:
        time.sleep(6)  # never joins the second collective in time
        return
    with pytest.raises(Exception):
        dist.all_reduce(t)  # ends with an error instead of hanging


def test_collective_timeout_instead_of_hang():
    run_distributed(_short_pg_timeout, 2)


def test_step_deadline_and_timer(tmp_path):
    with pytest.raises(TimeoutError):
        with StepDeadline(0.05):
            time.sleep(0.2)
    with StepDeadline(5):
        pass
    timer = DeviceTimer()
    with timer("work"):
        time.sleep(0.01)
    assert timer.summary()["work"] >= 5.0
    path = tmp_path / "m.jsonl"
    ml = MetricsLogger(str(path), rank=0)
    rec = ml.log_step(1, loss=2.5, tokens=1000, flops=1e12)
    assert rec["loss"] == 2.5 and json.loads(path.read_text().splitlines()[0])["step"] == 1


def test_roofline_and_config(monkeypatch):
    peaks = load_measured_peaks("/nonexistent")
    assert peaks["source"] == "fallback" and peaks["bf16_tflops"] == 1590.0
    r = roofline_fraction(flops=1e15, nvlink_bytes=1e9, seconds=1.0, peak_tflops=1000.0)
    assert abs(r["fraction"] - 1.0) < 1e-9 and r["t_link_s"] < r["t_compute_s"]
    monkeypatch.setenv("OSLO_B200_DDP_BUCKET_MB", "32")
    monkeypatch.setenv("OSLO_B200_USE_MULTIMEM", "0")
    c = cfgmod.OsloConfig.from_env()
    assert c.ddp_bucket_mb == 32 and c.use_multimem is False


@pytest.mark.parametrize("kind", ["gptj", "gpt2", "gpt_neo"])
def test_graphed_greedy_decoder_matches_generate_on_cpu(kind):
    """The device-position cache bookkeeping of the CUDA-graph decoder, run eagerly, equals generate()."""
    import oslo_b200 as ob
    from oslo_b200.generation import GraphedGreedyDecoder
    torch.manual_seed(0)
    if kind == "gptj":
        model = ob.GPTJForCausalLM(ob.GPTJConfig(vocab_size=512, n_positions=128, n_embd=64, n_layer=2, n_head=4,
                                                 rotary_dim=8)).eval()
    elif kind == "gpt2":
        model = ob.GPT2LMHeadModel(ob.GPT2Config(vocab_size=512, n_positions=128, n_embd=64, n_layer=2, n_head=4)).eval()
    else:
        model = ob.GPTNeoForCausalLM(ob.GPTNeoConfig(vocab_size=512, max_position_embeddings=128, hidden_size=64,
                                                     num_layers=2, num_heads=4, window_size=8)).eval()
    ids = torch.randint(0, 512, (2, 7))
    dec = GraphedGreedyDecoder(model, max_len=64)
    for prompt, n_new in ((7, 12), (5, 10)):
        want = model.generate(ids[:, :prompt], max_length=prompt + n_new, do_sample=False)
        assert torch.equal(dec.generate(ids[:, :prompt], n_new), want)


def test_generate_cuda_graph_flag_equals_greedy_search_with_eos():
    """generate(cuda_graph=True) pads rows after their eos and stops where greedy_search stops."""
    import oslo_b200 as ob
    torch.manual_seed(0)
    cfg = ob.GPTJConfig(vocab_size=64, n_positions=128, n_embd=64, n_layer=2, n_head=4, rotary_dim=8)
    model = ob.GPTJForCausalLM(cfg).eval()
    for rows in (1, 3):
        ids = torch.randint(0, 64, (rows, 7))
        full = model.generate(ids, max_length=32, do_sample=False)
        for eos in sorted(set(full[0, 7:].tolist()))[:6] + [None]:
            want = model.generate(ids, max_length=32, do_sample=False, eos_token_id=eos, pad_token_id=0)
            got = model.generate(ids, max_length=32, do_sample=False, eos_token_id=eos, pad_token_id=0, cuda_graph=True)
            assert want.shape == got.shape and torch.equal(want, got), (rows, eos)


def test_fake_tensor_implementations_trace_without_a_gpu():
    """The operators can be traced under FakeTensorMode: shapes, dtypes and the attention output layout."""
    from torch._subclasses.fake_tensor import FakeTensorMode
    from oslo_b200 import ops
    ext = ops.load_ext()
    if ext is None:
        pytest.skip("extension not built")
    with FakeTensorMode():
        a = torch.empty(64, 128, dtype=torch.bfloat16, device="cuda")
        w = torch.empty(256, 128, dtype=torch.bfloat16, device="cuda")
        y = ext.gemm(a, w, 0, 0, None, None, None, None, 0, 1.0)
        assert y.shape == (64, 256) and y.dtype == torch.bfloat16
        y32 = ext.gemm(a, w, 0, 0, None, None, None, None, 32, 1.0)
        assert y32.dtype == torch.float32
        q = torch.empty(2, 16, 4, 64, dtype=torch.bfloat16, device="cuda").permute(0, 2, 1, 3)
        o, lse = ext.flash_fwd(q, q, q, 0.125, True, 0, None, 1)
        assert o.shape == (2, 4, 16, 64) and o.stride(-1) == 1 and lse.shape == (2, 4, 16)
        ln, mean, rstd = ext.layernorm_fwd(a, torch.empty(128, dtype=torch.bfloat16, device="cuda"), None, 1e-5)
        assert ln.shape == a.shape and mean.shape == (64,) and mean.dtype == torch.float32
        assert ext.gemv_rows(a[:2], None, w, None, -1).shape == (2, 256)
        labels = torch.empty(64, dtype=torch.long, device="cuda")
        mx, se, tg = ext.gemm_ce_stats(a, w, 0, None, labels, 0)
        assert mx.shape == se.shape == tg.shape == (64,) and mx.dtype == torch.float32
        d = ext.gemm_ce_grad(a, w, 0, None, labels, 0, mx, se)
        assert d.shape == (64, 256) and d.dtype == torch.bfloat16


def test_debug_sync_wrapper_reports_the_failing_operator(monkeypatch):
    """OSLO_B200_DEBUG_SYNC: the checked namespace reads the error word after a call and names the operator."""
    from oslo_b200.ops import cuda_ops

    class FakeExt:
        def __init__(self):
            self.word = torch.zeros(1, dtype=torch.int32)
            self.calls = []

        def error_word(self, like):
            return self.word

        def gemm(self, a):
            self.calls.append("gemm")
            return a + 1

        def bad(self, a):
            self.word.fill_(5)
            return a

    class Cuda(torch.Tensor):      # a CPU tensor that claims to live on a GPU, so the wrapper looks at the error word
        @property
        def is_cuda(self):
            return True

    fake = FakeExt()
    checked = cuda_ops._CheckedOps(fake)
    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a, **k: None)
    monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: False)
    x = torch.zeros(3).as_subclass(Cuda)
    assert torch.equal(torch.Tensor(checked.gemm(x)), torch.ones(3)) and fake.calls == ["gemm"]
    with pytest.raises(RuntimeError, match="`bad`.*code 5"):
        checked.bad(x)
    assert int(fake.word.item()) == 0      # the word is cleared once reported


def test_training_resumes_bit_exactly_from_model_and_optimizer_state(tmp_path):
    """Checkpoint / resume: 2 steps + save + reload into fresh objects + 1 step == 3 uninterrupted steps."""
    import oslo_b200 as ob
    from oslo_b200.optim import FusedAdamW
    cfg = ob.GPTJConfig(vocab_size=64, n_positions=32, n_embd=32, n_layer=2, n_head=4, rotary_dim=4)
    ids = torch.randint(0, 64, (2, 16), generator=torch.Generator().manual_seed(3))

    def make():
        torch.manual_seed(0)
        m = ob.GPTJForCausalLM(cfg).train()
        return m, FusedAdamW(m.parameters(), lr=1e-2, weight_decay=0.1, max_grad_norm=1.0)

    def step(m, o):
        o.zero_grad()
        loss = m(input_ids=ids, labels=ids).loss
        loss.backward()
        o.step()
        return float(loss)

    m, o = make()
    want = [step(m, o) for _ in range(3)]
    want_state = {k: v.clone() for k, v in m.state_dict().items()}

    m, o = make()
    got = [step(m, o) for _ in range(2)]
    m.save_pretrained(str(tmp_path / "ckpt"))
    torch.save(o.state_dict(), tmp_path / "optim.pt")
    m2 = ob.GPTJForCausalLM.from_pretrained(str(tmp_path / "ckpt")).train()
    o2 = FusedAdamW(m2.parameters(), lr=1e-2, weight_decay=0.1, max_grad_norm=1.0)
    o2.load_state_dict(torch.load(tmp_path / "optim.pt", weights_only=False))
    got.append(step(m2, o2))
    assert got == want
    for k, v in m2.state_dict().items():
        assert torch.equal(v, want_state[k]), k


def test_dynamic_loss_scaler_matches_unscaled_training_and_skips_overflow():
    """Loss scaling: scaled and unscaled runs give the same parameters; an overflowed step changes nothing but the
    scale; the scale grows again after `growth_interval` clean steps; the scaler state rides in the optimizer state."""
    import oslo_b200 as ob
    from oslo_b200.optim import DynamicLossScaler, FusedAdamW
    cfg = ob.GPT2Config(vocab_size=64, n_positions=32, n_embd=32, n_layer=2, n_head=4, resid_pdrop=0.0,
                        embd_pdrop=0.0, attn_pdrop=0.0)
    ids = torch.randint(0, 64, (2, 16), generator=torch.Generator().manual_seed(5))

    def make(scaler):
        torch.manual_seed(0)
        m = ob.GPT2LMHeadModel(cfg).train()
        return m, FusedAdamW(m.parameters(), lr=1e-2, weight_decay=0.1, max_grad_norm=1.0, loss_scaler=scaler)

    def step(m, o, poison=False):
        o.zero_grad()
        loss = m(input_ids=ids, labels=ids).loss
        (o.loss_scaler.scale(loss) if o.loss_scaler is not None else loss).backward()
        if poison:
            o.buf.flat_g[3] = float("inf")
        return o.step()

    m0, o0 = make(None)
    for _ in range(3):
        assert step(m0, o0) is True
    scaler = DynamicLossScaler(init_scale=2.0 ** 8, growth_interval=2)
    m1, o1 = make(scaler)
    assert step(m1, o1) is True and scaler.loss_scale == 2.0 ** 8
    before = o1.buf.flat_p.clone()
    assert step(m1, o1, poison=True) is False                    # skipped: nothing moves, the scale halves
    assert torch.equal(o1.buf.flat_p, before) and o1.step_count == 1
    assert scaler.loss_scale == 2.0 ** 7 and scaler.skipped_steps == 1
    assert step(m1, o1) is True and step(m1, o1) is True         # two clean steps: the scale doubles again
    assert scaler.loss_scale == 2.0 ** 8 and o1.step_count == 3
    for a, b in zip(m0.parameters(), m1.parameters()):
        assert torch.allclose(a, b, atol=1e-6), float((a - b).detach().abs().max())
    sd = o1.state_dict()
    s2 = DynamicLossScaler()
    _, o2 = make(s2)
    o2.load_state_dict(sd)
    assert s2.loss_scale == scaler.loss_scale and s2.skipped_steps == 1
    with pytest.raises(ValueError):
        DynamicLossScaler(growth_factor=1.0)


def test_training_state_sidecar_restores_optimizer_step_and_generators(tmp_path):
    """`save_training_state` / `load_training_state`: the per-rank sidecar brings back the optimizer, the step
    counter, user extras and the random generators (dropout masks continue where they left off)."""
    import random
    import oslo_b200 as ob
    from oslo_b200.optim import FusedAdamW
    from oslo_b200.utils import load_training_state, save_training_state, state_file
    cfg = ob.GPT2Config(vocab_size=64, n_positions=32, n_embd=32, n_layer=1, n_head=4, resid_pdrop=0.1,
                        embd_pdrop=0.1, attn_pdrop=0.1)
    ids = torch.randint(0, 64, (2, 16), generator=torch.Generator().manual_seed(7))

    def make():
        torch.manual_seed(0)
        m = ob.GPT2LMHeadModel(cfg).train()
        return m, FusedAdamW(m.parameters(), lr=1e-2)

    def step(m, o):
        o.zero_grad()
        loss = m(input_ids=ids, labels=ids).loss
        loss.backward()
        o.step()
        return float(loss)

    m, o = make()
    step(m, o)
    m.save_pretrained(str(tmp_path))
    path = save_training_state(str(tmp_path), o, step=1, extra={"tokens_seen": 32})
    assert path == state_file(str(tmp_path)) and path.endswith("oslo_state_tp=0_pp=0_dp=0.pt")
    want = [step(m, o), random.random(), float(torch.rand(()))]

    torch.manual_seed(123)
    random.seed(99)
    m2 = ob.GPT2LMHeadModel.from_pretrained(str(tmp_path)).train()
    o2 = FusedAdamW(m2.parameters(), lr=1e-2)
    info = load_training_state(str(tmp_path), o2)
    assert info == {"step": 1, "extra": {"tokens_seen": 32}} and o2.step_count == 1
    assert [step(m2, o2), random.random(), float(torch.rand(()))] == want
    with pytest.raises(FileNotFoundError):
        load_training_state(str(tmp_path / "nowhere"), o2)


def test_rank_aware_logger_formats_records_of_child_loggers(capsys):
    """Records logged through `logging.getLogger("oslo_b200.<module>")` reach the package handler with a rank."""
    import logging
    from oslo_b200.utils import get_logger
    get_logger()
    logging.getLogger("oslo_b200.some_module").info("child says %s", "hello")
    err = capsys.readouterr().err
    assert "child says hello" in err and "[rank 0]" in err and "Logging error" not in err


def test_fp32_main_gradients_for_16_bit_parameters():
    """``FusedAdamW(..., grad_dtype=torch.float32)``: bf16 parameters, gradients of the micro-batches of a step add up
    in an fp32 flat buffer. The accumulated gradient equals the fp32 sum of the 16-bit micro-batch gradients exactly,
    where accumulation in bf16 (the default) differs from it by a rounding per addition; a step runs on it."""
    import oslo_b200 as ob
    from oslo_b200.optim import FusedAdamW

    def make():
        torch.manual_seed(0)
        cfg = ob.GPTJConfig(vocab_size=64, n_positions=16, n_embd=32, n_layer=2, n_head=2, rotary_dim=8,
                            torch_dtype=torch.bfloat16)
        return ob.GPTJForCausalLM(cfg).to(torch.bfloat16).train()

    ids = [torch.randint(0, 64, (2, 12), generator=torch.Generator().manual_seed(10 + i)) for i in range(16)]

    def accumulate(grad_dtype):
        model = make()
        opt = FusedAdamW(model.parameters(), lr=1e-3, grad_dtype=grad_dtype)
        opt.zero_grad()
        singles = []
        for x in ids:
            before = opt.buf.flat_g.clone()
            (model(input_ids=x, labels=x).loss / len(ids)).backward()
            singles.append((opt.buf.flat_g.double() - before.double()))
        return model, opt, singles

    model32, opt32, _ = accumulate(torch.float32)
    assert opt32.buf.flat_g.dtype == torch.float32 and opt32.buf.flat_p.dtype == torch.bfloat16
    p0 = next(model32.parameters())
    assert p0.grad.dtype == torch.float32 and p0.grad.data_ptr() == opt32.buf.flat_g.data_ptr()
    # every micro-batch gradient is a bf16 tensor that autograd adds into the fp32 buffer: replay that sum in fp64
    replay = make()
    exact = torch.zeros(opt32.buf.padded, dtype=torch.float64)
    for x in ids:
        replay.zero_grad()
        (replay(input_ids=x, labels=x).loss / len(ids)).backward()
        flat = torch.zeros_like(exact)
        for p, off in zip(replay.parameters(), opt32.buf.offsets):
            flat[off: off + p.numel()] = p.grad.reshape(-1).double()
        exact += flat
    err32 = (opt32.buf.flat_g.double() - exact).norm() / exact.norm()
    model16, opt16, _ = accumulate(None)
    assert opt16.buf.flat_g.dtype == torch.bfloat16
    err16 = (opt16.buf.flat_g.double() - exact).norm() / exact.norm()
    assert err32 < 1e-6 and err16 > 20 * err32, (float(err32), float(err16))
    w0 = opt32.buf.flat_p.clone()
    assert opt32.step() and not torch.equal(opt32.buf.flat_p, w0)
    opt32.zero_grad()
    assert float(opt32.buf.flat_g.abs().max()) == 0.0 and p0.grad.dtype == torch.float32


def test_checkpoint_generations_survive_a_failed_save_and_a_damaged_file(tmp_path):
    """``CheckpointManager`` in one process: the pointer names the newest complete generation, old generations are
    pruned, a save that dies half way (host-side injection: the sidecar writer raises) leaves pointer and files of
    the previous generation alone, ``atomic_save`` never replaces a file by a partial one, and an unreadable file is
    reported by name."""
    import oslo_b200 as ob
    from oslo_b200.optim import FusedAdamW
    from oslo_b200.utils import CheckpointManager, CheckpointUnreadable, atomic_save
    from oslo_b200.utils.checkpoint import load_file
    torch.manual_seed(0)
    model = ob.GPT2LMHeadModel(ob.GPT2Config(vocab_size=61, n_positions=16, n_embd=16, n_layer=1, n_head=2))
    opt = FusedAdamW(model.parameters(), lr=1e-3)
    mgr = CheckpointManager(str(tmp_path / "ck"), keep=2)
    assert mgr.pointer() is None and mgr.latest_usable() is None
    for step in (2, 4, 6):
        mgr.save(model, opt, step)
    assert [os.path.basename(g) for g in mgr.generations()] == ["step-00000006", "step-00000004"]
    assert os.path.basename(mgr.pointer()) == "step-00000006" == os.path.basename(mgr.latest_usable())

    def boom(*a, **k):
        raise OSError("disk full")
    good = model.save_training_state
    object.__setattr__(model, "save_training_state", boom)
    with pytest.raises(OSError):
        mgr.save(model, opt, 8)
    object.__setattr__(model, "save_training_state", good)
    assert os.path.basename(mgr.pointer()) == "step-00000006"           # the half-written generation is not "latest"
    assert os.path.basename(mgr.latest_usable()) == "step-00000006"     # ... and is skipped (no sidecar)

    victim = os.path.join(mgr.pointer(), "pytorch_model.bin")
    with open(victim, "r+b") as f:
        f.truncate(100)
    with pytest.raises(CheckpointUnreadable, match="pytorch_model.bin"):
        load_file(victim)
    assert os.path.basename(mgr.latest_usable()) == "step-00000004"     # falls back past the damaged generation

    target = str(tmp_path / "value.pt")
    atomic_save({"a": 1}, target)

    def half_write(obj, path):
        with open(path, "wb") as f:
            f.write(b"partial")
        raise OSError("killed while writing")
    with pytest.raises(OSError):
        atomic_save({"a": 2}, target, half_write)
    assert torch.load(target)["a"] == 1
