"""The GPU-only Python paths on a machine without a GPU: fused models run forward on FAKE CUDA tensors
(``FakeTensorMode``: shapes, dtypes, strides and devices flow, no memory, no kernels). Every ``x.is_cuda`` branch of
the models, of ``ops/cuda_ops.py`` and of the autograd functions' forward halves executes, with the operators'
shape implementations (``ops/fake_impls.py``) standing in for the kernels. The autograd ENGINE needs a CUDA runtime (it
asks for the device's context), so the backward halves are run by walking the graph and calling every custom
function's ``backward`` with gradients of the recorded shapes."""
import pytest
import torch
from torch._subclasses.fake_tensor import FakeTensorMode

import oslo_b200 as ob
from oslo_b200 import ops


def _model(kind, vocab=1024):
    if kind == "gpt2":
        return ob.GPT2LMHeadModel, ob.GPT2Config(vocab_size=vocab, n_positions=256, n_embd=512, n_layer=2, n_head=8,
                                                  attn_pdrop=0.0)       # with attention dropout the scores are materialised
    if kind == "gpt_neo":
        return ob.GPTNeoForCausalLM, ob.GPTNeoConfig(vocab_size=vocab, max_position_embeddings=256, hidden_size=512,
                                                     num_layers=2, num_heads=8, window_size=64,
                                                     attention_types=[[["global", "local"], 1]])
    return ob.GPTJForCausalLM, ob.GPTJConfig(vocab_size=vocab, n_positions=256, n_embd=512, n_layer=2, n_head=8, rotary_dim=32)


def run_custom_backwards(root):
    """Call ``backward`` of every ``torch.autograd.Function`` node reachable from ``root`` once, with empty gradients
    of the shapes / dtypes / devices the node recorded for its outputs. Returns the names of the functions run."""
    seen, keep, stack, ran = set(), [], [root], []
    while stack:
        node = stack.pop()
        if node is None or id(node) in seen:
            continue
        seen.add(id(node))
        keep.append(node)                  # a live reference: ids of collected wrapper objects would be reused
        stack += [fn for fn, _ in node.next_functions]
        cls = getattr(node, "_forward_cls", None)
        if cls is None:
            continue
        grads = [torch.empty(m.shape, dtype=m.dtype, device=m.device) for m in node._input_metadata]
        out = cls.backward(node, *grads)
        out = out if isinstance(out, tuple) else (out,)
        assert len(out) >= len(node.next_functions), cls.__name__
        for g in out:
            assert g is None or (torch.is_tensor(g) and g.is_cuda), cls.__name__
        ran.append(cls.__name__)
    return ran


@pytest.fixture
def kernels(monkeypatch):
    if ops.load_ext() is None:
        pytest.skip("extension not built")
    monkeypatch.setattr(ops, "kernels_available", lambda: True)


@pytest.mark.parametrize("kind", ["gpt2", "gpt_neo", "gptj"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fused_forward_paths_run_on_fake_cuda_tensors(kernels, kind, dtype):
    cls, cfg = _model(kind)
    with FakeTensorMode():
        with torch.device("cuda"):
            model = cls._from_config(cfg, torch_dtype=dtype)
        model.fuse().train()
        ids = torch.randint(0, 1024, (2, 256), device="cuda")
        out = model(input_ids=ids, labels=ids, output_logits=False)                 # LM head fused with the loss
        assert out.loss.shape == () and out.loss.is_cuda and out.logits is None
        ran = run_custom_backwards(out.loss.grad_fn)                                 # every backward half of the step
        assert ran.count("_Flash") == 2 and ran.count("_LayerNorm") >= 3 and "_LinearCrossEntropy" in ran, ran
        out = model(input_ids=ids, labels=ids)                                       # logits materialised
        assert out.logits.shape == (2, 256, 1024) and out.logits.dtype == dtype
        mask = torch.ones(2, 256, dtype=torch.long, device="cuda")
        out = model(input_ids=ids, attention_mask=mask, output_attentions=True, output_hidden_states=True)
        assert len(out.hidden_states) == 3 and out.attentions[0].shape[-2:] == (256, 256)
        model.gradient_checkpointing_enable()
        assert model(input_ids=ids, labels=ids, output_logits=False).loss.shape == ()
        model.eval()
        with torch.no_grad():
            out = model(input_ids=ids[:, :16], use_cache=True)                       # prefill, then one decode step
            nxt = model(input_ids=ids[:, 16:17], past_key_values=out.past_key_values, use_cache=True)
        assert nxt.logits.shape == (2, 1, 1024)
        from oslo_b200.models.common import StaticKVCache
        with torch.no_grad():                                                        # static cache: the decode kernels' wrappers
            out = model(input_ids=ids[:, :16], past_key_values=StaticKVCache(64), use_cache=True, last_token_logits=True)
            nxt = model(input_ids=ids[:, 16:17], past_key_values=out.past_key_values, use_cache=True)
        assert isinstance(out.past_key_values, StaticKVCache) and nxt.logits.shape == (2, 1, 1024)


def test_optimizer_and_elementwise_wrappers_on_fake_cuda_tensors(kernels):
    from oslo_b200.optim import FusedAdamW
    with FakeTensorMode():
        with torch.device("cuda"):
            lin = torch.nn.Linear(64, 64, dtype=torch.bfloat16)
        opt = FusedAdamW(lin.parameters(), lr=1e-3, max_grad_norm=1.0)
        assert opt.buf.flat_g.is_cuda and opt.master.dtype == torch.float32
        assert opt.step() is True                                                    # norm kernel + Adam kernel
        x = torch.empty(4, 8, 64, dtype=torch.bfloat16, device="cuda")
        assert ops.bias_gelu(x, lin.bias).shape == x.shape
        assert ops.bias_dropout_residual(x, lin.bias, x, 0.1, True).shape == x.shape
        assert ops.layer_norm(x, lin.bias, lin.bias, 1e-5).shape == x.shape
        lp = torch.empty(2, 1024, dtype=torch.float32, device="cuda")
        toks = torch.zeros(2, 9, dtype=torch.long, device="cuda")
        assert ops.ban_repeated_ngrams(toks, lp, 3).shape == lp.shape


# ---------------------------------------------------------------------------------------------------------------
# Tensor-parallel fused paths: rank 0 of a two-rank "fake" process group (collectives return without moving data),
# symmetric memory replaced by fake CUDA buffers. The fused GEMM + collective autograd functions, the fused
# vocabulary lookup and the loss combine then run their Python halves - forward and backward - without a GPU.

def _fake_group(tp, as_rank=0):
    """This process becomes rank ``as_rank`` of a ``tp``-rank fake process group whose symmetric memory is fake CUDA
    buffers."""
    import os
    import torch.distributed as dist
    from torch.testing._internal.distributed.fake_pg import FakeStore
    from oslo_b200.parallel import fused_tp, symmetric
    os.environ["OSLO_B200_BACKEND"] = "fake"
    ops.load_ext()
    ops.kernels_available = lambda: True
    torch.cuda.is_current_stream_capturing = lambda: False
    dist.init_process_group(backend="fake", rank=as_rank, world_size=tp, store=FakeStore())

    class FakeWorkspace(symmetric.SymmetricWorkspace):
        def __init__(self, group, nbytes, device=None):
            self.group, self.world, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
            self.numel = (int(nbytes) + 255) // 256 * 128
            self.buf = torch.empty(self.numel, dtype=torch.bfloat16, device="cuda")
            self.peer_ptrs_dev = self.signal_ptrs_dev = self.mc_ptr = 0
            self.oneshot_half = symmetric.ONESHOT_HALF
            self.oneshot_off = self.numel * 2 - 2 * self.oneshot_half
            self.embed_half = (self.oneshot_off // 2) // 256 * 256
            self.embed_counters = torch.empty(64, dtype=torch.int32, device="cuda")
            self.oneshot_counters = torch.empty(64, dtype=torch.int32, device="cuda")

    class FakeCombine(symmetric.CeCombine):
        def __init__(self, group, device):
            self.group, self.world, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
            self.peer_ptrs_dev = self.signal_ptrs_dev = 0
            self.counters = torch.empty(8, dtype=torch.int32, device="cuda")

    fused_tp.SymmetricWorkspace = symmetric.SymmetricWorkspace = FakeWorkspace
    symmetric.CeCombine = FakeCombine


def _fake_parameters(model):
    fake = {}
    for k, v in list(model.named_parameters()) + list(model.named_buffers()):
        t = torch.empty(v.shape, dtype=v.dtype, device="cuda")
        fake[k] = torch.nn.Parameter(t, requires_grad=v.requires_grad) if isinstance(v, torch.nn.Parameter) else t
    return fake


def _fake_tp_rank(rank, world, kind, seq_par, tp=2, vocab=1024, as_rank=0):
    from collections import Counter
    _fake_group(tp, as_rank)
    cls, cfg = _model(kind, vocab)
    cfg.torch_dtype = torch.bfloat16
    model = ob.parallelize(cls(cfg).to(torch.bfloat16), tensor_parallel_size=tp, sequence_parallel=seq_par)
    model.fuse().train()
    model.mpu.backend, model.mpu.device = "nccl", torch.device("cuda")        # what the fused paths ask for
    with FakeTensorMode():
        fake = _fake_parameters(model)
        ids = torch.randint(0, vocab, (2, 256), device="cuda")
        out = torch.func.functional_call(model, fake, (), dict(input_ids=ids, labels=ids, output_logits=False))
        assert out.loss.shape == () and out.loss.is_cuda
        ran = Counter(run_custom_backwards(out.loss.grad_fn))
        from oslo_b200.models.common import StaticKVCache
        model.eval()
        with torch.no_grad():                      # decode: few-row GEMMs and the one-kernel all-reduce
            pre = torch.func.functional_call(model, fake, (), dict(input_ids=ids[:, :16], past_key_values=StaticKVCache(64),
                                                                   use_cache=True, last_token_logits=True))
            nxt = torch.func.functional_call(model, fake, (), dict(input_ids=ids[:, 16:17], use_cache=True,
                                                                   past_key_values=pre.past_key_values))
        assert nxt.logits.shape == (2, 1, vocab), nxt.logits.shape
    fused = [n for n in ran if "Fused" in n or "TPBlock" in n or "VocabEmbed" in n]
    assert fused, ran                                                          # GEMM + collective functions took part
    assert ran["_LinearCrossEntropy"] == 1 and ran["_LayerNorm"] >= 3, ran
    if kind == "gptj" and not seq_par and tp == 2:
        assert ran["_TPBlockInput"] == 2 and ran["_RowParallelFused"] == 2 and ran["_VocabEmbed"] == 1, ran


@pytest.mark.parametrize("kind,seq_par,tp", [("gptj", False, 2), ("gptj", True, 2), ("gpt2", False, 2), ("gpt_neo", True, 2),
                                             ("gptj", False, 4), ("gpt2", False, 8), ("gpt_neo", False, 8)])
def test_tensor_parallel_fused_paths_on_a_fake_process_group(kind, seq_par, tp):
    from tests.dist_utils import run_distributed
    if ops.load_ext() is None:
        pytest.skip("extension not built")
    run_distributed(_fake_tp_rank, 1, kind, seq_par, tp)


@pytest.mark.parametrize("kind,vocab,tp,as_rank", [("gptj", 50400, 8, 0), ("gpt_neo", 50257, 2, 0), ("gpt_neo", 50257, 2, 1)])
def test_vocabulary_shards_with_unaligned_row_counts_on_fake_cuda(kind, vocab, tp, as_rank):
    """GPT-J's vocabulary over 8 ranks (6300 rows each) and GPT-Neo's over 2 (25129 and 25128 rows): shards whose row
    count is not a multiple of 8 take the logits + separate-kernel route of the loss and library products for the
    gradient GEMMs; both ranks of the uneven split must choose the same collectives."""
    from tests.dist_utils import run_distributed
    if ops.load_ext() is None:
        pytest.skip("extension not built")
    run_distributed(_fake_tp_rank, 1, kind, False, tp, vocab, as_rank)



# ---------------------------------------------------------------------------------------------------------------
# Data-parallel wrapper on symmetric buffers (ZeRO-1): bucket launches on the side stream, the parameter all-gather
# after the optimizer step and the per-unit waits of the next forward, with stand-ins for CUDA streams / events.

def _fake_dp_rank(rank, world):
    import contextlib
    import os
    import torch.distributed as dist
    from torch.testing._internal.distributed.fake_pg import FakeStore
    from oslo_b200.optim import FusedAdamW
    from oslo_b200.parallel import symmetric
    from oslo_b200.parallel.data_parallel import DistributedDataParallel
    from oslo_b200.parallel.mpu import MPU
    os.environ["OSLO_B200_BACKEND"] = "fake"
    ops.load_ext()
    ops.kernels_available = lambda: True
    dist.init_process_group(backend="fake", rank=0, world_size=2, store=FakeStore())
    log = []

    class Stream:
        def wait_stream(self, other):
            log.append("wait_stream")

        def wait_event(self, ev):
            log.append(("wait_event", ev.tag))

    class Event:
        count = 0

        def __init__(self, *a, **k):
            Event.count += 1
            self.tag = Event.count

        def record(self, stream=None):
            log.append(("record", self.tag))

    cur = Stream()
    torch.cuda.Stream, torch.cuda.Event = Stream, Event
    torch.cuda.current_stream = lambda *a: cur
    torch.cuda.stream = lambda s: contextlib.nullcontext()

    class FakeFlat(symmetric.SymmetricFlat):
        def __init__(self, group, numel, dtype, device):
            self.group, self.world, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
            self.tensor = torch.empty(int(numel), dtype=dtype, device=device)
            self.peer_ptrs_dev = self.signal_ptrs_dev = self.mc_ptr = 0
            self.shard = -(-int(numel) // (8 * self.world)) * 8

    symmetric.SymmetricFlat = FakeFlat
    symmetric.symmetric_flat_usable = lambda group, dtype, device: True
    mpu = MPU(1, 1)                                    # two data-parallel replicas
    cls, cfg = _model("gptj")
    with FakeTensorMode():
        with torch.device("cuda"):
            model = cls._from_config(cfg, torch_dtype=torch.bfloat16)
        model.fuse().train()
        opt = FusedAdamW(model.parameters(), lr=1e-4, max_grad_norm=1.0, shard_group=mpu.get_data_parallel_group())
        ddp = DistributedDataParallel(model, mpu, optimizer=opt, bucket_mb=1.0)
        n = len(ddp.buckets)
        assert ddp._symm and ddp._zero and n > 3 and len(ddp._param_events) == n
        ids = torch.randint(0, 1024, (2, 256), device="cuda")
        for _ in range(2):
            opt.zero_grad()
            for i in range(2):
                with (ddp.no_sync() if i == 0 else contextlib.nullcontext()):
                    out = ddp(input_ids=ids, labels=ids, output_logits=False)
                    assert not ddp._param_pending                  # every unit has waited for its parameter buckets
                    run_custom_backwards(out.loss.grad_fn)
                    before = log.count("wait_stream")
                    for p in reversed(opt.buf.params):             # what autograd's post-accumulate hooks do
                        ddp._hook(p)
                    launched = log.count("wait_stream") - before
                    assert launched == (0 if i == 0 else n), (i, launched)     # reductions in the last micro-batch only
            assert opt.step() is True
            assert sorted(ddp._param_pending) == list(range(n))     # all parameter buckets are in flight
            records = [e for e in log if isinstance(e, tuple) and e[0] == "record"][-n:]
            assert sorted(e[1] for e in records) == sorted(ev.tag for ev in ddp._param_events)
        model.state_dict()                                          # a checkpoint waits for everything that is left
        assert not ddp._param_pending


def test_symmetric_data_parallel_bookkeeping_on_fake_cuda():
    from tests.dist_utils import run_distributed
    if ops.load_ext() is None:
        pytest.skip("extension not built")
    run_distributed(_fake_dp_rank, 1)


def _bench_shape_rank(rank, world, tp, micro):
    """One GPT-J-6B-wide block + embeddings + head at the benchmark's per-step shapes on rank 0 of ``tp`` ranks."""
    from collections import Counter
    from oslo_b200.modeling_utils import no_weight_init
    from oslo_b200.parallel import fused_tp, vocab_parallel
    _fake_group(tp)
    calls, routes = Counter(), []
    real_call = fused_tp.FusedTP._call

    def spy(self, a, b, a_mn, b_mn, bias, aux_out, out, flags, M, N, K, mode, aux=None):
        calls[(mode, M, N, K)] += 1
        return real_call(self, a, b, a_mn, b_mn, bias, aux_out, out, flags, M, N, K, mode, aux)

    real_route = vocab_parallel._epilogue_ce_ok

    def route(*a):
        routes.append(real_route(*a))
        return routes[-1]

    fused_tp.FusedTP._call = spy
    vocab_parallel._epilogue_ce_ok = route
    cfg = ob.GPTJConfig(vocab_size=50400, n_positions=2048, n_embd=4096, n_layer=1, n_head=16, rotary_dim=64,
                        torch_dtype=torch.bfloat16)
    with no_weight_init():
        model = ob.GPTJForCausalLM(cfg).to(torch.bfloat16)
    model = ob.parallelize(model, tensor_parallel_size=tp)
    model.fuse().train()
    model.mpu.backend, model.mpu.device = "nccl", torch.device("cuda")
    with FakeTensorMode():
        ids = torch.randint(0, 50400, (micro, 2048), device="cuda")
        out = torch.func.functional_call(model, _fake_parameters(model), (), dict(input_ids=ids, labels=ids, output_logits=False))
        ran = Counter(run_custom_backwards(out.loss.grad_fn))
    tokens = micro * 2048
    # forward: attention projection + fc_out as ONE fused GEMM + all-reduce; backward: ONE for the four input gradients
    assert calls == {(1, tokens, 4096, 4 * 4096 // tp): 2}, dict(calls)
    assert ran["_TPBlockInput"] == 1 and ran["_RowParallelFused"] == 1 and ran["_Flash"] == 1, dict(ran)
    # the loss: cross-entropy inside the LM-head GEMM where every vocabulary shard has a multiple of 8 rows
    assert routes == [50400 // tp % 8 == 0], routes


@pytest.mark.parametrize("tp,micro", [(2, 8), (4, 16), (8, 8)])
def test_benchmark_shapes_take_the_fused_paths(tp, micro):
    """The per-step shapes of ``bench.py`` (GPT-J-6B width, 8 x 2048 tokens per GPU, tp2 / tp4 / tp8): which fused
    kernels the step consists of, checked on fake CUDA tensors."""
    from tests.dist_utils import run_distributed
    if ops.load_ext() is None:
        pytest.skip("extension not built")
    run_distributed(_bench_shape_rank, 1, tp, micro)


def _record_collectives(trace):
    """Append (name, shape, group size) of every collective this process issues - torch.distributed calls and this
    package's collective operators - to ``trace``."""
    import torch.distributed as dist
    from oslo_b200.parallel import fused_tp, symmetric

    def wrap_dist(name):
        real = getattr(dist, name)

        def spy(tensor, *a, **k):
            t = tensor[0] if isinstance(tensor, (list, tuple)) else tensor
            trace.append((name, tuple(t.shape), dist.get_world_size(k.get("group"))))
            return real(tensor, *a, **k)
        setattr(dist, name, spy)

    for name in ("all_reduce", "broadcast", "all_gather_into_tensor", "reduce_scatter_tensor", "all_gather"):
        wrap_dist(name)
    real_call = fused_tp.FusedTP._call

    def fused(self, a, b, a_mn, b_mn, bias, aux_out, out, flags, M, N, K, mode, aux=None):
        trace.append(("gemm_comm", (mode, M, N, K), self.world))
        return real_call(self, a, b, a_mn, b_mn, bias, aux_out, out, flags, M, N, K, mode, aux)
    fused_tp.FusedTP._call = fused
    real_combine = symmetric.CeCombine.__call__

    def combine(self, mx, se, tg):
        trace.append(("ce_combine", tuple(mx.shape), self.world))
        return real_combine(self, mx, se, tg)
    symmetric.CeCombine.__call__ = combine
    real_embed = symmetric.vocab_embed

    def embed(ws, ids, weight, lo, hi):
        trace.append(("vocab_embed", tuple(ids.shape), ws.world))
        return real_embed(ws, ids, weight, lo, hi)
    symmetric.vocab_embed = embed


def _neo_shape_rank(rank, world, as_rank, out_dir=None):
    """Two GPT-Neo-1.3B-wide blocks (one global, one local) at 4 x 2048 tokens per micro-batch on rank ``as_rank`` of 2:
    the shapes of the tp2 x pp2 x dp2 configuration, with its 50257-word vocabulary split 25129 / 25128."""
    from collections import Counter
    from oslo_b200.modeling_utils import no_weight_init
    from oslo_b200.parallel import fused_tp
    _fake_group(2, as_rank)
    trace = []
    _record_collectives(trace)
    cfg = ob.GPTNeoConfig(vocab_size=50257, max_position_embeddings=2048, hidden_size=2048, num_layers=2, num_heads=16,
                          window_size=256, attention_types=[[["global", "local"], 1]], torch_dtype=torch.bfloat16)
    with no_weight_init():
        model = ob.GPTNeoForCausalLM(cfg).to(torch.bfloat16)
    model = ob.parallelize(model, tensor_parallel_size=2)
    model.fuse().train()
    model.mpu.backend, model.mpu.device = "nccl", torch.device("cuda")
    assert model.transformer.wte.weight.size(0) == (25129 if as_rank == 0 else 25128)
    with FakeTensorMode():
        ids = torch.randint(0, 50257, (4, 2048), device="cuda")
        out = torch.func.functional_call(model, _fake_parameters(model), (), dict(input_ids=ids, labels=ids, output_logits=False))
        ran = Counter(run_custom_backwards(out.loss.grad_fn))
    # per block: out_proj and c_proj forward, q / k / v / c_fc input gradients backward, each a GEMM + all-reduce
    calls = Counter(shape for name, shape, _ in trace if name == "gemm_comm")
    assert calls == {(1, 8192, 2048, 1024): 8, (1, 8192, 2048, 4096): 4}, dict(calls)
    assert ran["_VocabEmbed"] == 1 and ran["_Flash"] == 2 and ran["_LinearCrossEntropy"] == 1, dict(ran)
    if out_dir:
        import json
        import os
        with open(os.path.join(out_dir, f"trace{as_rank}.json"), "w") as f:
            json.dump(trace, f)


def test_gpt_neo_1_3b_shapes_issue_the_same_collectives_on_both_ranks_of_an_uneven_vocabulary_split(tmp_path):
    """A rank that takes another route than its tensor-parallel peer (which the 25129 / 25128 split of GPT-Neo's
    vocabulary once caused in the loss) issues another sequence of collectives and the job hangs: the sequences of
    the two ranks - names, shapes, group sizes, in order - are compared."""
    import json
    from tests.dist_utils import run_distributed
    if ops.load_ext() is None:
        pytest.skip("extension not built")
    for r in (0, 1):
        run_distributed(_neo_shape_rank, 1, r, str(tmp_path))
    a, b = (json.load(open(tmp_path / f"trace{r}.json")) for r in (0, 1))
    assert len(a) > 15 and a == b, [(x, y) for x, y in zip(a, b) if x != y][:5]


def _trace_rank(rank, world, kind, tp, vocab, seq_par, as_rank, out_dir):
    import json
    import os
    _fake_group(tp, as_rank)
    trace = []
    _record_collectives(trace)
    cls, cfg = _model(kind, vocab)
    cfg.torch_dtype = torch.bfloat16
    model = ob.parallelize(cls(cfg).to(torch.bfloat16), tensor_parallel_size=tp, sequence_parallel=seq_par)
    model.fuse().train()
    model.mpu.backend, model.mpu.device = "nccl", torch.device("cuda")
    with FakeTensorMode():
        ids = torch.randint(0, vocab, (2, 256), device="cuda")
        for out_logits in (False, True):
            out = torch.func.functional_call(model, _fake_parameters(model), (),
                                             dict(input_ids=ids, labels=ids, output_logits=out_logits))
            run_custom_backwards(out.loss.grad_fn)
    with open(os.path.join(out_dir, f"trace{as_rank}.json"), "w") as f:
        json.dump(trace, f)


@pytest.mark.parametrize("kind,tp,vocab,seq_par", [("gptj", 2, 1021, False), ("gpt2", 4, 1021, False), ("gpt_neo", 4, 1030, True),
                                                   ("gptj", 8, 1000, False)])
def test_all_tensor_parallel_ranks_issue_the_same_collectives(tmp_path, kind, tp, vocab, seq_par):
    """Vocabulary sizes that do not divide evenly (1021 over 2 or 4 ranks) or leave shards with unaligned row counts
    (1000 over 8: 125 rows): every rank of the group issues the same collectives in the same order, for the fused loss
    and for materialised logits."""
    import json
    from tests.dist_utils import run_distributed
    if ops.load_ext() is None:
        pytest.skip("extension not built")
    for r in range(tp):
        run_distributed(_trace_rank, 1, kind, tp, vocab, seq_par, r, str(tmp_path))
    traces = [json.load(open(tmp_path / f"trace{r}.json")) for r in range(tp)]
    assert len(traces[0]) > 10
    for r in range(1, tp):
        assert traces[r] == traces[0], (r, [(x, y) for x, y in zip(traces[0], traces[r]) if x != y][:5])

