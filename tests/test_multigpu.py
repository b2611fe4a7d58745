"""2-GPU checks (NCCL, one process per GPU): tensor-parallel fused training against a single-GPU run,
ZeRO-1 data parallelism, and the symmetric-memory all-reduce kernels against NCCL."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args, errq):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE=os.environ.get("NCCL_NVLS_ENABLE", "1"))
    import traceback
    try:
        import oslo_b200  # noqa: F401 - before the CUDA context exists: the package sets CUDA_DEVICE_MAX_CONNECTIONS
        torch.cuda.set_device(rank)
        fn(rank, world, *args)
    except BaseException:
        errq.put((rank, traceback.format_exc()))
        raise
    finally:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()


def run_gpus(fn, world, *args, timeout=300):
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, errq)) for r in range(world)]
    import time
    for p in procs:
        p.start()
    deadline = time.monotonic() + timeout          # for the whole group, not per process
    for p in procs:
        p.join(max(0.0, deadline - time.monotonic()))
    bad = [p for p in procs if p.exitcode != 0]
    for p in procs:
        if p.is_alive():
            p.kill()
    for p in procs:
        p.join(10)
    if bad:
        msgs = []
        while not errq.empty():
            r, tb = errq.get()
            msgs.append(f"--- rank {r} ---\n{tb}")
        raise AssertionError("\n".join(msgs or ["worker crashed or timed out"]))


def _cfg():
    import oslo_b200 as ob
    return ob.GPTJConfig(vocab_size=2048, n_positions=256, n_embd=512, n_layer=2, n_head=4, rotary_dim=32,
                         torch_dtype=torch.bfloat16)


def _tp_train(rank, world, tmp):
    import oslo_b200 as ob
    from oslo_b200.optim import FusedAdamW
    torch.manual_seed(0)
    model = ob.GPTJForCausalLM(_cfg()).to(torch.bfloat16)
    ids = torch.randint(0, 2048, (4, 128), generator=torch.Generator().manual_seed(1)).cuda()
    ref = torch.load(os.path.join(tmp, "ref.pt"), weights_only=True)
    model.load_state_dict(ref["state"])
    model = ob.parallelize(model, tensor_parallel_size=2)
    model.fuse().train()
    opt = FusedAdamW(model.gpu_parameters(), lr=1e-3)
    losses = []
    for _ in range(3):
        opt.zero_grad()
        loss = model(input_ids=ids, labels=ids, output_logits=False).loss
        loss.backward()
        opt.step()
        losses.append(float(loss))
    for a, b in zip(losses, ref["losses"]):
        assert abs(a - b) < 0.05, (losses, ref["losses"])
    model.eval()
    gen = model.generate(ids[:, :8], max_new_tokens=8, eos_token_id=None, pad_token_id=0)
    assert gen.shape == (4, 16)
    assert int(ob.ops.load_ext().error_word(ids).item()) == 0


def test_tensor_parallel_fused_training(tmp_path):
    import oslo_b200 as ob
    from oslo_b200.optim import FusedAdamW
    torch.manual_seed(0)
    model = ob.GPTJForCausalLM(_cfg()).to(torch.bfloat16)
    state = {k: v.clone() for k, v in model.state_dict().items()}
    model = model.cuda().fuse().train()
    ids = torch.randint(0, 2048, (4, 128), generator=torch.Generator().manual_seed(1)).cuda()
    opt = FusedAdamW(model.parameters(), lr=1e-3)
    losses = []
    for _ in range(3):
        opt.zero_grad()
        loss = model(input_ids=ids, labels=ids, output_logits=False).loss
        loss.backward()
        opt.step()
        losses.append(float(loss))
    torch.save({"state": state, "losses": losses}, tmp_path / "ref.pt")
    run_gpus(_tp_train, 2, str(tmp_path))


def _symm_allreduce(rank, world):
    import torch.distributed as dist
    from oslo_b200.parallel.mpu import MPU
    from oslo_b200.parallel.symmetric import get_workspace
    import oslo_b200 as ob
    mpu = MPU(world, 1)
    ws = get_workspace(mpu.get_tensor_parallel_group(), 64 * 2 ** 20)
    for n in (8, 4096, 1 << 20, (1 << 22) + 8):
        for mm in ([False, True] if ws.has_multicast else [False]):
            torch.manual_seed(100 + rank)
            x = torch.randn(n, device="cuda").to(torch.bfloat16)
            want = x.clone().float()
            dist.all_reduce(want, group=mpu.get_tensor_parallel_group())
            for _ in range(3):  # back-to-back launches reuse the same signal words
                y = x.clone()
                ws.all_reduce_(y, use_multimem=mm)
            torch.cuda.synchronize()
            assert torch.allclose(y.float(), want, atol=0.05, rtol=0.02), (n, mm, (y.float() - want).abs().max())
    # the one-kernel path keeps its buffer parity on the device: replaying a captured call an odd number of times
    # must stay correct
    x = torch.randn(4096, device="cuda").to(torch.bfloat16)
    want = x.clone().float()
    dist.all_reduce(want, group=mpu.get_tensor_parallel_group())
    y = torch.empty_like(x)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        y.copy_(x)
        ws.all_reduce_(y)
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        y.copy_(x)
        ws.all_reduce_(y)
    for _ in range(5):
        g.replay()
        torch.cuda.synchronize()
        assert torch.allclose(y.float(), want, atol=0.05, rtol=0.02)
    del g
    assert int(ob.ops.load_ext().error_word(x).item()) == 0


def test_symmetric_memory_allreduce():
    run_gpus(_symm_allreduce, 2)


def _zero_dp(rank, world, tmp):
    import torch.distributed as dist
    import oslo_b200 as ob
    from oslo_b200.optim import FusedAdamW
    from oslo_b200.parallel.data_parallel import DistributedDataParallel
    torch.manual_seed(0)
    model = ob.GPTJForCausalLM(_cfg()).to(torch.bfloat16)
    ref = torch.load(os.path.join(tmp, "ref.pt"), weights_only=True)
    model.load_state_dict(ref["state"])
    model = ob.parallelize(model, tensor_parallel_size=1)
    model.fuse().train()
    mpu = model.mpu
    opt = FusedAdamW(model.gpu_parameters(), lr=1e-3, shard_group=mpu.get_data_parallel_group())
    ddp = DistributedDataParallel(model, mpu, optimizer=opt, bucket_mb=1)
    ids = torch.randint(0, 2048, (4, 128), generator=torch.Generator().manual_seed(1)).cuda()
    mine = ids[rank * 2:(rank + 1) * 2]
    losses = []
    for _ in range(3):
        opt.zero_grad()
        loss = ddp(input_ids=mine, labels=mine, output_logits=False).loss
        loss.backward()
        opt.step()
        t = loss.detach().clone()
        dist.all_reduce(t)
        losses.append(float(t) / world)
    for a, b in zip(losses, ref["losses"]):
        assert abs(a - b) < 0.05, (losses, ref["losses"])


def test_zero1_data_parallel(tmp_path):
    import oslo_b200 as ob
    from oslo_b200.optim import FusedAdamW
    torch.manual_seed(0)
    model = ob.GPTJForCausalLM(_cfg()).to(torch.bfloat16)
    state = {k: v.clone() for k, v in model.state_dict().items()}
    model = model.cuda().fuse().train()
    ids = torch.randint(0, 2048, (4, 128), generator=torch.Generator().manual_seed(1)).cuda()
    opt = FusedAdamW(model.parameters(), lr=1e-3)
    losses = []
    for _ in range(3):
        opt.zero_grad()
        loss = model(input_ids=ids, labels=ids, output_logits=False).loss
        loss.backward()
        opt.step()
        losses.append(float(loss))
    torch.save({"state": state, "losses": losses}, tmp_path / "ref.pt")
    run_gpus(_zero_dp, 2, str(tmp_path))


# ---------------------------------------------------------------------------------------------------------------
# pipeline / 3D parallel training on GPUs against a single-GPU run (the counterpart of the reference's
# tests/gpt2/gpt2_test_3d_training_with_ddp.py:87-139, with assertions)

def _make(kind):
    import oslo_b200 as ob
    if kind == "gptj":
        cfg = ob.GPTJConfig(vocab_size=2048, n_positions=256, n_embd=512, n_layer=4, n_head=8, rotary_dim=32,
                            torch_dtype=torch.bfloat16)
        return ob.GPTJForCausalLM(cfg)
    cfg = ob.GPTNeoConfig(vocab_size=2048, max_position_embeddings=256, hidden_size=512, num_layers=4, num_heads=8,
                          window_size=64, torch_dtype=torch.bfloat16)
    return ob.GPTNeoForCausalLM(cfg)


def _ids(step):
    return torch.randint(0, 2048, (8, 128), generator=torch.Generator().manual_seed(100 + step))


def _oracle(kind, tmp_path, steps=3):
    from oslo_b200.optim import FusedAdamW
    torch.manual_seed(0)
    model = _make(kind).to(torch.bfloat16)
    state = {k: v.clone() for k, v in model.state_dict().items()}
    model = model.cuda().fuse().train()
    opt = FusedAdamW(model.parameters(), lr=1e-3, max_grad_norm=1.0)
    losses = []
    for s in range(steps):
        ids = _ids(s).cuda()
        opt.zero_grad()
        loss = model(input_ids=ids, labels=ids, output_logits=False).loss
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    torch.save({"state": state, "losses": losses}, tmp_path / "ref.pt")


def _train_3d(rank, world, tmp, kind, tp, pp, seq_par, steps=3):
    import torch.distributed as dist
    import oslo_b200 as ob
    from oslo_b200.optim import FusedAdamW
    from oslo_b200.parallel.data_parallel import DistributedDataParallel
    ref = torch.load(os.path.join(tmp, "ref.pt"), weights_only=True)
    torch.manual_seed(0)
    model = _make(kind).to(torch.bfloat16)
    model.load_state_dict(ref["state"])
    model = ob.parallelize(model, tensor_parallel_size=tp, pipeline_parallel_size=pp, micro_batch_size=2,
                           sequence_parallel=seq_par)
    model.fuse().train()
    mpu = model.mpu
    dp, dpr = mpu.get_data_parallel_world_size(), mpu.get_data_parallel_rank()
    opt = FusedAdamW(model.gpu_parameters(), lr=1e-3, max_grad_norm=1.0, model=model,
                     shard_group=mpu.get_data_parallel_group() if dp > 1 else None,
                     model_parallel_group=mpu.get_model_parallel_group() if tp * pp > 1 else None)
    call = DistributedDataParallel(model, mpu, optimizer=opt, bucket_mb=1) if dp > 1 else model
    losses = []
    for s in range(steps):
        ids = _ids(s).cuda()
        n = ids.size(0) // dp
        mine = ids[dpr * n:(dpr + 1) * n]
        opt.zero_grad()
        if pp > 1:
            accum = n // 2
            tot = 0.0
            for out in call(input_ids=mine, labels=mine, output_logits=False):
                (out.loss / accum).backward()
                tot = tot + out.loss.detach().float()
            loss = tot / accum
        else:
            loss = call(input_ids=mine, labels=mine, output_logits=False).loss
            loss.backward()
            loss = loss.detach().float()
        opt.step()
        t = loss.reshape(1).clone()
        if dp > 1:
            dist.all_reduce(t, group=mpu.get_data_parallel_group())
            t /= dp
        losses.append(float(t))
    torch.cuda.synchronize()
    # every stage reports the loss of the last stage; compare on every rank
    for a, b in zip(losses, ref["losses"]):
        assert abs(a - b) < 0.08, (rank, losses, ref["losses"])
    assert int(ob.ops.load_ext().error_word(ids).item()) == 0


_LAYOUTS = [  # kind, tp, pp, sequence parallel, GPUs
    ("gptj", 1, 2, False, 2), ("gpt_neo", 1, 2, False, 2), ("gptj", 2, 1, True, 2),
    ("gptj", 2, 2, False, 4), ("gpt_neo", 2, 2, False, 4), ("gptj", 4, 1, False, 4), ("gptj", 1, 4, False, 4),
    ("gptj", 2, 2, True, 4),
    ("gpt_neo", 2, 2, False, 8), ("gptj", 2, 4, False, 8), ("gptj", 8, 1, False, 8), ("gptj", 2, 2, False, 8),
]


@pytest.mark.parametrize("kind,tp,pp,seq_par,world", _LAYOUTS,
                         ids=[f"{k}-tp{t}-pp{p}{'-sp' if sp else ''}-{w}gpus" for k, t, p, sp, w in _LAYOUTS])
def test_model_parallel_training_matches_one_gpu(tmp_path, kind, tp, pp, seq_par, world):
    """Tensor / pipeline / data parallel layouts (ZeRO-1 + bucketed reduction when there are replicas) reproduce the
    loss curve of one GPU over 3 optimizer steps with gradient clipping."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _oracle(kind, tmp_path)
    run_gpus(_train_3d, world, str(tmp_path), kind, tp, pp, seq_par)


def _dp_kernels(rank, world):
    """Bucket reduce-scatter / all-gather kernels on symmetric flat buffers against NCCL, NVSwitch multicast on and
    off, ragged bucket boundaries, repeated calls (the signal words are reused)."""
    import torch.distributed as dist
    import oslo_b200 as ob
    from oslo_b200.config import set_config
    from oslo_b200.parallel.mpu import MPU
    from oslo_b200.parallel.symmetric import SymmetricFlat
    mpu = MPU(1, 1)
    g = mpu.get_data_parallel_group()
    n = 8 * world * 40000 + 8 * world          # not a multiple of the kernels' per-pass span
    flat = SymmetricFlat(g, n, torch.bfloat16, torch.device("cuda", rank))
    assert flat.shard * world == n
    for mm in ([True, False] if flat.mc_ptr else [False]):
        set_config(use_multimem=mm)
        for rep, (lo, hi) in enumerate([(0, n), (8, n - 8), (flat.shard - 64, flat.shard + 4096), (1024, 1032), (0, n)]):
            torch.manual_seed(1000 * rep + rank)
            src = (torch.randn(n, device="cuda") * 2).to(torch.bfloat16)
            flat.tensor.copy_(src)
            want = src.float()
            dist.all_reduce(want, group=g)
            torch.cuda.synchronize()
            dist.barrier()
            flat.reduce_scatter_(lo, hi)
            torch.cuda.synchronize()
            a, b = max(lo, rank * flat.shard), min(hi, (rank + 1) * flat.shard)
            got = flat.tensor.float()
            if b > a:
                assert torch.allclose(got[a:b], want[a:b], atol=0.06, rtol=0.02), ("RS", mm, lo, hi, (got[a:b] - want[a:b]).abs().max())
            keep = torch.ones(n, dtype=torch.bool, device="cuda")
            keep[a:max(a, b)] = False
            assert torch.equal(flat.tensor[keep], src[keep]), ("RS touched elements outside this rank's part", mm, lo, hi)
            # all-gather: after it every rank holds every owner's part of [lo, hi)
            dist.barrier()
            flat.all_gather_(lo, hi)
            torch.cuda.synchronize()
            full = [torch.empty_like(flat.tensor) for _ in range(world)]
            dist.all_gather(full, flat.tensor.clone(), group=g)
            for r in range(1, world):
                assert torch.equal(full[r][lo:hi], full[0][lo:hi]), ("AG", mm, lo, hi, r)
            own = flat.tensor.float()
            assert torch.allclose(own[lo:hi], want[lo:hi], atol=0.06, rtol=0.02), ("AG values", mm, lo, hi)
    assert int(ob.ops.load_ext().error_word(flat.tensor).item()) == 0


def test_dp_symmetric_reduce_scatter_and_all_gather_kernels():
    run_gpus(_dp_kernels, 2)


@pytest.mark.parametrize("world", [4, 8])
def test_dp_symmetric_kernels_world_n(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    run_gpus(_dp_kernels, world)


def _zero_dp_ab(rank, world, tmp):
    """ZeRO-1 data parallelism with the symmetric-memory kernels and with NCCL: same losses, same final weights."""
    import torch.distributed as dist
    import oslo_b200 as ob
    from oslo_b200.config import set_config
    from oslo_b200.optim import FusedAdamW
    from oslo_b200.parallel.data_parallel import DistributedDataParallel
    ref = torch.load(os.path.join(tmp, "ref.pt"), weights_only=True)
    finals = {}
    for symmetric in (True, False):
        set_config(dp_symmetric=symmetric)
        torch.manual_seed(0)
        model = ob.GPTJForCausalLM(_cfg()).to(torch.bfloat16)
        model.load_state_dict(ref["state"])
        model = ob.parallelize(model, tensor_parallel_size=1)
        model.fuse().train()
        mpu = model.mpu
        opt = FusedAdamW(model.gpu_parameters(), lr=1e-3, max_grad_norm=1.0, shard_group=mpu.get_data_parallel_group())
        ddp = DistributedDataParallel(model, mpu, optimizer=opt, bucket_mb=1)
        assert ddp._symm == symmetric and (opt.param_gather is not None) == symmetric
        ids = torch.randint(0, 2048, (4, 128), generator=torch.Generator().manual_seed(1)).cuda()
        mine = ids[rank * 2:(rank + 1) * 2]
        losses = []
        for _ in range(4):
            opt.zero_grad()
            for i in range(2):                    # two micro-batches: reduction during the second backward only
                import contextlib
                with (ddp.no_sync() if i == 0 else contextlib.nullcontext()):
                    loss = ddp(input_ids=mine[i:i + 1], labels=mine[i:i + 1], output_logits=False).loss
                    (loss / 2).backward()
            opt.step()
            losses.append(float(loss.detach()))
        finals[symmetric] = (losses, {k: v.detach().float().clone() for k, v in model.state_dict().items()})
        # every replica ends with the same parameters
        flat = opt.buf.flat_p.float()
        other = flat.clone()
        dist.all_reduce(other, op=dist.ReduceOp.MAX)
        assert torch.equal(flat, other), "replicas diverged"
    for a, b in zip(finals[True][0], finals[False][0]):
        assert abs(a - b) < 0.03, finals
    for k, v in finals[True][1].items():
        assert torch.allclose(v, finals[False][1][k], atol=3e-2, rtol=3e-2), k
    assert int(ob.ops.load_ext().error_word(ids).item()) == 0


def test_zero1_symmetric_kernels_match_nccl(tmp_path):
    import oslo_b200 as ob
    torch.manual_seed(0)
    model = ob.GPTJForCausalLM(_cfg()).to(torch.bfloat16)
    torch.save({"state": {k: v.clone() for k, v in model.state_dict().items()}}, tmp_path / "ref.pt")
    run_gpus(_zero_dp_ab, 2, str(tmp_path))


def test_deployment_launcher_on_gpus():
    """The deployment launcher with GPU workers (the flow of the reference's tests/utils/test_deployment.py:6-35, with
    assertions): this process spawns two tensor-parallel workers, beam search through them matches one GPU in fp32;
    the fused bf16 model decodes greedily through the CUDA-graph path and agrees with one GPU on nearly every token."""
    import oslo_b200 as ob
    from oslo_b200.parallelism_utils import set_seed
    cfg = ob.GPTJConfig(vocab_size=2048, n_positions=128, n_embd=256, n_layer=2, n_head=4, rotary_dim=16)
    ids = torch.randint(0, 2048, (2, 12), generator=torch.Generator().manual_seed(3))
    set_seed(41)
    with torch.device("cuda", 0):                      # as the workers do: weights drawn by the device generator
        one = ob.GPTJForCausalLM._from_config(cfg, torch_dtype=None).eval()
    want = one.generate(ids.cuda(), max_length=24, num_beams=3, no_repeat_ngram_size=3, eos_token_id=None, pad_token_id=0).cpu()
    model = ob.GPTJForCausalLM.from_config_with_parallel(cfg, tensor_parallel_size=2, seed=41, deployment=True,
                                                         init_on_device=True)
    try:
        got = model.generate(ids, max_length=24, num_beams=3, no_repeat_ngram_size=3, eos_token_id=None, pad_token_id=0)
        assert got.shape == want.shape and (got == want).float().mean() > 0.9, (got, want)
    finally:
        model.cpu()
    del one
    cfg16 = ob.GPTJConfig(vocab_size=2048, n_positions=128, n_embd=256, n_layer=2, n_head=4, rotary_dim=16,
                          torch_dtype=torch.bfloat16)
    set_seed(41)
    with torch.device("cuda", 0):
        one = ob.GPTJForCausalLM._from_config(cfg16, torch_dtype=torch.bfloat16).eval().fuse()
    with torch.no_grad():
        want_logits = one(input_ids=ids.cuda()).logits.float().cpu()
    model = ob.GPTJForCausalLM.from_config_with_parallel(cfg16, tensor_parallel_size=2, seed=41, deployment=True,
                                                         init_on_device=True, torch_dtype=torch.bfloat16).fuse()
    try:
        # tokens of a random-init model sit on near-ties that bf16 rounding may flip, so the comparison with one GPU
        # is made on the logits; the decode loop is checked for what must hold exactly
        logits = model(input_ids=ids).logits.float()
        assert logits.shape == want_logits.shape
        assert (logits - want_logits).abs().max() <= 0.05 * want_logits.abs().max() + 1e-3
        outs = [model.generate(ids, max_new_tokens=16, eos_token_id=None, pad_token_id=0, cuda_graph=True)
                for _ in range(2)]                   # the second call replays the captured step
        assert outs[0].shape == (2, 28) and torch.equal(outs[0][:, :12], ids)
        assert torch.equal(outs[0], outs[1])
        assert int(outs[0].min()) >= 0 and int(outs[0].max()) < 2048
    finally:
        model.cpu()
