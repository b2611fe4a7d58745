"""GEMM + collective kernels. World size 1 exercises the whole flag / epoch protocol on one GPU; the
2-GPU cases compare every fused op (peer loads and NVSwitch multimem) with the unfused statement."""
import os

import pytest
import torch

from tests.test_multigpu import run_gpus

pytestmark = pytest.mark.gpu


def _check_ops(rank, world):
    import torch.distributed as dist
    import oslo_b200 as ob
    from oslo_b200.config import set_config
    from oslo_b200.parallel.fused_tp import FusedTP
    from oslo_b200.parallel.mpu import MPU
    mpu = MPU(world, 1)
    g = mpu.get_tensor_parallel_group()
    ext = ob.ops.load_ext(required=True)
    modes = [False, True]
    for use_mm in modes:
        set_config(use_multimem=use_mm)
        tp = FusedTP(g, workspace_mb=64)
        if use_mm and not tp.use_multimem:
            continue
        for (M, N, K) in [(256 * world, 512, 256), (1024 * world, 4096, 1024), (128 * world, 264, 64)]:
            for rep in range(3):  # repeated calls walk both workspace slots and grow the epochs
                torch.manual_seed(10 * rank + rep)
                a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
                b = (torch.randn(N, K, device="cuda") * 0.1).to(torch.bfloat16)
                want = a.float() @ b.float().t()
                dist.all_reduce(want, group=g)
                got = tp.gemm_all_reduce(a, b, False, False)
                assert torch.allclose(got.float(), want, atol=0.25, rtol=0.03), ("AR", use_mm, M, N, K, rep, (got.float() - want).abs().max())
                # a second per-rank partial sum joins the tiles before the reduction (two row-parallel products,
                # one collective)
                part = (torch.randn(M, N, device="cuda") * 0.5).to(torch.bfloat16)
                want_p = a.float() @ b.float().t() + part.float()
                dist.all_reduce(want_p, group=g)
                got_p = tp.gemm_all_reduce(a, b, False, False, partial=part)
                assert torch.allclose(got_p.float(), want_p, atol=0.3, rtol=0.03), ("AR+partial", use_mm, M, N, K, rep)
                got_rs = tp.gemm_reduce_scatter(a, b.t().contiguous(), False, True)
                rows = M // world
                assert torch.allclose(got_rs.float(), want[rank * rows:(rank + 1) * rows], atol=0.25, rtol=0.03), ("RS", use_mm, M, N, K)
                # all-gather of the A shards, then the product with a replicated B (+ bias, GeLU)
                shard = torch.randn(rows, K, device="cuda").to(torch.bfloat16)
                parts = [torch.empty_like(shard) for _ in range(world)]
                dist.all_gather(parts, shard, group=g)
                full = torch.cat(parts)
                torch.manual_seed(99 + rep)
                w = (torch.randn(N, K, device="cuda") * 0.1).to(torch.bfloat16)
                bias = torch.randn(N, device="cuda").to(torch.bfloat16)
                out, gathered = tp.all_gather_gemm(shard, w, False, bias, gelu=True)
                assert torch.equal(gathered, full), ("AG operand", use_mm)
                ref = ob.ops.reference.gelu_tanh(full.float() @ w.float().t() + bias.float())
                assert torch.allclose(out.float(), ref, atol=0.1, rtol=0.03), ("AG", use_mm, M, N, K, (out.float() - ref).abs().max())
        torch.cuda.synchronize()
        assert int(ext.error_word(a).item()) == 0


def _check_vocab_embed(rank, world):
    """Fused vocab-parallel embedding (owner pushes rows, one barrier) against a lookup in the whole table."""
    import torch.distributed as dist
    import oslo_b200 as ob
    from oslo_b200.parallel.mpu import MPU
    from oslo_b200.parallel.layers import VocabParallelEmbedding
    from oslo_b200.parallel.mpu import ceil_split_sizes
    from oslo_b200.config import set_config
    set_config(fused_vocab_embed=True)
    mpu = MPU(world, 1)
    torch.manual_seed(0)
    vocab, hidden = 1003, 256
    full = (torch.randn(vocab, hidden, device="cuda") * 0.5).to(torch.bfloat16)
    sizes = ceil_split_sizes(vocab, world)
    lo = sum(sizes[:rank])
    emb = VocabParallelEmbedding(sizes[rank], hidden).to(torch.bfloat16).cuda()
    emb.weight.data.copy_(full[lo: lo + sizes[rank]])
    emb.mpu, emb.full_num_embeddings, emb.oslo_fused = mpu, vocab, True
    for step in range(3):   # consecutive calls alternate the staging halves
        ids = torch.randint(0, vocab, (4, 37 + step), generator=torch.Generator().manual_seed(step)).cuda()
        out = emb(ids)
        assert torch.equal(out, full[ids]), (step, (out.float() - full[ids].float()).abs().max())
    g = torch.randn_like(out)
    out.backward(g)
    ref = full.clone().float().requires_grad_(True)
    torch.nn.functional.embedding(ids, ref).backward(g.float())
    want = ref.grad[lo: lo + sizes[rank]]
    assert torch.allclose(emb.weight.grad.float(), want, atol=2e-2, rtol=2e-2)
    assert int(ob.ops.load_ext().error_word(out).item()) == 0


@pytest.mark.multigpu
def test_fused_vocab_embedding_world2():
    run_gpus(_check_vocab_embed, 2)


def test_fused_ops_world1():
    run_gpus(_check_ops, 1)


@pytest.mark.multigpu
def test_fused_ops_world2():
    run_gpus(_check_ops, 2)


@pytest.mark.multigpu
@pytest.mark.parametrize("world", [4, 8])
def test_fused_ops_world_n(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    run_gpus(_check_ops, world)


def _tp_model(rank, world, tmp, seq_par):
    import oslo_b200 as ob
    from oslo_b200.config import set_config
    from oslo_b200.optim import FusedAdamW
    ref = torch.load(os.path.join(tmp, "ref.pt"), weights_only=True)
    cfg = ob.GPTJConfig(vocab_size=2048, n_positions=256, n_embd=512, n_layer=2, n_head=4, rotary_dim=32,
                        torch_dtype=torch.bfloat16)
    ids = torch.randint(0, 2048, (4, 128), generator=torch.Generator().manual_seed(1)).cuda()
    results = {}
    for fused_comm in (False, True):
        set_config(fused_tp_comm=fused_comm)
        torch.manual_seed(0)
        model = ob.GPTJForCausalLM(cfg).to(torch.bfloat16)
        model.load_state_dict(ref["state"])
        model = ob.parallelize(model, tensor_parallel_size=world, sequence_parallel=seq_par)
        model.fuse().train()
        opt = FusedAdamW(model.gpu_parameters(), lr=1e-3)
        losses = []
        for _ in range(3):
            opt.zero_grad()
            loss = model(input_ids=ids, labels=ids, output_logits=False).loss
            loss.backward()
            opt.step()
            losses.append(float(loss.detach()))
        results[fused_comm] = losses
        for a, b in zip(losses, ref["losses"]):
            assert abs(a - b) < 0.06, (fused_comm, losses, ref["losses"])
    assert int(ob.ops.load_ext().error_word(ids).item()) == 0


@pytest.mark.multigpu
@pytest.mark.parametrize("seq_par", [False])
def test_tp_training_with_fused_collectives(tmp_path, seq_par):
    import oslo_b200 as ob
    torch.manual_seed(0)
    cfg = ob.GPTJConfig(vocab_size=2048, n_positions=256, n_embd=512, n_layer=2, n_head=4, rotary_dim=32,
                        torch_dtype=torch.bfloat16)
    model = ob.GPTJForCausalLM(cfg).to(torch.bfloat16)
    state = {k: v.clone() for k, v in model.state_dict().items()}
    model = model.cuda().train()  # eager (library) single-GPU oracle
    ids = torch.randint(0, 2048, (4, 128), generator=torch.Generator().manual_seed(1)).cuda()
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3, weight_decay=0.01)
    losses = []
    for _ in range(3):
        opt.zero_grad()
        loss = model(input_ids=ids, labels=ids).loss
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    torch.save({"state": state, "losses": losses}, tmp_path / "ref.pt")
    run_gpus(_tp_model, 2, str(tmp_path), seq_par)
