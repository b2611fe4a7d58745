"""Rank layout and partition helpers (pure functions; no process group needed)."""
import torch

from oslo_b200.parallel.engine_pipeline import one_f_one_b_order
from oslo_b200.parallel.mpu import MPU, ceil_split_sizes


def test_sixteen_rank_example():
    # the 16-rank, tp=2, pp=4 example documented in the reference (oslo/parallelism/mpu.py:29-38)
    assert MPU.layout_pipeline_groups(16, 4) == [[0, 4, 8, 12], [1, 5, 9, 13], [2, 6, 10, 14], [3, 7, 11, 15]]
    assert MPU.layout_tensor_groups(16, 2) == [[i, i + 1] for i in range(0, 16, 2)]
    assert MPU.layout_data_groups(16, 2, 4) == [[0, 2], [1, 3], [4, 6], [5, 7], [8, 10], [9, 11], [12, 14], [13, 15]]
    assert MPU.layout_model_groups(16, 2, 4) == [[0, 1, 4, 5, 8, 9, 12, 13], [2, 3, 6, 7, 10, 11, 14, 15]]


def test_vocab_split_sizes():
    assert ceil_split_sizes(50257, 4) == [12565, 12565, 12565, 12562]
    assert ceil_split_sizes(50257, 2) == [25129, 25128]
    assert ceil_split_sizes(50400, 8) == [6300] * 8


def test_pipeline_partition():
    assert MPU.make_pipeline_partition(28, 4) == [0, 7, 14, 21, 28]
    assert MPU.make_pipeline_partition(10, 4) == [0, 2, 4, 6, 10]  # remainder goes to the last stage
    assert MPU.extend_pipeline_partition([0, 2, 5]) == [0, 0, 1, 1, 1]


def test_one_f_one_b_order():
    assert one_f_one_b_order(2, 0, 3) == ["F0", "F1", "B0", "F2", "B1", "B2"]
    assert one_f_one_b_order(2, 1, 3) == ["F0", "B0", "F1", "B1", "F2", "B2"]
    # every stage runs each forward before its backward and holds at most P - stage activations
    for P in (2, 4):
        for s in range(P):
            order = one_f_one_b_order(P, s, 8)
            live = peak = 0
            for a in order:
                live += 1 if a[0] == "F" else -1
                peak = max(peak, live)
                assert live >= 0
            assert peak <= P - s


def _p2p_ranks(rank, world):
    import torch
    import oslo_b200 as ob

    # before any pipeline engine exists: the transfer runs over the pipeline group, no per-pair groups yet
    mpu = MPU(1, world)
    assert mpu.get_p2p_communication_groups() == {}
    t = torch.full((3,), float(rank))
    took_part = mpu.p2p(t, 1, 2)
    assert took_part == (rank in (1, 2))
    assert t.tolist() == [1.0] * 3 if rank == 2 else t.tolist() == [float(rank)] * 3
    t = torch.full((3,), float(rank))
    assert mpu.p2p(t, 1, 0) == (rank in (0, 1))          # towards the first stage
    assert t[0].item() == (1.0 if rank == 0 else float(rank))
    for bad in ((0, 2), (0, 0), (-1, 0), (world - 1, world)):
        try:
            mpu.p2p(t, *bad)
        except ValueError:
            continue
        raise AssertionError(f"stages {bad} were accepted")

    # with a pipeline-parallel model: the engine's channels, keyed by (source rank, destination rank)
    cfg = ob.GPTJConfig(vocab_size=64, n_positions=16, n_embd=16, n_layer=4, n_head=2, rotary_dim=4)
    model = ob.parallelize(ob.GPTJForCausalLM(cfg), pipeline_parallel_size=world, micro_batch_size=1)
    groups = model.mpu.get_p2p_communication_groups()
    want = {(a, b) for a in range(world) for b in range(world) if abs(a - b) == 1 and rank in (a, b)}
    assert set(groups) == want
    t = torch.full((2,), float(rank))
    assert model.mpu.p2p(t, 2, 3) == (rank in (2, 3))
    assert t[0].item() == (2.0 if rank == 3 else float(rank))


def test_p2p_between_neighbouring_stages():
    """``mpu.p2p(tensor, src_stage, dst_stage)`` and ``get_p2p_communication_groups()`` of the reference's MPU
    (oslo/parallelism/mpu.py:321-368, :892-920) on 4 pipeline stages."""
    from tests.dist_utils import run_distributed
    run_distributed(_p2p_ranks, 4)


def _object_ranks(rank, world):
    import torch
    import oslo_b200 as ob
    from oslo_b200.modeling_utils import ModelOutput
    cfg = ob.GPTJConfig(vocab_size=64, n_positions=16, n_embd=16, n_layer=3, n_head=2, rotary_dim=4)
    model = ob.parallelize(ob.GPTJForCausalLM(cfg), pipeline_parallel_size=world, micro_batch_size=1)
    comm = model._pipe_engine.p2p
    value = None
    if rank == 0:
        value = {"flag": True, "n": 7, "x": 2.5, "z": 1 + 2j, "s": "héllo", "none": None, "kind": float,
                 "shape": torch.Size([2, 3]), "set": {1, 2}, "tup": (1, ("a", torch.arange(4))),
                 "list": [torch.ones(2, 2, dtype=torch.bfloat16), torch.zeros(0)],
                 "out": ModelOutput(loss=torch.tensor(0.5, requires_grad=True), logits=None)}
    got = comm.ring_exchange_forward(value)
    assert got["flag"] is True and got["n"] == 7 and got["x"] == 2.5 and got["z"] == 1 + 2j and got["s"] == "héllo"
    assert got["none"] is None and got["kind"] is float and got["shape"] == torch.Size([2, 3]) and got["set"] == {1, 2}
    assert isinstance(got["shape"], torch.Size) and isinstance(got["tup"], tuple)
    assert got["tup"][1][0] == "a" and got["tup"][1][1].tolist() == [0, 1, 2, 3]
    assert got["list"][0].dtype == torch.bfloat16 and got["list"][0].shape == (2, 2) and got["list"][1].numel() == 0
    assert isinstance(got["out"], ModelOutput) and got["out"].loss.requires_grad and float(got["out"].loss) == 0.5
    # the other way round, a bare tensor and scalars through the typed calls
    back = comm.ring_exchange_backward(torch.full((3,), float(rank)) if rank == world - 1 else None)
    assert back.tolist() == [float(world - 1)] * 3
    if rank == 0:
        comm.send_int(41, 1)
        comm.send_str("x", recv_stage=1, send_type=True)
        comm.send((1, 2), 1)
        try:
            comm.send_int(True, 1)
        except TypeError:
            pass
        else:
            raise AssertionError("a bool went through send_int")
    elif rank == 1:
        assert comm.recv_int(0) == 41 and comm.recv_str(0) == "x" and comm.recv(0) == (1, 2)
    try:
        comm.send_object(1, rank + 2)
    except ValueError:
        pass
    else:
        raise AssertionError("a non-neighbour was accepted")


def test_values_of_any_kind_travel_between_stages():
    """The object protocol of the reference's ``P2PCommunicator`` (oslo/parallelism/engine_pipeline.py:795-1199):
    nested containers, scalars, ``None``, types, sizes and tensors from the first stage reach every stage."""
    from tests.dist_utils import run_distributed
    run_distributed(_object_ranks, 3)


def _node_ranks(rank, world):
    import os
    import torch.distributed as dist
    from oslo_b200.parallel import symmetric
    # ranks 0-1 on host "a", ranks 2-3 on host "b": tensor-parallel pairs stay on one host, data-parallel pairs do not
    os.environ["OSLO_B200_NODE_ID"] = "a" if rank < 2 else "b"
    mpu = MPU(2, 1)
    assert mpu.node_of_rank == ["a", "a", "b", "b"]
    assert symmetric.group_on_one_node(mpu.get_tensor_parallel_group()) is True
    assert symmetric.group_on_one_node(mpu.get_data_parallel_group()) is False
    assert symmetric.symmetric_flat_usable(mpu.get_data_parallel_group(), torch.bfloat16, "cpu") is False
    # a group the MPU did not create: asked collectively on first use, then cached
    g = dist.new_group(ranks=[0, 1, 2, 3], backend="gloo")
    assert symmetric.group_on_one_node(g) is False and symmetric._ONE_NODE[g.group_name] is False
    pair = dist.new_group(ranks=[2, 3], backend="gloo")
    if rank >= 2:
        assert symmetric.group_on_one_node(pair) is True


def test_symmetric_memory_paths_ask_whether_a_group_sits_on_one_host():
    from tests.dist_utils import run_distributed
    run_distributed(_node_ranks, 4)
