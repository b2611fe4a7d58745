"""Property tests (hypothesis) of the pure planning functions: rank layout, splits, sharding, the 1F1B schedule."""
import torch
from hypothesis import given, settings, strategies as st

from oslo_b200.parallel.engine_pipeline import one_f_one_b_order
from oslo_b200.parallel.engine_tensor import shard_tensor, unshard_tensors
from oslo_b200.parallel.mpu import MPU, ceil_split_sizes


@st.composite
def grids(draw):
    tp = draw(st.sampled_from([1, 2, 3, 4, 8]))
    pp = draw(st.sampled_from([1, 2, 3, 4]))
    dp = draw(st.integers(1, 4))
    return tp, pp, dp


@given(grids())
@settings(max_examples=60, deadline=None)
def test_every_rank_is_in_exactly_one_group_of_each_kind(g):
    tp, pp, dp = g
    world = tp * pp * dp
    for groups, size in ((MPU.layout_tensor_groups(world, tp), tp), (MPU.layout_pipeline_groups(world, pp), pp),
                         (MPU.layout_data_groups(world, tp, pp), dp), (MPU.layout_model_groups(world, tp, pp), tp * pp)):
        flat = [r for grp in groups for r in grp]
        assert sorted(flat) == list(range(world))
        assert all(len(grp) == size for grp in groups)
    # a tensor group and a data group share at most one rank; same for pipeline vs data
    for t in MPU.layout_tensor_groups(world, tp):
        for d in MPU.layout_data_groups(world, tp, pp):
            assert len(set(t) & set(d)) <= 1
    for p in MPU.layout_pipeline_groups(world, pp):
        for d in MPU.layout_data_groups(world, tp, pp):
            assert len(set(p) & set(d)) <= 1


@given(st.integers(1, 100000), st.integers(1, 16))
@settings(max_examples=200, deadline=None)
def test_ceil_split_matches_torch_chunk(total, parts):
    sizes = ceil_split_sizes(total, parts)
    want = [c.numel() for c in torch.chunk(torch.empty(total), parts)]
    assert [s for s in sizes if s] == want and sum(sizes) == total and len(sizes) == parts


@given(st.integers(1, 4), st.sampled_from([1, 2, 3]), st.integers(1, 5), st.integers(1, 4), st.sampled_from([0, 1]))
@settings(max_examples=80, deadline=None)
def test_shard_round_trip(tp, n_fused, per, other, dim):
    size = tp * n_fused * per
    shape = [other, other]
    shape[dim] = size
    t = torch.arange(shape[0] * shape[1], dtype=torch.float32).view(shape)
    shards = [shard_tensor(t, tp, r, dim, n_fused) for r in range(tp)]
    assert torch.equal(unshard_tensors(shards, dim, n_fused), t)
    if n_fused > 1:   # rank r holds its slice of every fused piece, in piece order
        pieces = torch.chunk(t, n_fused, dim=dim)
        for r in range(tp):
            want = torch.cat([torch.chunk(p, tp, dim=dim)[r] for p in pieces], dim=dim)
            assert torch.equal(shards[r], want)


@given(st.integers(1, 6), st.integers(1, 12))
@settings(max_examples=80, deadline=None)
def test_one_f_one_b_schedule_is_complete_bounded_and_deadlock_free(stages, micro):
    orders = [one_f_one_b_order(stages, s, micro) for s in range(stages)]
    for s, order in enumerate(orders):
        assert sorted(order) == sorted([f"F{i}" for i in range(micro)] + [f"B{i}" for i in range(micro)])
        live = peak = 0
        for a in order:
            assert a[0] == "F" or f"F{a[1:]}" in order[:order.index(a)]
            live += 1 if a[0] == "F" else -1
            peak = max(peak, live)
        assert peak <= min(stages - s, micro)            # activations held at once: the 1F1B memory bound
    # run all stages against the message dependencies: F_i needs F_i of the previous stage, B_i needs B_i of the next
    done = [set() for _ in range(stages)]
    pos = [0] * stages
    progressed = True
    while progressed:
        progressed = False
        for s in range(stages):
            if pos[s] == len(orders[s]):
                continue
            a = orders[s][pos[s]]
            ready = ((a[0] == "F" and (s == 0 or a in done[s - 1]))
                     or (a[0] == "B" and (s == stages - 1 or a in done[s + 1])))
            if ready:
                done[s].add(a)
                pos[s] += 1
                progressed = True
    assert all(pos[s] == len(orders[s]) for s in range(stages)), "the schedule dead-locks"


def test_cross_entropy_route_is_the_same_on_every_tensor_parallel_rank():
    """The choice between the symmetric-memory combine and the NCCL all-reduces of the vocabulary-parallel loss is made
    from the sizes of ALL shards: an uneven split (50257 over 2 ranks gives 25129 and 25128 rows, only one of them a
    multiple of 8) must not send the two ranks down different collectives."""
    from oslo_b200.parallel.mpu import ceil_split_sizes
    from oslo_b200.parallel.vocab_parallel import shard_rows_aligned
    assert ceil_split_sizes(50257, 2) == [25129, 25128]
    assert not shard_rows_aligned(50257, 2) and not shard_rows_aligned(50400, 8)
    assert shard_rows_aligned(50400, 2) and shard_rows_aligned(50400, 4) and shard_rows_aligned(50400, 1)
    for vocab in (50257, 50400, 2048, 1003):
        for tp in (1, 2, 4, 8):
            answers = {shard_rows_aligned(vocab, tp) for _rank in range(tp)}      # no rank-dependent input exists
            assert len(answers) == 1
