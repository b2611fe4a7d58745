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


def test_balanced_pipeline_partition():
    from oslo_b200.parallel.engine_pipeline import balanced_partition
    assert balanced_partition(28, 4) == [7, 7, 8, 6]          # GPT-J-6B: the head stage gives a block away
    assert balanced_partition(28, 1) == [28] and balanced_partition(4, 4) == [1, 1, 1, 1]
    for L in (2, 3, 5, 8, 12, 16, 24, 28, 32, 40, 48):
        for P in range(1, min(L, 8) + 1):
            parts = balanced_partition(L, P)
            assert len(parts) == P and sum(parts) == L and min(parts) >= 1
            even = [L // P] * (P - 1) + [L - (L // P) * (P - 1)]
            load = lambda ps: max(n + (0.15 if i == 0 else 0) + (1.5 if i == len(ps) - 1 else 0) for i, n in enumerate(ps))  # noqa: E731
            assert load(parts) <= load(even) + 1e-9
    import pytest
    with pytest.raises(ValueError):
        balanced_partition(3, 4)


def test_bf16_gradient_accumulation_over_16_micro_batches():
    """Weight gradients of the micro-batches of a step are added into a bf16 buffer (the GEMM epilogue reads the
    running sum, adds the new product in fp32 and rounds once). Against fp32 accumulation of the same 16 micro-batch
    gradients the relative error of the sum stays at the level of ONE bf16 rounding of the result (2^-9 = 0.2 %),
    far below the noise between micro-batches, and the direction of the step is unchanged."""
    import torch
    torch.manual_seed(0)
    n, m = 1 << 16, 16
    common = torch.randn(n) * 0.02                        # the part of the gradient all micro-batches agree on
    grads = [(common + torch.randn(n) * 0.05) / m for _ in range(m)]     # per-micro-batch noise larger than the signal
    exact = torch.zeros(n, dtype=torch.float64)
    acc16 = torch.zeros(n, dtype=torch.bfloat16)
    for g in grads:
        g16 = g.to(torch.bfloat16)                        # what a 16-bit product would hand over
        exact += g16.double()
        acc16 = (acc16.float() + g16.float()).to(torch.bfloat16)        # fp32 add, one rounding: the epilogue's rule
    err = (acc16.double() - exact).norm() / exact.norm()
    one_rounding = (exact.float().to(torch.bfloat16).double() - exact).norm() / exact.norm()
    cos = torch.nn.functional.cosine_similarity(acc16.double(), exact, dim=0)
    assert one_rounding < 0.003
    assert err < 4 * one_rounding and err < 0.01, (float(err), float(one_rounding))
    assert cos > 0.9999


_leaves = st.one_of(st.none(), st.booleans(), st.integers(-10 ** 12, 10 ** 12), st.floats(allow_nan=False),
                    st.complex_numbers(allow_nan=False, allow_infinity=False), st.text(max_size=8),
                    st.sampled_from([int, float, str, dict]),
                    st.lists(st.integers(0, 5), max_size=3).map(torch.Size),
                    st.lists(st.integers(1, 3), min_size=0, max_size=3).map(
                        lambda shape: torch.arange(int(torch.tensor(shape or [1]).prod())).reshape(shape or [1]).float()))
_values = st.recursive(_leaves, lambda inner: st.one_of(
    st.lists(inner, max_size=3), st.lists(inner, max_size=3).map(tuple),
    st.dictionaries(st.text(max_size=4), inner, max_size=3)), max_leaves=12)


def _same(a, b) -> bool:
    if torch.is_tensor(a) or torch.is_tensor(b):
        return torch.is_tensor(a) and torch.is_tensor(b) and a.dtype == b.dtype and a.shape == b.shape and torch.equal(a, b)
    if type(a) is not type(b):
        return False
    if isinstance(a, dict):
        return a.keys() == b.keys() and all(_same(a[k], b[k]) for k in a)
    if isinstance(a, (list, tuple)) and not isinstance(a, torch.Size):
        return len(a) == len(b) and all(_same(x, y) for x, y in zip(a, b))
    return a == b


@given(_values)
@settings(max_examples=150, deadline=None)
def test_pipeline_message_structure_round_trips(value):
    """What ``P2PCommunicator.send_object`` puts on the wire (pickled structure with tensor slots + the tensors) turns
    back into the same value on the other side, for any nesting of the kinds the reference's communicator names."""
    import pickle
    from oslo_b200.parallel.engine_pipeline import _collect_slots, _fill_slots, _strip_tensors
    tensors = []
    wire = pickle.dumps(_strip_tensors(value, tensors))
    skeleton = pickle.loads(wire)
    slots = []
    _collect_slots(skeleton, slots)
    assert sorted(s.index for s in slots) == list(range(len(tensors)))
    for s in slots:
        assert s.shape == tuple(tensors[s.index].shape) and s.dtype == tensors[s.index].dtype
    back = _fill_slots(skeleton, {i: t.clone() for i, t in enumerate(tensors)})
    assert _same(back, value)
