"""Host-side models of the cross-GPU protocols, run as threads with adversarial delays.

The kernels cannot be raced on purpose on a shared GPU, so the ordering arguments their comments make are checked
here on a model: ranks are threads, symmetric memory is a shared list, the per-block cross-rank barrier is a
``threading.Barrier``. A rank that reads a value that does not belong to the current call fails the test.
"""
import random
import threading
import time

import pytest


def _run(world, calls, halves, trailing_barrier, delays):
    """One-shot all-reduce protocol of ``allreduce_oneshot_kernel``: write own slot of half ``parity``, ONE barrier,
    read every rank's slot. Returns the list of (rank, call, seen) violations."""
    stage = [[None] * world for _ in range(halves)]
    barrier = threading.Barrier(world)
    bad = []

    def rank_fn(r):
        rnd = random.Random(1000 + r)
        counter = 0                                   # the device-side per-block counter
        for call in range(calls):
            h = counter % halves
            time.sleep(delays(r, call, "before_write", rnd))
            stage[h][r] = call
            barrier.wait()
            time.sleep(delays(r, call, "before_read", rnd))
            seen = list(stage[h])
            if any(v != call for v in seen):
                bad.append((r, call, seen))
            if trailing_barrier:
                barrier.wait()
            counter += 1

    threads = [threading.Thread(target=rank_fn, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(60)
    return bad


def _jitter(r, call, where, rnd):
    return rnd.random() * 0.002


def _slow_reader(r, call, where, rnd):
    # rank 0 dawdles before reading, everybody else races ahead into the next call
    return 0.02 if (r == 0 and where == "before_read") else 0.0


@pytest.mark.parametrize("world", [2, 4, 8])
def test_two_alternating_halves_need_no_trailing_barrier(world):
    assert _run(world, calls=40, halves=2, trailing_barrier=False, delays=_jitter) == []
    assert _run(world, calls=12, halves=2, trailing_barrier=False, delays=_slow_reader) == []


def test_single_buffer_without_trailing_barrier_is_caught_by_the_model():
    """Negative control: with one staging buffer a fast rank overwrites what a slow rank has not read yet."""
    bad = _run(4, calls=6, halves=1, trailing_barrier=False, delays=_slow_reader)
    assert bad, "the model failed to expose the overwrite-before-read hazard"
    assert _run(4, calls=6, halves=1, trailing_barrier=True, delays=_slow_reader) == []


def test_generation_tagged_words_survive_reuse_with_other_shapes():
    """Readiness words of the fused GEMM + collective kernels are WRITTEN with the call's generation and waited for
    with >=; stale words of earlier calls (any shape, any mode) are smaller, so a slot never needs a reset."""
    words = [0] * 64
    gen = 0
    rnd = random.Random(7)
    for call in range(50):
        gen += 1
        n = rnd.choice([4, 16, 64])                    # this call uses the first n words of the slot
        order = list(range(n))
        rnd.shuffle(order)
        ready = lambda i: words[i] - gen >= 0          # noqa: E731 - the kernel's signed-distance test
        assert not any(ready(i) for i in range(n)), "a stale word satisfied a wait of a later generation"
        for i in order:
            words[i] = gen
        assert all(ready(i) for i in range(n))


def _run_vocab_embed(world, token_counts, max_blocks, fixed_grid, delays):
    """Model of ``vocab_embed_kernel``: the owner of a token (``t % world`` here) writes the token's row into EVERY
    rank's staging half, the ranks meet once, every rank copies its rows out. Each block keeps its own half parity;
    ``fixed_grid`` says whether the launcher always starts ``max_blocks`` blocks (the real launcher) or only as many
    as there are tokens (the defect this model documents). Returns the violations."""
    tmax = max(token_counts)
    stage = [[[None] * tmax for _ in range(2)] for _ in range(world)]     # [rank][half][token offset]
    barrier = threading.Barrier(world)
    bad = []

    def rank_fn(r):
        rnd = random.Random(2000 + r)
        counters = [0] * max_blocks
        for call, tokens in enumerate(token_counts):
            grid = max_blocks if fixed_grid else min(tokens, max_blocks)
            per = -(-tokens // grid)
            blocks = [(b, range(b * per, min(tokens, (b + 1) * per))) for b in range(grid)]
            time.sleep(delays(r, call, "before_write", rnd))
            for b, toks in blocks:
                h = counters[b] & 1
                for t in toks:
                    if t % world == r:
                        for peer in range(world):
                            stage[peer][h][t] = (call, t)
            barrier.wait()                                  # stands for the per-block cross-rank barriers
            time.sleep(delays(r, call, "before_read", rnd))
            for b, toks in blocks:
                h = counters[b] & 1
                for t in toks:
                    if stage[r][h][t] != (call, t):
                        bad.append((r, call, t, stage[r][h][t]))
                counters[b] += 1

    threads = [threading.Thread(target=rank_fn, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(60)
    return bad


def test_vocab_embed_halves_stay_in_lockstep_for_any_token_counts():
    """Prefill, a run of decode steps (1 token: fewer tokens than blocks), then two larger calls of different sizes:
    with the fixed grid no rank ever reads a row of another call; with a grid that follows the token count the
    per-block parities drift apart and a fast owner overwrites rows that a slow rank has not copied out yet."""
    counts = [64, 1, 1, 1, 48, 24, 64, 3, 40, 20]
    for world in (2, 4):
        assert _run_vocab_embed(world, counts, 8, True, _slow_reader) == []
        assert _run_vocab_embed(world, counts * 2, 8, True, _jitter) == []
    assert _run_vocab_embed(2, counts, 8, False, _slow_reader), "the model failed to expose the drifting parities"
