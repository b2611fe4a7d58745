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


def _run_fused_grid(world, grid, tiles, resident, aligned, all_ctas_wait_for_done):
    """Discrete model of the GEMM + all-reduce kernel's dependencies. Every rank launches ``grid`` CTAs but only
    ``resident`` of them fit on the device at once (the rest start when a resident one exits - what happens when
    another kernel holds some SMs). CTA c PRODUCES tiles c, c + grid, ...; tile t is REDUCED on rank t % world, by
    the CTA that produces it there (``aligned``) or by CTA (j % grid) for the j-th owned tile (the earlier assignment);
    a reduction needs the tile from every rank. ``all_ctas_wait_for_done``: no CTA exits before every tile is final
    (the earlier kernel); otherwise only the last CTA of the grid waits for that. Returns True when every rank's kernel
    finishes."""
    produced = [set() for _ in range(world)]        # per rank: tiles whose partial sums are in place
    final = set()                                   # tiles reduced and broadcast
    ctas = {}
    for r in range(world):
        owned = [t for t in range(tiles) if t % world == r]
        for c in range(grid):
            mine = list(range(c, tiles, grid))
            if aligned:
                red = [t for t in mine if t % world == r]
            else:
                red = [t for j, t in enumerate(owned) if j % grid == c]
            ctas[(r, c)] = dict(state="queued", prod=mine, red=red)
    for r in range(world):
        for c in range(min(resident, grid)):
            ctas[(r, c)]["state"] = "run"
    while True:
        progress = False
        for (r, c), s in ctas.items():
            if s["state"] != "run":
                continue
            if s["prod"]:                                   # the tensor-core part never waits for anybody
                produced[r].update(s["prod"])
                s["prod"] = []
                progress = True
            while s["red"] and all(s["red"][0] in produced[q] for q in range(world)):
                final.add(s["red"].pop(0))
                progress = True
            must_see_all = all_ctas_wait_for_done or c == grid - 1    # the highest-index CTA: started after all others
            if not s["red"] and (not must_see_all or len(final) == tiles):
                s["state"] = "done"
                progress = True
                nxt = next((k for k in range(grid) if ctas[(r, k)]["state"] == "queued"), None)
                if nxt is not None:
                    ctas[(r, nxt)]["state"] = "run"        # the freed SM takes the next CTA of the grid
        if all(s["state"] == "done" for s in ctas.values()):
            return True
        if not progress:
            return False


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_gemm_collective_does_not_need_its_whole_grid_resident(world):
    grid, tiles = 16, 112
    for resident in (16, 15, 9, 1):
        assert _run_fused_grid(world, grid, tiles, resident, aligned=True, all_ctas_wait_for_done=False)
    # the earlier kernel: fine when every CTA is resident, stuck as soon as one is not
    assert _run_fused_grid(world, grid, tiles, 16, aligned=False, all_ctas_wait_for_done=True)
    assert not _run_fused_grid(world, grid, tiles, 15, aligned=False, all_ctas_wait_for_done=True)
    assert not _run_fused_grid(world, grid, tiles, 15, aligned=True, all_ctas_wait_for_done=True)


# ---------------------------------------------------------------------------------------------------------------
# Signal words of the compare-and-swap barrier when consecutive kernels use DIFFERENT grids (comm.cu:
# block_barrier_all_ranks; dp_reduce_scatter_kernel / dp_all_gather_kernel / allreduce_symm_kernel meet twice per
# launch, the second time at slot offset grid * world, and a bucket's grid depends on its size). A word is a one-bit
# mailbox from one source rank: "put" spins until it is empty, "wait" spins until it is full and empties it. The
# model tags every put with (launch, meeting, block) and fails when a wait consumes a tag that is not its own.

def _run_signal_words(world, grids, delays, meetings=2, blind_put=False):
    words = [dict() for _ in range(world)]            # per rank: slot -> tag (absent = empty)
    lock = threading.Lock()
    bad, dead = [], []

    def put(peer, slot, tag, deadline):
        while True:
            with lock:
                if blind_put or slot not in words[peer]:
                    words[peer][slot] = tag
                    return True
            if time.monotonic() > deadline:
                return False
            time.sleep(0)

    def wait(me, slot, tag, deadline):
        while True:
            with lock:
                got = words[me].pop(slot, None)
            if got is not None:
                if got != tag:
                    bad.append((me, slot, tag, got))
                return True
            if time.monotonic() > deadline:
                return False
            time.sleep(0)

    def block_fn(rank, launch, grid, block, rnd, deadline):
        for meeting in range(meetings):
            time.sleep(delays(rank, launch, block, meeting, "before", rnd))
            slot0 = meeting * grid * world
            for peer in range(world):                 # thread `peer` of the block: put to the peer, wait for its put
                if not put(peer, slot0 + block * world + rank, (launch, meeting, block), deadline):
                    dead.append(("put", rank, launch, block, meeting))
                    return
            time.sleep(delays(rank, launch, block, meeting, "between", rnd))
            for peer in range(world):
                if not wait(rank, slot0 + block * world + peer, (launch, meeting, block), deadline):
                    dead.append(("wait", rank, launch, block, meeting))
                    return

    def rank_fn(rank):
        rnd = random.Random(77 + rank)
        deadline = time.monotonic() + (3 if blind_put else 30)
        for launch, grid in enumerate(grids):         # launches of one stream run one after the other
            blocks = [threading.Thread(target=block_fn, args=(rank, launch, grid, b, rnd, deadline)) for b in range(grid)]
            for t in blocks:
                t.start()
            for t in blocks:
                t.join(40)

    ranks = [threading.Thread(target=rank_fn, args=(r,)) for r in range(world)]
    for t in ranks:
        t.start()
    for t in ranks:
        t.join(60)
    leftovers = [w for w in words if w]
    return bad, dead, leftovers


def _jitter4(rank, launch, block, meeting, where, rnd):
    return rnd.random() * 0.001


def _one_rank_lags(rank, launch, block, meeting, where, rnd):
    # rank 0 is slow to look at its own words after it has signalled its peers, who race ahead meanwhile
    return 0.01 if (rank == 0 and where == "between") else 0.0


@pytest.mark.parametrize("world", [2, 3])
def test_signal_words_survive_grids_that_change_between_launches(world):
    """Growing, shrinking and repeated grids: the second meeting's words of one launch overlap the first meeting's
    words of a launch with a larger grid, and still every wait consumes exactly the put that was meant for it (a
    word is a one-deep FIFO from one source: puts wait for an empty word, and a rank puts in program order)."""
    grids = [1, 4, 2, 4, 1, 3, 3, 2]
    for delays in (_jitter4, _one_rank_lags):
        bad, dead, leftovers = _run_signal_words(world, grids, delays)
        assert not bad and not dead and not leftovers, (bad[:3], dead[:3], leftovers[:1])


def test_signal_word_model_catches_a_put_that_does_not_wait_for_an_empty_word():
    """Negative control: a put that stores without waiting for the word to be empty. A peer that races ahead then
    overwrites the signal a slow rank has not consumed yet, which shows as a wrong tag or as a wait that never ends."""
    def long_lag(rank, launch, block, meeting, where, rnd):
        return 0.05 if (rank == 0 and where == "between") else 0.0

    exposed = False
    for _ in range(3):                                 # a loaded machine may hide the race once; not three times
        bad, dead, leftovers = _run_signal_words(3, [1, 2, 1, 2, 1, 2], long_lag, blind_put=True)
        exposed = bool(bad or dead or leftovers)
        if exposed:
            break
    assert exposed, "the model failed to expose the overwritten signal"
