"""CPU model (threads + locked counters) of the flag protocol of the GEMM -> reduce-scatter kernel:
producers bump the owner's per-row-tile counter after their stores, reducers claim work items from
a queue and wait - with a deadline - until the counter shows every rank's contribution.  The model
checks the properties the device code relies on: every item is reduced exactly once with complete
data under any interleaving, and a missing producer ends in a reported time-out instead of a hang."""
import random
import threading
import time

W, TILES, N_TILES_N, WARPS, SPLIT = 4, 3, 2, 4, 4


class Rank:
    def __init__(self):
        self.lock = threading.Lock()
        self.flags = [0] * TILES                       # bumped by every rank's epilogue warps
        self.stage = [[0] * W for _ in range(TILES)]   # stage[j][src] = contributions landed
        self.work = 0
        self.reduced = []
        self.timeouts = 0


def producer(ranks, me, missing, seed):
    rng = random.Random(seed)
    order = [(j, (me + 1 + oi) % W) for j in range(TILES) for oi in range(W)]      # row-tile major, own block last
    for j, owner in order:
        if (me, owner) in missing:
            continue
        for _ in range(N_TILES_N):
            time.sleep(rng.random() * 1e-4)
            for _ in range(WARPS):
                with ranks[owner].lock:                 # stores, fence, then the counter bump
                    ranks[owner].stage[j][me] += 1
                    ranks[owner].flags[j] += 1


def reducer(rank: Rank, limit_s: float):
    want = W * N_TILES_N * WARPS
    while True:
        with rank.lock:
            it = rank.work
            rank.work += 1
        if it >= TILES * SPLIT:
            return
        j = it // SPLIT
        t0 = time.monotonic()
        while True:
            with rank.lock:
                ready = rank.flags[j] >= want
            if ready:
                break
            if time.monotonic() - t0 > limit_s:
                with rank.lock:
                    rank.timeouts += 1
                return                                   # report and leave: never spin for ever
            time.sleep(1e-5)
        with rank.lock:
            assert all(c == N_TILES_N * WARPS for c in rank.stage[j]), "reduced before every contribution landed"
            rank.reduced.append(it)


def _run(missing=(), limit_s=2.0, seed=0):
    ranks = [Rank() for _ in range(W)]
    threads = [threading.Thread(target=producer, args=(ranks, r, set(missing), seed * 10 + r)) for r in range(W)]
    threads += [threading.Thread(target=reducer, args=(ranks[r], limit_s)) for r in range(W) for _ in range(3)]
    random.Random(seed).shuffle(threads)
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=20)
    assert not any(t.is_alive() for t in threads), "a thread is stuck"
    return ranks


def test_every_item_reduced_once_under_random_interleavings():
    for seed in range(5):
        ranks = _run(seed=seed)
        for r in ranks:
            assert sorted(r.reduced) == list(range(TILES * SPLIT)) and r.timeouts == 0


def test_missing_contribution_times_out_instead_of_hanging():
    ranks = _run(missing=[(2, 0)], limit_s=0.2)          # rank 2 never sends its tiles of rank 0's rows
    assert ranks[0].timeouts > 0 and ranks[0].reduced == []
    for r in ranks[1:]:
        assert sorted(r.reduced) == list(range(TILES * SPLIT)) and r.timeouts == 0
