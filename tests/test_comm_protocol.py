"""Host model of the one-shot all-reduce protocol of csrc/comm.cu + the GEMV push epilogue,
run under random interleavings of the ranks' memory operations.

The device protocol: all-reduce number e (a counter kept in device memory) writes every
partial value together with e as ONE 64-bit word into slot [e & 1][source rank][element] of
every peer; the finishing kernel of a rank polls each word of its own slots until the epoch
half equals e and sums the value halves in rank order.  There is no flag, no fence and no
barrier: the model checks that two slot generations are enough (a rank can start all-reduce
e + 2 only after every peer has finished reading e), that results are exact, and, as a negative
control, that ONE generation is not enough (a fast rank overwrites words a slow rank still
needs, which the bounded poll reports as a timeout instead of hanging)."""
import random

import pytest


class Timeout(Exception):
    pass


def _rank_program(r, world, slots, n_elem, n_rounds, depth, results, poll_limit):
    """Generator: yields after every memory operation so a scheduler can interleave ranks."""
    for e in range(1, n_rounds + 1):
        gen = e % depth
        for p in range(world):                      # push epilogue: {value, epoch} words to every peer
            for i in range(n_elem):
                slots[p][gen][r][i] = (float(r * 1000 + e * 10 + i), e)
                yield
        out = []
        for i in range(n_elem):                     # finishing kernel: poll, then sum in rank order
            acc = 0.0
            for s in range(world):
                polls = 0
                while True:
                    val, epoch = slots[r][gen][s][i]
                    yield
                    if epoch == e:
                        break
                    polls += 1
                    # a later epoch in the word means the wanted one was overwritten: the device poll
                    # would run into its time limit; the model reports it at once
                    if epoch > e or polls > poll_limit:
                        raise Timeout(f"rank {r} waits for epoch {e} of rank {s}, sees {epoch}")
                acc += val
            out.append(acc)
        results[r].append(out)


def _run(world, depth, seed, n_elem=3, n_rounds=6, poll_limit=2_000_000, bias=None):
    rng = random.Random(seed)
    slots = [[[[(0.0, 0)] * n_elem for _ in range(world)] for _ in range(depth)] for _ in range(world)]
    results = [[] for _ in range(world)]
    progs = {r: _rank_program(r, world, slots, n_elem, n_rounds, depth, results, poll_limit) for r in range(world)}
    weights = bias or [1.0] * world
    while progs:
        live = list(progs)
        r = rng.choices(live, weights=[weights[x] for x in live])[0]
        try:
            next(progs[r])
        except StopIteration:
            del progs[r]
    return results


@pytest.mark.parametrize("world", [2, 4, 8])
def test_two_slot_generations_are_enough_under_any_interleaving(world):
    for seed in range(12):
        # a heavily biased scheduler lets one rank run far ahead of the others
        bias = [20.0 if r == seed % world else 1.0 for r in range(world)] if seed % 2 else None
        results = _run(world, depth=2, seed=seed, bias=bias)
        for e in range(1, 7):
            want = [sum(float(s * 1000 + e * 10 + i) for s in range(world)) for i in range(3)]
            for r in range(world):
                assert results[r][e - 1] == want


def test_one_slot_generation_loses_words_and_the_bounded_poll_reports_it():
    failures = 0
    for seed in range(12):
        try:
            _run(2, depth=1, seed=seed, bias=[20.0, 1.0])
        except Timeout:
            failures += 1
    assert failures > 0
