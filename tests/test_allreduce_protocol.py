"""The mark / parity protocol of the one-kernel all-reduce (csrc/ixb_allreduce.cuh), modelled on the CPU.

Every rank is a generator that performs the kernel's steps one memory operation at a time (peer stores of
{value, call number} words, polls of its own copies until they carry the call number, sum in rank order); a
scheduler interleaves the ranks at random, so fast ranks run as far ahead of slow ones as the protocol lets them.
The model checks what the kernel relies on: two slot parities are enough, and every rank adds in rank order."""
import random

import numpy as np
import pytest


def rank_program(rank, world, mem, inputs, outputs):
    """mem[r]['slots'][parity][sender] = (value, mark); one word per call stands for the vector."""
    epoch = 0
    for x in inputs[rank]:
        e = epoch + 1
        par = e & 1
        for r in range(world):                      # 1. marked data to every rank
            mem[r]["slots"][par][rank] = (x, e)
            yield
        total = np.float32(0)
        for s in range(world):                      # 2. wait for every sender's mark, 3. sum in rank order
            while mem[rank]["slots"][par][s][1] != e:
                yield
            total = np.float32(total + mem[rank]["slots"][par][s][0])
            yield
        outputs[rank].append(total)
        epoch = e


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_two_parities_suffice_under_any_interleaving(world, seed):
    rng = random.Random(seed)
    calls = 40
    nprng = np.random.default_rng(seed)
    inputs = nprng.standard_normal((world, calls)).astype(np.float32)
    mem = [{"slots": [[(np.float32(0), 0)] * world for _ in range(2)]} for _ in range(world)]
    outputs = [[] for _ in range(world)]
    progs = [rank_program(r, world, mem, inputs, outputs) for r in range(world)]
    alive = list(range(world))
    # biased scheduler: some ranks get far more turns than others, so they run ahead as far as the protocol lets them
    weights = [rng.choice([1, 1, 5, 25]) for _ in range(world)]
    steps = 0
    while alive:
        r = rng.choices(alive, weights=[weights[a] for a in alive])[0]
        try:
            next(progs[r])
        except StopIteration:
            alive.remove(r)
        steps += 1
        assert steps < 5_000_000, "the model deadlocked"
    want = []
    for k in range(calls):
        t = np.float32(0)
        for s in range(world):
            t = np.float32(t + inputs[s, k])
        want.append(t)
    for r in range(world):
        assert outputs[r] == want               # the same bits on every rank, in every call


def test_a_single_parity_would_not_be_enough():
    """The same model with one slot buffer goes wrong for some interleaving (a fast rank's next call overwrites a
    word that a slow rank has not read yet, which then never sees its mark) -- the reason for the parity bit."""
    world, calls = 2, 30
    bad = False
    for seed in range(30):
        rng = random.Random(seed)
        inputs = np.arange(world * calls, dtype=np.float32).reshape(world, calls) + 1
        mem = [{"slots": [[(np.float32(0), 0)] * world]} for _ in range(world)]
        outputs = [[] for _ in range(world)]

        def prog(rank):
            epoch = 0
            for x in inputs[rank]:
                e = epoch + 1
                for r in range(world):
                    mem[r]["slots"][0][rank] = (x, e)
                    yield
                total = np.float32(0)
                for s in range(world):
                    polls = 0
                    while mem[rank]["slots"][0][s][1] != e:
                        polls += 1
                        if polls > 2000:                 # the mark was overwritten by a later call: give up
                            break
                        yield
                    total = np.float32(total + mem[rank]["slots"][0][s][0])
                    yield
                outputs[rank].append(total)
                epoch = e

        progs = [prog(r) for r in range(world)]
        alive = list(range(world))
        weights = [1, 40]
        while alive:
            r = rng.choices(alive, weights=[weights[a] for a in alive])[0]
            try:
                next(progs[r])
            except StopIteration:
                alive.remove(r)
        want = [np.float32(inputs[0, k] + inputs[1, k]) for k in range(calls)]
        if outputs[0] != want or outputs[1] != want:
            bad = True
            break
    assert bad
