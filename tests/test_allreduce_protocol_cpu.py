"""Model of the two-shot all-reduce protocol of csrc/comm.cu on CPU threads.

One thread per rank walks through the same sequence of reductions; inside a reduction it
runs its blocks one after the other (the worst case for a GPU: blocks of one grid need not
be resident together), each block following the kernel step by step: flag exchange A, reduce
this rank's slice from every rank's partial buffer, store the result into every rank's
result buffer, flag exchange C. Buffers alternate between two sets as in the communicator.
The model checks what the kernel relies on: block-wise pairing across ranks is enough (no
deadlock without co-residency), epochs kept per block stay consistent when the number of
blocks changes from call to call, slices cover the vector for any size, and the double
buffering makes reuse safe under arbitrary rank skew.
"""

import random
import threading
import time

import numpy as np
import pytest

BLOCK = 4            # elements per "block iteration" (512 16-byte pieces in the kernel)
MAX_BLOCKS = 8       # kMaxArBlocks in the kernel is 128


class Rank:
    def __init__(self, world, cap):
        self.part = [np.zeros(cap), np.zeros(cap)]
        self.res = [np.zeros(cap), np.zeros(cap)]
        self.flags = np.zeros((2, world, MAX_BLOCKS), dtype=np.int64)   # [phase][source][block]
        self.epochs = np.zeros(MAX_BLOCKS, dtype=np.int64)


def _exchange(ranks, me, phase, b, e, deadline):
    for peer in ranks:                       # publish to every rank, my own copy included
        peer.flags[phase, me, b] = e
    mine = ranks[me].flags
    for j in range(len(ranks)):
        while mine[phase, j, b] < e:
            if time.time() > deadline:
                raise TimeoutError("rank %d block %d phase %d waits for rank %d" % (me, b, phase, j))
            time.sleep(0)


def _block(ranks, me, key, n, b, nblocks, deadline):
    world = len(ranks)
    r = ranks[me]
    e = r.epochs[b] + 1
    _exchange(ranks, me, 0, b, e, deadline)
    slice_len = (n + world - 1) // world
    lo = me * slice_len
    hi = min(lo + slice_len, n)
    i = lo + b * BLOCK
    while i < hi:
        j = min(i + BLOCK, hi)
        acc = np.zeros(j - i)
        for peer in ranks:                   # fixed rank order
            acc = acc + peer.part[key][i:j]
        for peer in ranks:
            peer.res[key][i:j] = acc
        i += nblocks * BLOCK
    _exchange(ranks, me, 1, b, e, deadline)
    r.epochs[b] = e


def _rank_thread(ranks, me, sizes, inputs, outputs, errors, seed):
    rng = random.Random(seed)
    world = len(ranks)
    deadline = time.time() + 60
    try:
        for k, n in enumerate(sizes):
            key = k & 1
            if rng.random() < 0.3:
                time.sleep(rng.random() * 0.003)          # rank skew
            ranks[me].part[key][:n] = inputs[k][me]       # the GEMM writes its partial product
            slice_len = (n + world - 1) // world
            nblocks = max(1, min(MAX_BLOCKS, (slice_len + BLOCK - 1) // BLOCK))
            for b in range(nblocks):
                _block(ranks, me, key, n, b, nblocks, deadline)
            outputs[me].append(ranks[me].res[key][:n].copy())   # the consumer reads the result
    except Exception as exc:  # noqa: BLE001 - reported by the test
        errors.append(exc)


@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_two_shot_protocol_model(world):
    rng = np.random.default_rng(world)
    sizes = [int(rng.integers(1, 150)) for _ in range(24)]
    cap = max(sizes)
    inputs = [[rng.integers(-50, 50, size=n).astype(np.float64) for _ in range(world)] for n in sizes]
    ranks = [Rank(world, cap) for _ in range(world)]
    outputs = [[] for _ in range(world)]
    errors: list = []
    threads = [threading.Thread(target=_rank_thread, args=(ranks, r, sizes, inputs, outputs, errors, 7 * r + world))
               for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=90)
    assert not errors, errors
    assert all(not t.is_alive() for t in threads)
    for k, n in enumerate(sizes):
        want = sum(inputs[k])
        for r in range(world):
            assert np.array_equal(outputs[r][k], want), (k, n, r)
