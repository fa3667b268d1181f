"""A host-side model of the schedule inside fp8_linear_skinny_kernel (csrc/fp8_linear.cu): every thread issues the
weights of k step j as cp.async group j into slot j % depth of a shared-memory ring, fetches a chunk of activations
together with the first step of the chunk into one of two buffers, and multiplies step i after waiting until at most
depth - 1 groups are pending.  The model replays that schedule for many step counts and asserts what the kernel relies
on: a step's group has been committed and waited for before the step is multiplied, a ring slot is never refilled
before its step has been multiplied, an activation buffer is never refilled while a warp that is one block barrier
behind could still read it, and the split of k over the cluster and of the fragments over a warp covers every weight
byte exactly once in both weight layouts.  The constants are read from the source, so the model follows the kernel.
"""
import os
import re

import pytest

SRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "gpuk_b200", "csrc", "fp8_linear.cu")


def _const(name):
    m = re.search(r"constexpr int %s = (\d+);" % name, open(SRC).read())
    assert m, name
    return int(m.group(1))


DEPTH, XSTEPS, STEP, TILE, WARPS = (_const(n) for n in ("kDepth", "kXSteps", "kStepBytes", "kTileN", "kWarps"))


def test_constants_satisfy_what_the_schedule_needs():
    assert DEPTH & (DEPTH - 1) == 0 and XSTEPS & (XSTEPS - 1) == 0      # slots and chunks are taken with masks
    assert TILE == WARPS * 16 and STEP == 64                            # one 16-row fragment per warp, 16 bytes per thread and row


@pytest.mark.parametrize("nsteps", list(range(0, 40)) + [56, 64, 65, 128, 448])
def test_ring_slots_groups_and_activation_buffers(nsteps):
    committed = 0                    # cp.async groups committed so far by this thread
    slot_holds = [None] * DEPTH      # step whose weights a ring slot holds (or is being filled with)
    multiplied = set()
    buf_holds = [None, None]         # chunk an activation buffer holds
    barrier_passed = -1              # last chunk whose block barrier this thread has passed

    def issue(j):
        nonlocal committed
        if j < nsteps:
            s = j & (DEPTH - 1)
            assert slot_holds[s] is None or slot_holds[s] in multiplied, (j, slot_holds[s])      # refilled only after use
            slot_holds[s] = j
            if j & (XSTEPS - 1) == 0:
                c = j // XSTEPS
                old = buf_holds[c & 1]
                # the chunk this buffer held must be behind the last barrier this thread passed: every other warp
                # has then finished multiplying it (it arrived at that barrier too)
                assert old is None or old < barrier_passed, (j, old, barrier_passed)
                buf_holds[c & 1] = c
        committed += 1               # an empty group past the end keeps the count uniform

    for j in range(DEPTH - 1):
        issue(j)
    for i in range(nsteps):
        issue(i + DEPTH - 1)
        complete = committed - (DEPTH - 1)          # cp.async.wait_group depth - 1
        assert complete >= i + 1                    # group i has landed
        if i & (XSTEPS - 1) == 0:
            barrier_passed = i // XSTEPS            # __syncthreads: the chunk is visible to all warps
        assert slot_holds[i & (DEPTH - 1)] == i
        assert buf_holds[(i // XSTEPS) & 1] == i // XSTEPS and barrier_passed == i // XSTEPS
        multiplied.add(i)
    assert multiplied == set(range(nsteps))


@pytest.mark.parametrize("k,ks", [(64, 1), (64, 8), (1024, 8), (3584, 8), (4160, 4), (8192, 4), (8192, 8)])
def test_k_split_over_the_cluster_covers_every_step_once(k, ks):
    steps = k // STEP
    base, extra = divmod(steps, ks)
    seen = []
    for part in range(ks):
        begin = part * base + min(part, extra)
        seen += list(range(begin, begin + base + (1 if part < extra else 0)))
    assert seen == list(range(steps))


@pytest.mark.parametrize("packed", [False, True])
def test_every_weight_byte_of_a_tile_is_fetched_once(packed):
    n, k = TILE, 4 * STEP
    fetched = {}
    for warp in range(WARPS):
        for lane in range(32):
            g, t = lane >> 2, lane & 3
            n0 = warp * 16
            for step in range(k // STEP):
                for h in range(2):
                    if packed:      # block (n0 / 16, step): row r of the fragment at r * 64
                        off = (n0 // 16) * k * 16 + step * 16 * STEP + (h * 8 + g) * STEP + 16 * t
                        row, col = n0 + (off % (16 * STEP)) // STEP, step * STEP + off % STEP
                    else:
                        off = (n0 + h * 8 + g) * k + step * STEP + 16 * t
                        row, col = off // k, off % k
                    assert (row, col) == (n0 + h * 8 + g, step * STEP + 16 * t)
                    for b in range(16):
                        fetched[(row, col + b)] = fetched.get((row, col + b), 0) + 1
    assert len(fetched) == n * k and set(fetched.values()) == {1}
