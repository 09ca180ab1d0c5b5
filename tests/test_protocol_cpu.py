"""Host-side replay of the cross-rank flag protocol of the fused tensor-parallel GEMM -> reduce-scatter kernel.

The kernel (``ops/csrc/fused_tp_gemm.cu``, COMM 2) has no lock: rank ``p`` stores its partial tile into slot
``[epoch parity][p]`` of the owner's receive buffer and then publishes ``flag[parity][p][tile] = epoch``; the owner
waits until every peer's flag is ``>= epoch`` and reads the slots. Flags are never reset and slots are reused every
second call, so correctness rests on one claim: *a rank cannot start call e + 2 before every peer has finished reading
call e*, because call e + 1 needs data that each peer produces only after it has finished call e. This test replays the
protocol as a state machine under thousands of random interleavings (each memory operation is one atomic step; a
rank's own steps keep program order, as release/acquire gives) and checks that every read returns the value of the
epoch it was issued for and that no wait is satisfied by a stale flag."""
import random

import pytest


class Rank:
    def __init__(self, r, tp, calls, tiles):
        self.r, self.tp, self.calls, self.tiles = r, tp, calls, tiles
        self.pc = self._program()
        self.waiting = None

    def _program(self):
        """Yield the atomic steps of this rank in program order."""
        for e in range(1, self.calls + 1):
            par = e & 1
            # remote-owned tiles first (the order the kernel uses), then the own tiles
            for step in range(1, self.tp):
                owner = (self.r + step) % self.tp
                for t in range(self.tiles):
                    yield ("store", owner, par, t, e)
                    yield ("flag", owner, par, t, e)
            for t in range(self.tiles):
                for p in range(self.tp):
                    if p != self.r:
                        yield ("wait", p, par, t, e)
                for p in range(self.tp):
                    if p != self.r:
                        yield ("read", p, par, t, e)


def replay(tp, calls, tiles, seed, rank_cls=None):
    rng = random.Random(seed)
    ranks = [(rank_cls or Rank)(r, tp, calls, tiles) for r in range(tp)]
    # memory of every owner: slot[par][src][tile] = epoch of the data, flag[par][src][tile] = epoch
    slot = [[[[0] * tiles for _ in range(tp)] for _ in range(2)] for _ in range(tp)]
    flag = [[[[0] * tiles for _ in range(tp)] for _ in range(2)] for _ in range(tp)]
    pending = [next(rk.pc, None) for rk in ranks]
    steps = 0
    while any(p is not None for p in pending):
        runnable = []
        for r, op in enumerate(pending):
            if op is None:
                continue
            if op[0] == "wait":
                _, src, par, t, e = op
                if flag[r][par][src][t] >= e:
                    runnable.append(r)
            else:
                runnable.append(r)
        assert runnable, "protocol deadlock"
        r = rng.choice(runnable)
        kind, peer, par, t, e = pending[r]
        if kind == "store":
            slot[peer][par][r][t] = e
        elif kind == "flag":
            flag[peer][par][r][t] = e
        elif kind == "wait":
            assert flag[r][par][peer][t] == e, "a wait was satisfied by a flag of another epoch"
        elif kind == "read":
            assert slot[r][par][peer][t] == e, f"rank {r} read epoch {slot[r][par][peer][t]} data in call {e}"
        pending[r] = next(ranks[r].pc, None)
        steps += 1
    return steps


@pytest.mark.parametrize("tp", [2, 3, 4])
def test_reduce_scatter_flag_protocol_never_reads_stale_or_overwritten_tiles(tp):
    for seed in range(300):
        replay(tp, calls=5, tiles=2, seed=seed)


def test_the_replay_detects_a_protocol_without_the_parity_double_buffer():
    """Sanity of the model itself: with ONE slot per source (no parity) a fast peer overwrites data that the owner has
    not read yet, and the replay must notice under some interleaving."""
    class OneSlot(Rank):
        def _program(self):
            for op in super()._program():
                yield (op[0], op[1], 0, op[3], op[4])

    found = False
    for seed in range(400):
        try:
            replay(2, calls=4, tiles=1, seed=seed, rank_cls=OneSlot)
        except AssertionError:
            found = True
            break
    assert found


# ---- low-latency all-reduce: sentinel-carrying data in rotating generations of the receive buffer -----------------------
def _ll_program(rank, world, calls, generations):
    """The memory operations of one rank, in program order, as the kernel issues them per call: store the contribution
    into slot [rank] of the call's generation on every rank, reset the generation two calls ahead (mod the number of
    generations), then poll every source's slot of the call's generation."""
    ops = []
    for k in range(calls):
        gen = k % generations
        for p in range(world):
            ops.append(("store", (rank + p) % world, gen, rank, k))
        clr = (k + generations - 1) % generations
        for r in range(world):
            ops.append(("reset", rank, clr, r, k))
        for r in range(world):
            ops.append(("poll", rank, gen, r, k))
    return ops


def _ll_replay(world, calls, generations, seed):
    import random
    rng = random.Random(seed)
    SENT = None
    buf = [[[SENT] * world for _ in range(generations)] for _ in range(world)]      # [rank][generation][source]
    progs = [_ll_program(r, world, calls, generations) for r in range(world)]
    pc = [0] * world
    while any(pc[r] < len(progs[r]) for r in range(world)):
        runnable = []
        for r in range(world):
            if pc[r] >= len(progs[r]):
                continue
            op, where, gen, src, k = progs[r][pc[r]]
            if op == "poll" and buf[where][gen][src] is SENT:
                continue                                   # still waiting for the data
            runnable.append(r)
        if not runnable:
            return "deadlock"
        r = rng.choice(runnable)
        op, where, gen, src, k = progs[r][pc[r]]
        if op == "store":
            buf[where][gen][src] = (src, k)
        elif op == "reset":
            buf[where][gen][src] = SENT
        else:
            if buf[where][gen][src] != (src, k):
                return f"rank {r} call {k}: read {buf[where][gen][src]} from source {src}"
        pc[r] += 1
    return "ok"


@pytest.mark.parametrize("world", [2, 3, 8])
def test_ll_allreduce_generations_never_lose_or_mix_contributions(world):
    """Random interleavings of the ranks' stores, resets and polls: with three generations every poll returns the
    polled source's value of the same call, and no schedule deadlocks."""
    for seed in range(300 if world < 8 else 60):
        assert _ll_replay(world, calls=7, generations=3, seed=seed) == "ok"


def test_the_ll_replay_detects_that_two_generations_are_not_enough():
    """With two generations the reset of call k hits the buffer that a faster peer already fills for call k + 1: some
    schedule loses that contribution (the slower rank then waits for ever) or reads a wrong one."""
    outcomes = {_ll_replay(2, calls=6, generations=2, seed=s) for s in range(400)}
    assert outcomes - {"ok"}, outcomes
