"""CPU model of the flag hand-shake of the cross-GPU merge over peer memory (csrc/peer_exchange.cu,
sharding.PeerExchange): R ranks, each one stream of

    wait  done[*]  >= e - 1     (every reader of my previous partial has finished)
    write my partial of epoch e  (peer-load form: into my own memory; scatter form: slice j into rank j's slot `me`)
    signal ready[me] := e        (into every rank's flag block, after the writes)
    merge: wait ready[*] >= e, read the R partials of my slice
    signal done[me] := e         (into every rank's flag block)

The flag words a rank polls live in its own memory; a signal is R remote stores that arrive after arbitrary delays and
in any order (each word is written by one rank with increasing values, so a word only grows). The model runs the ranks
under random interleavings with delayed flag delivery and checks that a merge of epoch e reads nothing but partials of
epoch e, that no partial is overwritten while a rank still reads it, and that every rank finishes (no deadlock). It
mirrors the protocol by hand: a change there must be made here too."""
import random

import pytest


def run(ranks, epochs, rng, scatter, skip=None):
    ready = [[0] * ranks for _ in range(ranks)]          # ready[r][j]: rank r's copy of rank j's ready flag
    done = [[0] * ranks for _ in range(ranks)]
    # memory[r][j]: peer-load form: slice j of rank r's partial; scatter form: slot j of rank r (written by rank j)
    memory = [[0] * ranks for _ in range(ranks)]
    reading = [[0] * ranks for _ in range(ranks)]        # readers currently inside memory[r][j]
    in_flight = []                                       # (table, target rank, word, value)
    merged = [[] for _ in range(ranks)]

    def rank(me):
        for e in range(1, epochs + 1):
            if skip != "done":
                yield ("wait", done[me], e - 1)
            for j in range(ranks):                       # the attention kernel, tile by tile
                r, slot = (j, me) if scatter else (me, j)
                assert reading[r][slot] == 0, f"rank {me} overwrites memory[{r}][{slot}] while it is being read (epoch {e})"
                memory[r][slot] = e
                yield ("step",)
            for t in range(ranks):                       # kernel boundary, fence, then the flag stores
                in_flight.append((ready, t, me, e))
            yield ("step",)
            if skip != "ready":
                yield ("wait", ready[me], e)
            cells = [(me, j) if scatter else (j, me) for j in range(ranks)]
            for r, slot in cells:
                reading[r][slot] += 1
            yield ("step",)
            for r, slot in cells:
                assert memory[r][slot] == e, f"rank {me} merges epoch {e} but memory[{r}][{slot}] holds epoch {memory[r][slot]}"
            yield ("step",)
            for r, slot in cells:
                reading[r][slot] -= 1
            merged[me].append(e)
            for t in range(ranks):
                in_flight.append((done, t, me, e))
            yield ("step",)

    procs = [rank(r) for r in range(ranks)]
    pending, alive, steps = [None] * ranks, [True] * ranks, 0
    while True:
        choices = []
        for r in range(ranks):
            if not alive[r]:
                continue
            op = pending[r]
            if op is None or op[0] != "wait" or all(v >= op[2] for v in op[1]):
                choices.append(r)
        if in_flight:
            choices.append(-1)
        if not choices:
            break
        pick = rng.choice(choices)
        steps += 1
        assert steps < 1_000_000
        if pick < 0:
            table, target, word, value = in_flight.pop(rng.randrange(len(in_flight)))
            table[target][word] = max(table[target][word], value)
            continue
        pending[pick] = None
        try:
            pending[pick] = next(procs[pick])
        except StopIteration:
            alive[pick] = False
    stuck = [r for r in range(ranks) if alive[r]]
    assert not stuck, f"deadlock: ranks {stuck} blocked on {[pending[r][2] for r in stuck]}"
    assert all(m == list(range(1, epochs + 1)) for m in merged)


@pytest.mark.parametrize("scatter", [False, True])
@pytest.mark.parametrize("ranks", [1, 2, 4, 8])
def test_every_merge_reads_its_own_epoch_and_nothing_is_overwritten_under_a_reader(ranks, scatter):
    rng = random.Random(31 * ranks + int(scatter))
    for _ in range(30):
        run(ranks, 5, rng, scatter)


@pytest.mark.parametrize("scatter", [False, True])
@pytest.mark.parametrize("skip", ["done", "ready"])
def test_model_catches_a_missing_wait(skip, scatter):
    """The model must be able to fail: without the wait on the done flags a partial is overwritten under a reader (or
    read an epoch late), without the wait on the ready flags a merge reads an old partial."""
    rng = random.Random(5)
    hits = 0
    for _ in range(40):
        try:
            run(3, 4, rng, scatter, skip=skip)
        except AssertionError:
            hits += 1
    assert hits > 0
