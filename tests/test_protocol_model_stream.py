"""CPU model of the hand-over protocol of the persistent summary selector
(csrc/indexer_summary_stream.cu).

Roles of one CTA: TMA producer warp, single-thread MMA issuer, eight epilogue warps, two chunk
filter warps, four settle warps. They talk through mbarriers only: a ring of two key-tile slots,
one query-descriptor buffer per work unit, two TMEM accumulators, two score-chunk buffers, and one
candidate area per settle warp (filled by the filter warp that keeps its lists). Every
role derives ring slot, accumulator, chunk buffer and the phase it waits for from its own
counters (tiles, chunks, units handled so far). The model restates each role's control flow and
runs the roles under random interleavings with asynchronous TMA completion and an in-order
tensor pipe, checking at every step that

* no wait finds its barrier two or more phases ahead (a parity wait would alias) and every role
  finishes (no deadlock);
* an MMA reads the key tile / query buffer the issuer thinks is there and no TMA load overwrites
  one that an issued MMA has yet to read;
* an accumulator is not overwritten before all eight epilogue warps have read it, a chunk buffer
  is neither overwritten while a filter warp still reads it nor read before all eight epilogue
  warps have written their part;
* every filter warp sees every chunk of every unit exactly once, in order; a settle warp finds
  the candidates of the unit it expects, and they are not overwritten while it works on them.

Mirrors the kernel by hand: a change of its protocol must be made here too. Same purpose as the
reference's attention/q_centric/tests/test_schedule.py:6-100 for its own ring schedule.
"""
import random

import pytest

A_STAGES, EPI, NFLT, NSEL = 2, 8, 2, 4


class Bar:
    def __init__(self, name, count):
        self.name, self.count, self.pending, self.tx, self.phase = name, count, count, 0, 0

    def arrive(self):
        assert self.pending > 0, f"{self.name}: more arrivals than expected in phase {self.phase}"
        self.pending -= 1
        self._flip()

    def expect_tx(self, n):
        self.tx += n
        self.arrive()

    def complete_tx(self, n):
        self.tx -= n
        self._flip()

    def _flip(self):
        if self.pending == 0 and self.tx == 0:
            self.phase += 1
            self.pending = self.count

    def done(self, k):
        assert self.phase <= k + 1, f"{self.name}: waiting for phase {k} but the barrier is in phase {self.phase}"
        return self.phase > k


def run_cta(units, num_tiles, ch_tiles, rng, skip=None):
    """units: number of work units of this CTA. skip: name prefix of a barrier whose waits are ignored
    (to show that the model can fail)."""
    num_chunks = -(-num_tiles // ch_tiles)
    B = {}
    for s in range(A_STAGES):
        B["A_FULL", s] = Bar(f"A_FULL{s}", 1)
        B["A_EMPTY", s] = Bar(f"A_EMPTY{s}", 1)
    B["B_FULL"] = Bar("B_FULL", 1)
    B["B_EMPTY"] = Bar("B_EMPTY", 1)
    for i in range(2):
        B["ACC_FULL", i] = Bar(f"ACC_FULL{i}", 1)
        B["ACC_EMPTY", i] = Bar(f"ACC_EMPTY{i}", EPI)
        B["SC_FULL", i] = Bar(f"SC_FULL{i}", EPI)
        B["SC_EMPTY", i] = Bar(f"SC_EMPTY{i}", NFLT)
    for w in range(NSEL):
        B["FIN_FULL", w] = Bar(f"FIN_FULL{w}", 1)
        B["FIN_EMPTY", w] = Bar(f"FIN_EMPTY{w}", 1)
    fin = [None] * NSEL                 # unit whose candidates sit in each settle warp's area
    fin_busy = [False] * NSEL           # the settle warp is working on them
    ring = [None] * A_STAGES
    ring_readers = [0] * A_STAGES
    qbuf, qbuf_readers = None, 0
    acc = [None, None]                  # (unit, tile) held by each accumulator
    acc_unread = [0, 0]                 # epilogue warps that have yet to read it
    sc = [None, None]                   # (unit, chunk) of each chunk buffer
    sc_written = [0, 0]                 # epilogue warps that have finished their part of it
    sc_readers = [0, 0]                 # selection warps still reading
    tma_inflight, pipe = [], []
    seen = [[] for _ in range(NFLT)]
    settled = [[] for _ in range(NSEL)]

    def wait(bar, phase):
        return ("wait", bar, phase)

    def producer():
        nonlocal qbuf
        fills = 0
        for u in range(units):
            if u > 0:
                yield wait(B["B_EMPTY"], u - 1)
            assert qbuf_readers == 0, "query buffer overwritten before its MMAs ran"
            B["B_FULL"].expect_tx(1)
            tma_inflight.append((B["B_FULL"], "q", None, ("Q", u)))
            for t in range(num_tiles):
                s, use = fills % A_STAGES, fills // A_STAGES
                if use > 0:
                    yield wait(B["A_EMPTY", s], use - 1)
                assert ring_readers[s] == 0, f"ring slot {s} overwritten before its MMAs ran"
                B["A_FULL", s].expect_tx(1)
                tma_inflight.append((B["A_FULL", s], "ring", s, ("K", u, t)))
                fills += 1
                yield ("step",)

    def issuer():
        nonlocal qbuf_readers
        g = 0
        for u in range(units):
            yield wait(B["B_FULL"], u)
            for t in range(num_tiles):
                s, a = g % A_STAGES, g & 1
                yield wait(B["A_FULL", s], g // A_STAGES)
                if g >= 2:
                    yield wait(B["ACC_EMPTY", a], (g >> 1) - 1)
                assert ring[s] == ("K", u, t), f"MMA of unit {u} tile {t} finds {ring[s]} in slot {s}"
                assert qbuf == ("Q", u), f"MMA of unit {u} finds {qbuf} in the query buffer"
                assert acc_unread[a] == 0, f"accumulator {a} overwritten with {acc_unread[a]} readers left"
                ring_readers[s] += 1
                qbuf_readers += 1

                def mma(s=s, a=a, u=u, t=t):
                    nonlocal qbuf_readers
                    ring_readers[s] -= 1
                    qbuf_readers -= 1
                    acc[a] = (u, t)
                    acc_unread[a] = EPI
                pipe.append(("mma", mma))
                pipe.append(("commit", B["A_EMPTY", s]))
                pipe.append(("commit", B["ACC_FULL", a]))
                if t == num_tiles - 1:
                    pipe.append(("commit", B["B_EMPTY"]))
                g += 1
                yield ("step",)

    def epilogue(w):
        g = h = 0
        for u in range(units):
            for t in range(num_tiles):
                a, slot = g & 1, t % ch_tiles
                yield wait(B["ACC_FULL", a], g >> 1)
                if slot == 0 and h >= 2:
                    yield wait(B["SC_EMPTY", h & 1], (h >> 1) - 1)
                assert acc[a] == (u, t), f"epilogue {w} of unit {u} tile {t} finds {acc[a]}"
                yield ("step",)                      # TMEM loads
                acc_unread[a] -= 1
                yield ("arrive", B["ACC_EMPTY", a])
                buf = h & 1
                assert sc_readers[buf] == 0, f"chunk buffer {buf} written while {sc_readers[buf]} selection warps read it"
                if slot == 0 and w == 0:
                    sc[buf] = (u, t // ch_tiles)
                yield ("step",)                      # score stores
                if slot == ch_tiles - 1 or t == num_tiles - 1:
                    sc_written[buf] += 1
                    yield ("arrive", B["SC_FULL", buf])
                    h += 1
                g += 1

    def chunk_filter(f):
        h = 0
        for u in range(units):
            for c in range(num_chunks):
                buf = h & 1
                yield wait(B["SC_FULL", buf], h >> 1)
                assert sc_written[buf] >= EPI, f"filter {f} reads chunk buffer {buf} with {sc_written[buf]} parts written"
                sc_readers[buf] += 1
                yield ("step",)
                seen[f].append((u, c))
                sc_readers[buf] -= 1
                if sc_readers[buf] == 0 and all(len(x) >= len(seen[f]) for x in seen):
                    sc_written[buf] = 0              # the last reader of this use of the buffer
                yield ("arrive", B["SC_EMPTY", buf])
                h += 1
            for y in range(2):                       # hand the unit's candidates to the two settle warps
                w = 2 * f + y
                if u > 0:
                    yield wait(B["FIN_EMPTY", w], u - 1)
                assert not fin_busy[w], f"candidate area of settle warp {w} overwritten while it is in use"
                fin[w] = u
                yield ("step",)
                yield ("arrive", B["FIN_FULL", w])

    def settle(w):
        for u in range(units):
            yield wait(B["FIN_FULL", w], u)
            assert fin[w] == u, f"settle warp {w} expects unit {u}, its area holds {fin[w]}"
            fin_busy[w] = True
            for _ in range(rng.randrange(1, 200)):   # settling a unit's lists takes a while
                yield ("step",)
            assert fin[w] == u
            settled[w].append(u)
            fin_busy[w] = False
            yield ("arrive", B["FIN_EMPTY", w])

    roles = [producer(), issuer()] + [epilogue(w) for w in range(EPI)] + [chunk_filter(f) for f in range(NFLT)] \
        + [settle(w) for w in range(NSEL)]
    pending, alive, steps = [None] * len(roles), [True] * len(roles), 0
    while True:
        choices = []
        for r in range(len(roles)):
            if not alive[r]:
                continue
            op = pending[r]
            if op is None or op[0] != "wait" or (skip and op[1].name.startswith(skip)) or op[1].done(op[2]):
                choices.append(("role", r))
        if tma_inflight:
            choices.append(("tma", None))
        if pipe:
            choices.append(("pipe", None))
        if not choices:
            break
        kind, r = rng.choice(choices)
        steps += 1
        assert steps < 3_000_000, "model did not terminate"
        if kind == "tma":
            bar, where, index, tag = tma_inflight.pop(rng.randrange(len(tma_inflight)))
            if where == "ring":
                ring[index] = tag
            else:
                qbuf = tag
            bar.complete_tx(1)
        elif kind == "pipe":
            what, arg = pipe.pop(0)
            if what == "mma":
                arg()
            else:
                arg.arrive()
        else:
            pending[r] = None
            try:
                op = next(roles[r])
            except StopIteration:
                alive[r] = False
                continue
            if op[0] == "arrive":
                op[1].arrive()
            elif op[0] == "wait":
                pending[r] = op
    stuck = [r for r in range(len(roles)) if alive[r]]
    assert not stuck, f"deadlock: roles {stuck} blocked on {[(pending[r][1].name, pending[r][2], pending[r][1].phase) for r in stuck]}"
    assert not tma_inflight and not pipe
    expected = [(u, c) for u in range(units) for c in range(num_chunks)]
    for f in range(NFLT):
        assert seen[f] == expected, f"filter warp {f} saw {seen[f][:6]}..."
    for w in range(NSEL):
        assert settled[w] == list(range(units))


@pytest.mark.parametrize("units", [1, 2, 5])
@pytest.mark.parametrize("num_tiles,ch_tiles", [(1, 1), (2, 8), (5, 1), (16, 8), (9, 4), (22, 16), (7, 2)])
def test_roles_agree_on_slots_buffers_and_phases(units, num_tiles, ch_tiles):
    rng = random.Random(100 * units + 10 * num_tiles + ch_tiles)
    for _ in range(4):
        run_cta(units, num_tiles, ch_tiles, rng)


@pytest.mark.parametrize("skip", ["SC_EMPTY", "ACC_EMPTY", "A_EMPTY", "B_EMPTY", "FIN_EMPTY"])
def test_model_catches_a_missing_release(skip):
    """The model must be able to fail: ignore one of the release barriers and a hazard, a phase alias
    or a deadlock has to show up."""
    rng = random.Random(7)
    hits = 0
    for _ in range(20):
        try:
            run_cta(3, 9, 2, rng, skip=skip)
        except AssertionError:
            hits += 1
    assert hits > 0
