"""CPU model of the attention kernel's hand-over protocol (csrc/q_centric.cu).

The kernel's roles (TMA producer warp, single-thread MMA issuer, 2 x 4 softmax warps, 4 epilogue
warps) talk only through mbarriers; the producer and the MMA issuer walk the SAME token order
(K and V tiles of two streams through one ring, the first K tile and the Q tile of a stream's next
item primed before the current item has drained) without ever exchanging it. A mistake in that
protocol shows on hardware as a bounded-wait abort at best. This model restates every role's
control flow operation by operation (waits with the phase they expect, arrives, TMA loads, MMAs,
commits) and runs them under random interleavings with asynchronous TMA completion and an
in-order tensor pipe, checking at every step:

* no wait ever finds its barrier two or more phases ahead (a parity wait would alias) and every
  role finishes (no deadlock);
* an MMA reads from a ring slot / Q buffer exactly the tile the issuer thinks it holds, and no TMA
  load overwrites a slot that an issued MMA has yet to read;
* S is not overwritten while a softmax warp still reads it, PV only runs on completely written P,
  O is not overwritten before the epilogue has read it out, the row statistics are not
  overwritten before the epilogue has read them;
* every (item, stream) is produced exactly once and with the right number of tiles.

Same purpose as the reference's attention/q_centric/tests/test_schedule.py:6-100 (a CPU model of
its own, simpler, ring schedule). Mirrors q_centric.cu by hand: a change of the kernel's protocol
must be made here too.
"""
import random

import pytest

RING = 4


class Bar:
    """mbarrier: `count` arrivals (+ outstanding transaction bytes) complete a phase."""

    def __init__(self, name, count):
        self.name, self.count, self.pending, self.tx, self.phase = name, count, count, 0, 0

    def arrive(self):
        assert self.pending > 0, f"{self.name}: more arrivals than the barrier expects in phase {self.phase}"
        self.pending -= 1
        self._maybe_flip()

    def expect_tx(self, n):
        self.tx += n
        self.arrive()

    def complete_tx(self, n):
        self.tx -= n
        self._maybe_flip()

    def _maybe_flip(self):
        if self.pending == 0 and self.tx == 0:
            self.phase += 1
            self.pending = self.count

    def done(self, k):
        """Has phase k completed? A parity wait cannot tell phase k from phase k + 2."""
        assert self.phase <= k + 1, f"{self.name}: waiting for phase {k} but the barrier is in phase {self.phase}"
        return self.phase > k


class Model:
    def __init__(self, counts, pair_mode, grid, rng):
        """counts[item] = (count of stream 0, count of stream 1 or None when the stream does not exist)."""
        self.counts, self.pair, self.grid, self.rng = counts, pair_mode, grid, rng
        self.failures = []

    # ------------------------------------------------------------------ one CTA
    def run_cta(self, cta):
        items = list(range(cta, len(self.counts), self.grid))
        rng = self.rng
        B = {}
        for q in range(2):
            for name, cnt in (("Q_FULL", 1), ("Q_EMPTY", 1), ("S_FULL", 1), ("P_FULL", 4), ("O_FULL", 1), ("P_HALF", 4),
                              ("STATS_FULL", 4), ("O_EMPTY", 4), ("STATS_EMPTY", 4)):
                B[(name, q)] = Bar(f"{name}{q}", cnt)
        for s in range(RING):
            B[("KV_FULL", s)] = Bar(f"KV_FULL{s}", 1)
            B[("KV_EMPTY", s)] = Bar(f"KV_EMPTY{s}", 1)
        ring = [None] * RING            # tile tag held by each slot
        ring_readers = [0] * RING       # issued MMAs that have yet to read the slot
        qbuf = [None, None]
        qbuf_readers = [0, 0]
        s_version = [None, None]        # (item, tile) whose scores are in S[q]
        s_reading = [[None] * 4, [None] * 4]   # what each softmax warp is still reading
        p_ready = [[None] * 4, [None] * 4]     # (item, tile, part) written by each warp: part 1 = 3/4, 2 = all
        o_state = [None, None]          # (item, tiles accumulated)
        o_unread = [None, None]         # item whose O the epilogue has yet to read
        o_readers = [0, 0]              # epilogue warps that have yet to read it
        stats_item = [None, None]
        stats_unread = [[False] * 4, [False] * 4]
        stored = {}
        tma_inflight = []               # (barrier, kind, index, tag)
        pipe = []                       # in-order tensor pipe: ("mma", fn) / ("commit", bar)
        cnt = lambda item, q: (self.counts[item][q] or 0)
        valid = lambda item, q: self.counts[item][q] is not None

        def tag_k(item, q, i):
            return ("K", item, None if self.pair else q, i)

        def tag_v(item, q, i):
            return ("V", item, None if self.pair else q, i)

        # -------------------------------------------------------------- producer warp
        def producer():
            fills, qloads, primed = 0, [0, 0], [False, False]

            def push(tag):
                nonlocal fills
                slot, use = fills % RING, fills // RING
                if use > 0:
                    yield ("wait", B[("KV_EMPTY", slot)], use - 1)
                assert ring_readers[slot] == 0, f"TMA overwrites ring slot {slot} before its MMAs ran"
                B[("KV_FULL", slot)].expect_tx(1)
                tma_inflight.append((B[("KV_FULL", slot)], "ring", slot, tag))
                fills += 1

            def push_q(q, item):
                if qloads[q] > 0:
                    yield ("wait", B[("Q_EMPTY", q)], qloads[q] - 1)
                assert qbuf_readers[q] == 0, f"TMA overwrites Q{q} before its MMAs ran"
                B[("Q_FULL", q)].expect_tx(1)
                tma_inflight.append((B[("Q_FULL", q)], "q", q, ("Q", item, q)))
                qloads[q] += 1

            for pos, item in enumerate(items):
                has_next = pos + 1 < len(items)
                nxt = items[pos + 1] if has_next else None
                if self.pair:
                    n = cnt(item, 0)
                    was_primed, primed[0], primed[1] = primed[0], False, False
                    if n == 0:
                        continue
                    if not was_primed:
                        yield from push_q(0, item)
                        yield from push_q(1, item)
                        yield from push(tag_k(item, 0, 0))
                    for i in range(n):
                        yield from push(tag_v(item, 0, i))
                        if i + 1 < n:
                            yield from push(tag_k(item, 0, i + 1))
                        elif has_next and cnt(nxt, 0) > 0:
                            yield from push_q(0, nxt)
                            yield from push(tag_k(nxt, 0, 0))
                            yield from push_q(1, nxt)
                            primed[0] = primed[1] = True
                else:
                    was_primed = list(primed)
                    primed[0] = primed[1] = False
                    for q in range(2):
                        if cnt(item, q) > 0 and not was_primed[q]:
                            yield from push_q(q, item)
                            yield from push(tag_k(item, q, 0))
                    for i in range(max(cnt(item, 0), cnt(item, 1))):
                        for q in range(2):
                            if i < cnt(item, q):
                                yield from push(tag_v(item, q, i))
                                if i + 1 < cnt(item, q):
                                    yield from push(tag_k(item, q, i + 1))
                                elif has_next and cnt(nxt, q) > 0:
                                    yield from push_q(q, nxt)
                                    yield from push(tag_k(nxt, q, 0))
                                    primed[q] = True

        # -------------------------------------------------------------- MMA issuer
        def issuer():
            taken, qtaken, pphase, hphase, o_done = 0, [0, 0], [0, 0], [0, 0], [0, 0]
            primed = [False, False]

            def acquire(box):
                nonlocal taken
                slot = taken % RING
                yield ("wait", B[("KV_FULL", slot)], taken // RING)
                taken += 1
                box.append(slot)

            def wait_q(q):
                yield ("wait", B[("Q_FULL", q)], qtaken[q])
                qtaken[q] += 1

            def issue_qk(q, slot, item, i):
                ring_readers[slot] += 1
                qbuf_readers[q] += 1

                def run():
                    assert ring[slot] == tag_k(item, q, i), f"QK of item {item} stream {q} tile {i} reads {ring[slot]}"
                    assert qbuf[q] == ("Q", item, q), f"QK of item {item} stream {q} reads {qbuf[q]}"
                    assert all(r is None for r in s_reading[q]), f"S{q} overwritten while a softmax warp reads it"
                    s_version[q] = (item, i)
                    ring_readers[slot] -= 1
                    qbuf_readers[q] -= 1
                pipe.append(("mma", run))

            def issue_pv(q, slot, item, i, part):
                ring_readers[slot] += 1

                def run():
                    assert ring[slot] == tag_v(item, q, i), f"PV of item {item} stream {q} tile {i} reads {ring[slot]}"
                    need = 1 if part == 1 else 2
                    assert all(p is not None and p[:2] == (item, i) and p[2] >= need for p in p_ready[q]), \
                        f"PV part {part} of item {item} stream {q} tile {i} runs on incomplete P {p_ready[q]}"
                    if part == 1 or not self.pair:
                        if i == 0:
                            assert o_readers[q] == 0, f"O{q} overwritten before the epilogue read item {o_unread[q]}"
                            o_state[q] = (item, 1)
                        else:
                            assert o_state[q] == (item, i), f"PV accumulates onto {o_state[q]}"
                            o_state[q] = (item, i + 1)
                    ring_readers[slot] -= 1
                pipe.append(("mma", run))

            def pv(q, slot, item, i):
                if self.pair:
                    yield ("wait", B[("P_HALF", q)], hphase[q])
                    hphase[q] += 1
                else:
                    yield ("wait", B[("P_FULL", q)], pphase[q])
                    pphase[q] += 1
                if i == 0 and o_done[q] > 0:
                    yield ("wait", B[("O_EMPTY", q)], o_done[q] - 1)
                if self.pair:
                    issue_pv(q, slot, item, i, 1)
                    yield ("wait", B[("P_FULL", q)], pphase[q])
                    pphase[q] += 1
                    issue_pv(q, slot, item, i, 2)
                else:
                    issue_pv(q, slot, item, i, 2)

            def commit(bar):
                pipe.append(("commit", bar))

            def commit_o(q, item):
                def mark():
                    o_unread[q] = item
                    o_readers[q] = 4
                pipe.append(("mma", mark))
                commit(B[("O_FULL", q)])
                o_done[q] += 1

            for pos, item in enumerate(items):
                has_next = pos + 1 < len(items)
                nxt = items[pos + 1] if has_next else None
                if self.pair:
                    n = cnt(item, 0)
                    was_primed, primed[0], primed[1] = primed[0], False, False
                    if n == 0:
                        continue
                    if not was_primed:
                        yield from wait_q(0)
                        yield from wait_q(1)
                        ks = []
                        yield from acquire(ks)
                        issue_qk(0, ks[0], item, 0); commit(B[("S_FULL", 0)])
                        issue_qk(1, ks[0], item, 0); commit(B[("S_FULL", 1)])
                        commit(B[("KV_EMPTY", ks[0])])
                        if n == 1:
                            commit(B[("Q_EMPTY", 0)]); commit(B[("Q_EMPTY", 1)])
                    for i in range(n):
                        more = i + 1 < n
                        prime = (not more) and has_next and cnt(nxt, 0) > 0
                        vs, ks = [], []
                        yield from acquire(vs)
                        yield from pv(0, vs[0], item, i)
                        if more:
                            yield from acquire(ks)
                            issue_qk(0, ks[0], item, i + 1); commit(B[("S_FULL", 0)])
                        else:
                            commit_o(0, item)
                            if prime:
                                yield from wait_q(0)
                                yield from acquire(ks)
                                issue_qk(0, ks[0], nxt, 0); commit(B[("S_FULL", 0)])
                        yield from pv(1, vs[0], item, i)
                        commit(B[("KV_EMPTY", vs[0])])
                        if more:
                            issue_qk(1, ks[0], item, i + 1); commit(B[("S_FULL", 1)])
                            commit(B[("KV_EMPTY", ks[0])])
                            if i + 2 == n:
                                commit(B[("Q_EMPTY", 0)]); commit(B[("Q_EMPTY", 1)])
                        else:
                            commit_o(1, item)
                            if prime:
                                yield from wait_q(1)
                                issue_qk(1, ks[0], nxt, 0); commit(B[("S_FULL", 1)])
                                commit(B[("KV_EMPTY", ks[0])])
                                if cnt(nxt, 0) == 1:
                                    commit(B[("Q_EMPTY", 0)]); commit(B[("Q_EMPTY", 1)])
                                primed[0] = primed[1] = True
                else:
                    was_primed = list(primed)
                    primed[0] = primed[1] = False
                    for q in range(2):
                        if cnt(item, q) > 0 and not was_primed[q]:
                            yield from wait_q(q)
                            ks = []
                            yield from acquire(ks)
                            issue_qk(q, ks[0], item, 0); commit(B[("S_FULL", q)])
                            commit(B[("KV_EMPTY", ks[0])])
                            if cnt(item, q) == 1:
                                commit(B[("Q_EMPTY", q)])
                    for i in range(max(cnt(item, 0), cnt(item, 1))):
                        for q in range(2):
                            if i < cnt(item, q):
                                vs, ks = [], []
                                yield from acquire(vs)
                                yield from pv(q, vs[0], item, i)
                                commit(B[("KV_EMPTY", vs[0])])
                                if i + 1 < cnt(item, q):
                                    yield from acquire(ks)
                                    issue_qk(q, ks[0], item, i + 1); commit(B[("S_FULL", q)])
                                    commit(B[("KV_EMPTY", ks[0])])
                                    if i + 2 == cnt(item, q):
                                        commit(B[("Q_EMPTY", q)])
                                else:
                                    commit_o(q, item)
                                    if has_next and cnt(nxt, q) > 0:
                                        yield from wait_q(q)
                                        yield from acquire(ks)
                                        issue_qk(q, ks[0], nxt, 0); commit(B[("S_FULL", q)])
                                        commit(B[("KV_EMPTY", ks[0])])
                                        if cnt(nxt, q) == 1:
                                            commit(B[("Q_EMPTY", q)])
                                        primed[q] = True

        # -------------------------------------------------------------- softmax warp w of stream q
        def softmax(q, w):
            sphase, handed = 0, 0
            for item in items:
                if not valid(item, q):
                    continue
                if cnt(item, q) == 0:
                    if w == 0:
                        stored[(item, q)] = stored.get((item, q), 0) + 1      # zeros and -inf written directly
                    continue
                for i in range(cnt(item, q)):
                    yield ("wait", B[("S_FULL", q)], sphase)
                    sphase += 1
                    assert s_version[q] == (item, i), f"softmax {q}.{w} expects scores of {(item, i)}, S holds {s_version[q]}"
                    if i > 0:
                        assert o_state[q] == (item, i), f"rescale of O{q} while PV of tile {i - 1} is outstanding: {o_state[q]}"
                    s_reading[q][w] = (item, i)
                    yield ("step",)
                    if self.pair:
                        p_ready[q][w] = (item, i, 1)
                        yield ("arrive", B[("P_HALF", q)])
                        yield ("step",)
                    p_ready[q][w] = (item, i, 2)
                    s_reading[q][w] = None
                    yield ("arrive", B[("P_FULL", q)])
                if handed > 0:
                    yield ("wait", B[("STATS_EMPTY", q)], handed - 1)
                assert not stats_unread[q][w], f"row statistics of stream {q} overwritten before the epilogue read them"
                handed += 1
                stats_unread[q][w] = True
                if w == 0:
                    stats_item[q] = item
                yield ("arrive", B[("STATS_FULL", q)])

        # -------------------------------------------------------------- epilogue warp w
        def epilogue(w):
            done = [0, 0]
            for item in items:
                for q in range(2):
                    if not valid(item, q) or cnt(item, q) == 0:
                        continue
                    yield ("wait", B[("STATS_FULL", q)], done[q])
                    yield ("wait", B[("O_FULL", q)], done[q])
                    done[q] += 1
                    assert stats_unread[q][w] and stats_item[q] == item, f"epilogue reads statistics of {stats_item[q]} for {item}"
                    stats_unread[q][w] = False
                    yield ("arrive", B[("STATS_EMPTY", q)])
                    assert o_state[q] == (item, cnt(item, q)) and o_unread[q] == item, \
                        f"epilogue of item {item} stream {q} finds O = {o_state[q]}, unread {o_unread[q]}"
                    yield ("step",)
                    o_readers[q] -= 1
                    yield ("arrive", B[("O_EMPTY", q)])
                    if w == 0:
                        stored[(item, q)] = stored.get((item, q), 0) + 1

        roles = [producer(), issuer()] + [softmax(q, w) for q in range(2) for w in range(4)] + [epilogue(w) for w in range(4)]
        pending = [None] * len(roles)       # the operation a role is blocked on
        alive = [True] * len(roles)
        steps = 0
        while True:
            choices = []
            for r, role in enumerate(roles):
                if not alive[r]:
                    continue
                op = pending[r]
                if op is None or op[0] != "wait" or op[1].done(op[2]):
                    choices.append(("role", r))
            if tma_inflight:
                choices.append(("tma", None))
            if pipe:
                choices.append(("pipe", None))
            if not choices:
                break
            kind, r = rng.choice(choices)
            steps += 1
            assert steps < 2_000_000, "model did not terminate"
            if kind == "tma":
                bar, where, index, tag = tma_inflight.pop(rng.randrange(len(tma_inflight)))
                if where == "ring":
                    ring[index] = tag
                else:
                    qbuf[index] = tag
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
        for item in items:
            for q in range(2):
                if valid(item, q):
                    assert stored.get((item, q), 0) == 1, f"item {item} stream {q} stored {stored.get((item, q), 0)} times"
        return stored


def make_counts(rng, n_items, topk, pair_mode, family):
    counts = []
    for i in range(n_items):
        def draw():
            if family == "uniform":
                return topk
            if family == "short":                    # the case of a bounded-wait abort found on hardware: lists of one block
                return rng.choice([0, 1, 1, 1, 2, topk])
            return rng.randint(0, topk)
        if pair_mode:
            c = draw()
            counts.append((c, c))
        else:
            last_odd = (i == n_items - 1) and rng.random() < 0.5      # odd tile count: the second stream does not exist
            counts.append((draw(), None if last_odd else draw()))
    return counts


@pytest.mark.parametrize("pair_mode", [True, False])
@pytest.mark.parametrize("family", ["uniform", "short", "ragged"])
@pytest.mark.parametrize("grid", [1, 3, 148])
def test_roles_agree_on_token_order_and_barrier_phases(pair_mode, family, grid):
    rng = random.Random(1000 * grid + 10 * len(family) + int(pair_mode))
    for trial in range(6):
        topk = rng.choice([1, 2, 3, 5, 8])
        n_items = rng.choice([1, 2, 5, 9]) * (1 if grid == 148 else grid) + rng.randrange(grid if grid < 148 else 1)
        n_items = max(1, min(n_items, 40)) if grid != 148 else rng.choice([1, 7, 148, 300])
        counts = make_counts(rng, n_items, topk, pair_mode, family)
        model = Model(counts, pair_mode, grid, rng)
        produced = {}
        for cta in range(min(grid, n_items)):
            produced.update(model.run_cta(cta))
        expected = {(i, q) for i in range(n_items) for q in range(2) if counts[i][q] is not None}
        assert set(produced) == expected            # every (batch, head, tile) once, by exactly one CTA


def test_model_catches_a_missing_release():
    """The model must be able to fail: drop the statistics release barrier (the bug once found on
    hardware with lists of one block) and a hazard or a phase alias has to show up."""
    rng = random.Random(5)
    hits = 0
    for trial in range(30):
        counts = [(1, 1)] * 6
        model = Model(counts, True, 1, rng)
        original = Bar.done

        def done_without_stats_empty(self, k):
            if self.name.startswith("STATS_EMPTY"):
                return True
            return original(self, k)
        Bar.done = done_without_stats_empty
        try:
            model.run_cta(0)
        except AssertionError:
            hits += 1
        finally:
            Bar.done = original
    assert hits > 0
