"""CPU: host-side rules of the escape-time launcher, restated and checked exhaustively.

The first is the rule by which escape_time launches that were declared independent of their predecessors
are grouped into runs (vernondsl_b200/csrc/k_escape.cu, launch_escape_time).

A launch declares k: it touches nothing the k escape_time launches before it on its stream write.
The launcher starts a launch "overlapped" (it may begin before the launch before it ends) only inside
a run; since a grid of a run never completes before the grid before it, a launch of a run may in
principle run beside EVERY earlier launch of the same run, and beside nothing else.  The property
that makes this safe: every earlier launch of the run is one the launch was declared independent of.
"""
import itertools


def plan(events):
    """events: k (0..7) for an escape_time launch, or 'x' for anything else the library sees on the stream.
    Returns per launch (index into events) a tuple (overlapped, counter slot, index of the run's first launch)."""
    out = {}
    run = 0          # launches of the current run so far (the stream's escape_chain)
    first = None
    for i, e in enumerate(events):
        if e == "x":
            run = 0
            continue
        overlapped = e != 0 and 1 <= run <= e and run < 8
        if not overlapped:
            first = i
        out[i] = (overlapped, run if overlapped else 0, first)
        run = 0 if e == 0 else run + 1 if overlapped else 1
    return out


def check(events):
    got = plan(events)
    launches = [i for i, e in enumerate(events) if e != "x"]
    for i, (overlapped, slot, first) in got.items():
        assert 0 <= slot < 8
        if not overlapped:
            assert slot == 0
            continue
        beside = [j for j in launches if first <= j < i]
        # nothing but escape_time launches lies between the run's first launch and this one
        assert all(events[j] != "x" for j in range(first, i))
        assert len(beside) == i - first
        # every launch it may run beside is among the k launches before it ...
        assert len(beside) <= events[i], (events, i)
        # ... and takes its work from another counter
        assert len({got[j][1] for j in beside} | {slot}) == len(beside) + 1
    # a launch that declares nothing is never overlapped and nothing after it overlaps it
    for i in launches:
        if events[i] == 0:
            assert not got[i][0]
            assert all(got[j][2] > i for j in launches if j > i)


def test_every_overlapped_launch_only_runs_beside_launches_it_was_declared_independent_of():
    for n in range(1, 8):
        for events in itertools.product([0, 1, 2, 3, "x"], repeat=n):
            check(events)
    for events in itertools.product([0, 7, 5], repeat=10):
        check(events)


def test_a_ring_of_four_orders_every_fourth_launch():
    got = plan([3] * 12)
    assert [got[i][0] for i in range(12)] == [False, True, True, True] * 3
    assert [got[i][1] for i in range(12)] == [0, 1, 2, 3] * 3
    got = plan([7] * 17)
    assert [i for i in range(17) if not got[i][0]] == [0, 8, 16]
    got = plan([1] * 6)
    assert [got[i][0] for i in range(6)] == [False, True] * 3
    # anything else on the stream ends the run
    got = plan([3, 3, "x", 3, 3])
    assert [got[i][0] for i in (0, 1, 3, 4)] == [False, True, False, True]


def test_rows_visited_from_the_middle_outwards_are_each_visited_once():
    """The order in which a launch of the work-stealing kernel visits its rows (middle_out in
    vernondsl_b200/csrc/escape_common.cuh), restated: a permutation for every row count, middle first."""
    def middle_out(k, rows):
        mid, h = rows >> 1, (k + 1) >> 1
        if k & 1:
            return mid - h if h <= mid else k
        return mid + h if mid + h < rows else rows - 1 - k

    for rows in list(range(1, 600)) + [1080, 2048, 16384]:
        order = [middle_out(k, rows) for k in range(rows)]
        assert sorted(order) == list(range(rows)), rows
        assert order[0] == rows // 2
        # distance from the middle never shrinks by more than one row from one visit to the next
        dist = [abs(r - rows // 2) for r in order]
        assert all(b >= a - 1 for a, b in zip(dist, dist[1:])), rows
    assert [middle_out(k, 7) for k in range(7)] == [3, 2, 4, 1, 5, 0, 6]
