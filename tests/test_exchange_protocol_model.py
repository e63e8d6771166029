"""CPU: the ordering rules of the image exchange (vrhi_exchange_*), checked over EVERY interleaving.

A GPU test runs the interleavings the hardware happens to produce.  This is a small model of the
protocol for two ranks: what each rank's three streams do per group (compute, send + raise the
sequence number, wait + widen), the orderings the library enforces (stream order, the events behind
which sends and widenings are enqueued, the flag a widening waits for, `complete` gating the next
step), and wire images that are plain arrays.  A search visits every reachable state and checks
that a widening of step s only ever reads counts of step s: from its own wire image (what the peer
sent) and, in the squeezed form, from the owner's wire image over the link.

With two wire images in turn the property holds in every interleaving.  With one (the form an
earlier version of the gather had) the search finds the interleaving in which a fast rank's rows of
the next step land before the slow rank has widened the previous ones."""
import pytest


def explore(steps, groups, n_wires, remote_fetch):
    """Depth-first over all interleavings.  Returns None if the property always holds, else a description
    of the first violation.  State per rank: ops done on the compute, send and widen streams (each
    stream's ops are k = step * groups + group, in order) and the contents of its wire images:
    wire[b][owner][group] = step whose counts are stored there (-1: none yet)."""
    total = steps * groups
    start = ((0, 0, 0), (0, 0, 0),
             tuple(tuple(tuple(-1 for _ in range(groups)) for _ in range(2)) for _ in range(n_wires)),
             tuple(tuple(tuple(-1 for _ in range(groups)) for _ in range(2)) for _ in range(n_wires)))
    seen, stack = {start}, [start]

    def put(wire, b, owner, g, value):
        w = [list(map(list, plane)) for plane in wire]
        w[b][owner][g] = value
        return tuple(tuple(map(tuple, plane)) for plane in w)

    while stack:
        state = stack.pop()
        prog, wires = [list(state[0]), list(state[1])], [state[2], state[3]]
        for r in (0, 1):
            peer = 1 - r
            c, p, w = prog[r]
            nxt = []
            # compute op k: own rows of group g of step s into the step's wire image; the first group of a step
            # is ordered behind `complete` of the step before (all of that step's widenings and sends of this rank)
            if c < total:
                s, g = divmod(c, groups)
                if g > 0 or s == 0 or (w >= s * groups and p >= s * groups):
                    nw = put(wires[r], s % n_wires, r, g, s)
                    nxt.append(((c + 1, p, w), nw, wires[peer]))
            # send op k: behind compute op k; copies the rows into the same place of the peer's wire image, then the flag
            if p < total and c > p:
                s, g = divmod(p, groups)
                b = s % n_wires
                value = wires[r][b][r][g]
                if value != s:
                    return f"rank {r} sends group {g} of step {s} but its own wire image holds step {value} there"
                nxt.append(((c, p + 1, w), wires[r], put(wires[peer], b, r, g, value)))
            # widen op k: behind compute op k of this rank (the event it is enqueued behind) and the peer's flag for k
            if w < total and c > w and prog[peer][1] > w:
                s, g = divmod(w, groups)
                b = s % n_wires
                got = wires[r][b][peer][g]
                if got != s:
                    return f"rank {r} widens group {g} of step {s} and reads counts of step {got} from its wire image"
                if remote_fetch and wires[peer][b][peer][g] != s:
                    return f"rank {r} widens group {g} of step {s} and fetches counts of step {wires[peer][b][peer][g]} from the owner"
                nxt.append(((c, p, w + 1), wires[r], wires[peer]))
            for new_prog, own_wire, peer_wire in nxt:
                progs, ws = [None, None], [None, None]
                progs[r], progs[peer] = new_prog, tuple(prog[peer])
                ws[r], ws[peer] = own_wire, peer_wire
                new_state = (progs[0], progs[1], ws[0], ws[1])
                if new_state not in seen:
                    seen.add(new_state)
                    stack.append(new_state)
    done = ((total,) * 3, (total,) * 3)
    assert any(s[0] == done[0] and s[1] == done[1] for s in seen), "the model deadlocks: no interleaving finishes"
    return None


@pytest.mark.parametrize("remote_fetch", [False, True])
@pytest.mark.parametrize("steps,groups", [(3, 2), (4, 1), (3, 3)])
def test_two_wire_images_are_safe_in_every_interleaving(steps, groups, remote_fetch):
    assert explore(steps, groups, n_wires=2, remote_fetch=remote_fetch) is None


def test_one_wire_image_is_not():
    """The negative control, and the reason the exchange alternates two wire images."""
    found = explore(3, 2, n_wires=1, remote_fetch=False)
    assert found is not None and "reads counts of step" in found
