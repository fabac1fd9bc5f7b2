"""A model of the peer-memory exchange protocol (``parallel/fused_exchange.py``), checked over ALL interleavings of the ranks.

Every rank runs the same sequential program per step; the only synchronisation is the epoch flags (a rank may pass a wait
when every peer's flag for that channel has reached the step's epoch). Buffers carry a tag (writer, step) so that every read
can assert that it sees exactly the data of its own step: a write that could land too early (overwriting data a slower peer
has not consumed yet) or too late shows up as an assertion in some interleaving. The explorer walks the whole state graph
(memoised), so a property that holds here holds for any relative speed of the ranks; it also proves that the program cannot
deadlock. The lagging-optimizer variant models gradient accumulation, where a staged gradient window is consumed at the start
of the next forward pass."""
import itertools

import pytest

IDS, EMB, GRAD = 0, 1, 2


def program(steps, flush_late):
    """The action list of one rank. ``flush_late``: the owner consumes the gradients of step t only at the start of step t+1."""
    prog = []
    for t in range(steps):
        if flush_late and t > 0:
            prog += [("wait", GRAD, t - 1), ("reduce", t - 1)]
        prog += [("write_ids", t), ("signal", IDS, t), ("wait", IDS, t), ("pull", t), ("push", t), ("signal", EMB, t),
                 ("wait", EMB, t), ("pool", t), ("grad_push", t), ("signal", GRAD, t)]
        if not flush_late:
            prog += [("wait", GRAD, t), ("reduce", t)]
    if flush_late:
        prog += [("wait", GRAD, steps - 1), ("reduce", steps - 1)]
    return prog


def explore(world, steps, flush_late=False, broken=None):
    prog = program(steps, flush_late)
    if broken == "no_emb_wait":            # a deliberately wrong protocol, to show that the checker can see a hazard
        prog = [a for a in prog if not (a[0] == "wait" and a[1] == EMB)]
    n = len(prog)
    W = world
    # state: pcs, flags[ch][dst][src], ids[r], uemb[dst][src], gin[dst][src]  (tags are step numbers, -1 = never written)
    init = (tuple([0] * W), tuple([-1] * (3 * W * W)), tuple([-1] * W), tuple([-1] * (W * W)), tuple([-1] * (W * W)))
    seen, stack, violations = {init}, [init], []
    finished = False
    while stack:
        pcs, flags, ids, uemb, gin = stack.pop()
        if all(pc == n for pc in pcs):
            finished = True
            continue
        progressed = False
        for r in range(W):
            if pcs[r] == n:
                continue
            act = prog[pcs[r]]
            kind = act[0]
            f, i_, u, g = list(flags), list(ids), list(uemb), list(gin)
            if kind == "wait":
                ch, t = act[1], act[2]
                if any(flags[(ch * W + r) * W + p] < t for p in range(W)):
                    continue                                     # blocked
            elif kind == "signal":
                ch, t = act[1], act[2]
                for p in range(W):
                    f[(ch * W + p) * W + r] = t
            elif kind == "write_ids":
                i_[r] = act[1]
            elif kind == "pull":
                for p in range(W):
                    if ids[p] != act[1]:
                        violations.append(("pull", r, p, act[1], ids[p]))
            elif kind == "push":
                for p in range(W):
                    u[p * W + r] = act[1]
            elif kind == "pool":
                for p in range(W):
                    if uemb[r * W + p] != act[1]:
                        violations.append(("pool", r, p, act[1], uemb[r * W + p]))
            elif kind == "grad_push":
                for o in range(W):
                    g[o * W + r] = act[1]
            elif kind == "reduce":
                for p in range(W):
                    if gin[r * W + p] != act[1]:
                        violations.append(("reduce", r, p, act[1], gin[r * W + p]))
            progressed = True
            nxt = (tuple(pc + 1 if k == r else pc for k, pc in enumerate(pcs)), tuple(f), tuple(i_), tuple(u), tuple(g))
            if nxt not in seen:
                seen.add(nxt)
                stack.append(nxt)
        if not progressed:
            violations.append(("deadlock", pcs))
        if violations:
            break
    return finished, violations, len(seen)


@pytest.mark.parametrize("world,steps", [(2, 3), (3, 2)])
def test_protocol_is_safe_and_live_under_every_interleaving(world, steps):
    finished, violations, states = explore(world, steps)
    assert finished and not violations, violations[:3]
    assert states > 100                                       # the ranks really do interleave


def test_lagging_optimizer_consumes_gradients_before_the_window_is_rewritten():
    finished, violations, _ = explore(2, 3, flush_late=True)
    assert finished and not violations, violations[:3]


def test_checker_detects_a_missing_wait():
    finished, violations, _ = explore(2, 2, broken="no_emb_wait")
    assert violations and violations[0][0] in ("pool", "pull", "reduce")
