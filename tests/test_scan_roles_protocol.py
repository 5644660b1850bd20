"""The scans' role protocol as a small model, explored over every interleaving.

The walk kernels (``gdn_fwd_h_kernel``, ``gdn_bwd_dh_kernel``) are warp-specialised: epilogue threads, one or two
MMA-issuing threads and a copy thread meet on mbarriers only.  An mbarrier wait names its phase by parity, so a waiter
that looks after the barrier has completed twice since its last look misses its phase for good.  This test restates
each role's sequence of arrivals, commits and waits per chunk step (in the order the kernels execute them), lets every
asynchronous completion (a product's commit, a tile copy) happen at any later time, and checks over all interleavings

* that no wait can ever find its barrier two or more phases ahead (the phase it names is the one it gets), and
* that the roles never block one another for good.

It also checks that the protocol WITHOUT the copy thread's "seen" arrival (the form the kernels had before it) is
caught: there the wait for a free stage is safe only by timing.  The model is host-side bookkeeping only: no kernel
runs here, and a change of the kernels' synchronisation has to be restated in ``_roles`` below.
"""

from __future__ import annotations

import pytest

STEPS = 5


def _roles(kernel: str, fused: bool, tapes: bool, seen: bool):
    """{role: [op, ...]} with ops ("wait", barrier, phase), ("arrive", barrier), ("commit", barrier) -- an arrival
    that happens once the role's earlier products are done, in order -- and ("load", barrier): a copy whose completion
    is the barrier's arrival.  Also {barrier: arrivals per phase}."""
    S = STEPS
    fwd = kernel == "fwd"
    fused = fused and fwd
    free_x = "bar_free_vn" if fwd else "bar_free_dv"
    stage_free = "bar_o" if fused else "bar_d2"  # what the copy thread waits on before it refills a stage
    counts = {name: 1 for name in ("bar_load0", "bar_load1", "bar_h", "bar_vs", "bar_d1", "bar_d2", "bar_o",
                                   "bar_free_h", free_x, "bar_out", "bar_free_o", "bar_seen")}
    if not fwd:
        counts["bar_d1"] = 2  # one commit per issuing thread
    epilogue, issuer, issuer2, mover = [], [], [], [("load", "bar_load0")]
    for s in range(S):
        # --- epilogue threads (one agent: they all arrive on the same barriers) ------------------------------------
        epilogue += [("wait", f"bar_load{s & 1}", s >> 1), ("arrive", "bar_h")]
        if fused and s > 0:
            epilogue.append(("wait", "bar_o", s - 1))  # the previous chunk's output products
            if s > 1:
                epilogue.append(("wait", "bar_free_o", s - 2))  # the store of the tile before this one
        epilogue.append(("wait", "bar_h", s))
        if tapes and s > 0:
            epilogue.append(("wait", free_x, s - 1))
        if seen:
            epilogue.append(("wait", "bar_seen", s))
        epilogue += [("wait", "bar_d1", s), ("arrive", "bar_vs")]
        if fused and s > 0:
            epilogue.append(("arrive", "bar_out"))
        if tapes:
            epilogue.append(("wait", "bar_free_h", s))
        epilogue.append(("wait", "bar_d2", s))
        # --- issuing thread(s) -----------------------------------------------------------------------------------------
        issuer += [("wait", "bar_h", s), ("commit", "bar_d1"), ("wait", "bar_vs", s), ("commit", "bar_d2")]
        if fused:
            issuer.append(("commit", "bar_o"))
        if not fwd:
            issuer2 += [("wait", "bar_h", s), ("commit", "bar_d1")]
        # --- copy thread -------------------------------------------------------------------------------------------------
        if s + 1 < S:
            if s > 0:
                mover.append(("wait", stage_free, s - 1))
            mover.append(("load", f"bar_load{(s + 1) & 1}"))
        if seen:
            mover.append(("arrive", "bar_seen"))
        if tapes:
            mover += [("wait", "bar_h", s), ("arrive", "bar_free_h")]
        if seen or tapes:
            mover.append(("wait", "bar_vs", s))
        if tapes:
            mover.append(("arrive", free_x))
            if fused and s > 0:
                mover += [("wait", "bar_out", s - 1), ("arrive", "bar_free_o")]
    roles = {"epilogue": epilogue, "issuer": issuer, "mover": mover}
    if issuer2:
        roles["issuer2"] = issuer2
    return roles, counts


def _explore(roles, counts):
    """Every interleaving.  Returns (missed, stuck): the first wait found two phases behind its barrier, and whether
    some reachable state has unfinished roles and nothing enabled."""
    names = sorted(roles)
    bars = sorted(counts)
    index = {b: i for i, b in enumerate(bars)}

    def arrive(state_bars, b):
        got, done = state_bars[index[b]]
        got += 1
        if got == counts[b]:
            got, done = 0, done + 1
        out = list(state_bars)
        out[index[b]] = (got, done)
        return tuple(out)

    start = (tuple(0 for _ in names), tuple((0, 0) for _ in bars), tuple(() for _ in names), ())
    seen_states = {start}
    todo = [start]
    missed = None
    stuck = False
    while todo:
        pcs, state_bars, commits, loads = todo.pop()
        moves = []
        unfinished = False
        for r, name in enumerate(names):
            prog = roles[name]
            if pcs[r] >= len(prog):
                continue
            unfinished = True
            op = prog[pcs[r]]
            step = tuple(p + (1 if i == r else 0) for i, p in enumerate(pcs))
            if op[0] == "wait":
                done = state_bars[index[op[1]]][1]
                if done >= op[2] + 2 and missed is None:
                    missed = (name, op, done)
                if done % 2 != op[2] % 2:  # the hardware's test: the phase of this parity has completed
                    moves.append((step, state_bars, commits, loads))
            elif op[0] == "arrive":
                moves.append((step, arrive(state_bars, op[1]), commits, loads))
            elif op[0] == "commit":  # completes later, after the role's earlier commits
                queued = tuple(q + ((op[1],) if i == r else ()) for i, q in enumerate(commits))
                moves.append((step, state_bars, queued, loads))
            else:  # a copy: completes at any later time
                moves.append((step, state_bars, commits, tuple(sorted(loads + (op[1],)))))
        for r, queue in enumerate(commits):
            if queue:
                rest = tuple(q[1:] if i == r else q for i, q in enumerate(commits))
                moves.append((pcs, arrive(state_bars, queue[0]), rest, loads))
        for i, b in enumerate(loads):
            moves.append((pcs, arrive(state_bars, b), commits, loads[:i] + loads[i + 1:]))
        if unfinished and not moves:
            stuck = True
        for m in moves:
            if m not in seen_states:
                seen_states.add(m)
                todo.append(m)
    return missed, stuck


@pytest.mark.parametrize("kernel,fused,tapes", [
    ("fwd", True, True),    # the walk with the output fused in
    ("fwd", False, True),   # the walk that writes the tapes only
    ("fwd", False, False),  # a pre-scan: no tape, no output
    ("bwd", False, True),
    ("bwd", False, False),
])
def test_no_wait_can_miss_its_phase_and_no_role_blocks_for_good(kernel, fused, tapes):
    missed, stuck = _explore(*_roles(kernel, fused, tapes, seen=True))
    assert missed is None, f"{missed[0]} waits for phase {missed[1][2]} of {missed[1][1]} which has completed {missed[2]} times"
    assert not stuck


@pytest.mark.parametrize("kernel,fused,tapes", [("fwd", True, True), ("fwd", False, False), ("bwd", False, True)])
def test_without_the_seen_arrival_the_stage_wait_is_safe_by_timing_only(kernel, fused, tapes):
    missed, _ = _explore(*_roles(kernel, fused, tapes, seen=False))
    assert missed is not None and missed[0] == "mover"
    assert missed[1][1] == ("bar_o" if fused else "bar_d2")
