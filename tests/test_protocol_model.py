"""Exhaustive interleaving check of the flag protocol of the pipelined collectives (a model, no GPU).

The kernels in csrc/kernels/collectives.cu split a grid into link CTAs (push sub-chunk c, then raise flag c+1 on
every peer) and local CTAs (wait for flag c+1 of every link CTA of every source, then consume sub-chunk c; in the
three-phase kinds: combine, raise an own flag, and collect sub-chunk c-1 once every peer's local CTAs raised theirs).
This test runs that state machine for 2-3 ranks, 1-2 link CTAs, 1-2 local CTAs and 1-3 sub-chunks under EVERY
interleaving of the CTAs' steps and checks that no consumer ever reads a sub-chunk that has not been fully written
and that every schedule terminates (no deadlock).  Steps are atomic and sequentially consistent: the model checks the
indices, counts and flag values of the protocol, not the memory model (release/acquire pairs carry that on the GPU)."""
import itertools

import pytest


def _programs(n, L, NL, chunks, depth):
    """One step list per CTA of every rank.  Steps are tuples interpreted by _run."""
    progs = {}
    for r in range(n):
        for x in range(L):
            steps = []
            for c in range(chunks):
                steps.append(("push", c))          # this link CTA's share of sub-chunk c to every peer
                steps.append(("post", c + 1))      # flag slot x on every peer
            progs[(r, x)] = steps
        for y in range(L, L + NL):
            steps = []
            for c in range(chunks):
                steps.append(("wait_links", c + 1))
                if depth == 2:
                    steps.append(("pull", c))
                else:
                    steps.append(("combine", c))   # reads the slices, writes results to every peer
                    steps.append(("post", c + 1))  # flag slot y on every peer
                    if c >= 1:
                        steps.append(("wait_locals", c))
                        steps.append(("collect", c - 1))
            if depth == 3:
                steps.append(("wait_locals", chunks))
                steps.append(("collect", chunks - 1))
            progs[(r, y)] = steps
    return progs


def _explore(n, L, NL, chunks, depth):
    progs = _programs(n, L, NL, chunks, depth)
    agents = sorted(progs)
    # state: pc per agent, flags[(on_rank, slot, from_rank)] = value, pushed[(dst, src, x, c)], results[(dst, src, y, c)]
    start = (tuple(0 for _ in agents), frozenset(), frozenset(), frozenset())
    seen, stack, terminal = {start}, [start], 0
    while stack:
        pcs, flags, pushed, results = stack.pop()
        fl = dict(flags)
        moved = False
        for i, (r, slot) in enumerate(agents):
            if pcs[i] >= len(progs[(r, slot)]):
                continue
            op, arg = progs[(r, slot)][pcs[i]]
            nf, npu, nre = fl, pushed, results
            if op == "push":
                npu = pushed | {(p, r, slot, arg) for p in range(n) if p != r}
            elif op == "post":
                nf = dict(fl)
                for p in range(n):
                    if p != r:
                        assert nf.get((p, slot, r), 0) < arg, "flag values must grow"
                        nf[(p, slot, r)] = arg
            elif op == "wait_links":
                if not all(fl.get((r, x, p), 0) >= arg for x in range(L) for p in range(n) if p != r):
                    continue  # blocked
            elif op == "wait_locals":
                if not all(fl.get((r, y, p), 0) >= arg for y in range(L, L + NL) for p in range(n) if p != r):
                    continue
            elif op in ("pull", "combine"):
                for p in range(n):
                    if p != r:
                        for x in range(L):
                            assert (r, p, x, arg) in pushed, f"rank {r} consumed sub-chunk {arg} of rank {p} before link CTA {x} wrote it"
                if op == "combine":
                    nre = results | {(p, r, slot, arg) for p in range(n) if p != r}
            elif op == "collect":
                for p in range(n):
                    if p != r:
                        for y in range(L, L + NL):
                            assert (r, p, y, arg) in results, f"rank {r} collected result {arg} of rank {p} before its CTA {y} wrote it"
            moved = True
            npcs = pcs[:i] + (pcs[i] + 1,) + pcs[i + 1:]
            st = (npcs, frozenset(nf.items()), npu, nre)
            if st not in seen:
                seen.add(st)
                stack.append(st)
        if not moved:
            assert all(pcs[i] >= len(progs[a]) for i, a in enumerate(agents)), f"deadlock at {pcs}"
            terminal += 1
    return len(seen), terminal


@pytest.mark.parametrize("n,L,NL,chunks,depth", [(2, 1, 1, 3, 2), (2, 2, 1, 2, 2), (3, 1, 1, 2, 2), (2, 1, 1, 3, 3), (2, 1, 2, 2, 3),
                                                 (3, 1, 1, 2, 3)])
def test_flag_protocol_has_no_early_read_and_no_deadlock(n, L, NL, chunks, depth):
    states, terminal = _explore(n, L, NL, chunks, depth)
    assert states > 10 and terminal >= 1


def _explore_unified(n, chunks, depth):
    """The NVLS kinds keep one role per CTA and the unit-ownership rule: CTA x of every rank runs
    A(i); wait(peers finished iteration i-1); B(i-1); [C(i-2)]; post(i+1).  One CTA index suffices for the model."""
    iters = chunks + depth - 1
    progs = {}
    for r in range(n):
        steps = []
        for i in range(iters):
            if i < chunks:
                steps.append(("A", i))
            if i >= 1:
                steps.append(("wait", i))
                if i - 1 < chunks:
                    steps.append(("B", i - 1))
            if depth == 3 and i >= 2 and i - 2 < chunks:
                steps.append(("C", i - 2))
            if i + 1 < iters:
                steps.append(("post", i + 1))
        progs[r] = steps
    start = (tuple(0 for _ in range(n)), tuple(0 for _ in range(n)), frozenset(), frozenset())
    seen, stack, terminal = {start}, [start], 0
    while stack:
        pcs, posted, doneA, doneB = stack.pop()
        moved = False
        for r in range(n):
            if pcs[r] >= len(progs[r]):
                continue
            op, arg = progs[r][pcs[r]]
            np_, nA, nB = posted, doneA, doneB
            if op == "A":
                nA = doneA | {(r, arg)}
            elif op == "post":
                assert posted[r] < arg
                np_ = posted[:r] + (arg,) + posted[r + 1:]
            elif op == "wait":
                if not all(posted[p] >= arg for p in range(n) if p != r):
                    continue
            elif op == "B":
                assert all((p, arg) in doneA for p in range(n)), f"rank {r} reduced sub-chunk {arg} before every rank staged it"
                nB = doneB | {(r, arg)}
            elif op == "C":
                assert all((p, arg) in doneB for p in range(n)), f"rank {r} copied out sub-chunk {arg} before every rank finished it"
            moved = True
            st = (pcs[:r] + (pcs[r] + 1,) + pcs[r + 1:], np_, nA, nB)
            if st not in seen:
                seen.add(st)
                stack.append(st)
        if not moved:
            assert all(pcs[r] >= len(progs[r]) for r in range(n)), f"deadlock at {pcs}"
            terminal += 1
    return len(seen), terminal


@pytest.mark.parametrize("n,chunks,depth", [(2, 1, 2), (2, 4, 2), (3, 3, 2), (2, 1, 3), (2, 4, 3), (3, 3, 3)])
def test_split_phase_pipeline_of_the_switch_kinds(n, chunks, depth):
    states, terminal = _explore_unified(n, chunks, depth)
    assert states > 3 and terminal >= 1
