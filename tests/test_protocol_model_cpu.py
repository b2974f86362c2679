"""Exhaustive interleaving check of the epoch-flag protocols that the in-kernel collectives use
(csrc/comm.cu, csrc/gemm_sm100.cu / gemm2_sm100.cu coupling, parallel/tp_native.py, serve/tp.py).

Each rank is a straight-line program of atomic steps over a shared memory of symmetric buffers
and flags; a wait is a step that is enabled only when its predicate holds.  The checker walks
every interleaving (states are memoised) and reports

* a *violation* - a read that sees anything but the value its call must see (a buffer reused
  before its reader was done, a counter cleared under an arrival), and
* a *deadlock* - a state in which some rank is unfinished and no step is enabled.

The protocols as built pass for 2 and 3 ranks over several calls; each is also run with one rule
removed (the back-pressure wait, the second parity, the order of clear and release) to show that
the model is able to find the failure that rule prevents.

Data writes and the flag write that publishes them are separate steps in program order, which is
what the kernels guarantee with a system fence + release store; flags only grow (epochs), except
the arrival counters of the reduce-scatter, which their owner clears.
"""
from __future__ import annotations

from typing import Callable, Optional

import pytest

Step = tuple[str, Callable[[dict], object]]      # ("wait", predicate) | ("do", action) ; an action may return an error string


def explore(programs: list[list[Step]], init: dict) -> Optional[str]:
    """Depth-first walk over all interleavings.  Returns None, or a description of the first
    violation / deadlock found."""
    n = len(programs)
    seen = set()
    stack = [((0,) * n, init)]
    while stack:
        pcs, mem = stack.pop()
        key = (pcs, tuple(sorted(mem.items())))
        if key in seen:
            continue
        seen.add(key)
        if all(pcs[r] == len(programs[r]) for r in range(n)):
            continue
        progressed = False
        for r in range(n):
            if pcs[r] == len(programs[r]):
                continue
            kind, fn = programs[r][pcs[r]]
            if kind == "wait":
                if not fn(mem):
                    continue
                nxt = mem
            else:
                nxt = dict(mem)
                err = fn(nxt)
                if err:
                    return f"violation at rank {r}, step {pcs[r]}: {err}"
            progressed = True
            stack.append((pcs[:r] + (pcs[r] + 1,) + pcs[r + 1:], nxt))
        if not progressed:
            return f"deadlock at program counters {pcs}"
    return None


def g(mem: dict, key, default=0):
    return mem.get(key, default)


# ----------------------------------------------------------------------------- all-gather -> GEMM
def all_gather_programs(world: int, calls: int, back_pressure: bool = True, parities: int = 2):
    """kb_ag_push + the flag-gated GEMM producer + the `done` signal (tp_native._push / _gemm_ag /
    _ag_done): call c uses staging buffer c % 2; a rank pushes call c only after every peer has
    signalled that it finished reading call c - 2."""
    progs = []
    for r in range(world):
        p: list[Step] = []
        for c in range(1, calls + 1):
            par = c % parities
            if back_pressure and c > 2:
                p.append(("wait", lambda m, c=c, r=r: all(g(m, ("done", r, q)) >= c - 2 for q in range(world))))
            for q in range(world):                      # shard into every rank's staging buffer
                p.append(("do", lambda m, q=q, par=par, r=r, c=c: m.__setitem__(("stage", q, par, r), c)))
            for q in range(world):                      # ... then its ready flag
                p.append(("do", lambda m, q=q, par=par, r=r, c=c: m.__setitem__(("ready", q, par, r), c)))
            for s in range(world):                      # the GEMM: wait for a shard, read it
                p.append(("wait", lambda m, s=s, par=par, r=r, c=c: g(m, ("ready", r, par, s)) >= c))
                p.append(("do", lambda m, s=s, par=par, r=r, c=c:
                          None if g(m, ("stage", r, par, s)) == c else
                          f"call {c} read shard {s} of call {g(m, ('stage', r, par, s))}"))
            for q in range(world):                      # finished reading: tell every peer
                p.append(("do", lambda m, q=q, r=r, c=c: m.__setitem__(("done", q, r), c)))
        progs.append(p)
    return progs


@pytest.mark.parametrize("world,calls", [(2, 5), (3, 3)])
def test_all_gather_staging_is_never_overwritten_before_it_is_read(world, calls):
    assert explore(all_gather_programs(world, calls), {}) is None


def test_all_gather_model_shows_what_each_rule_is_for():
    # Two staging buffers are already safe when a rank's push, product and next push run in program
    # order (a rank reaches call c + 2 only after its product of c + 1, which needed every peer's push
    # of c + 1, which that peer issued after its product of c): the explicit `done` wait is a second
    # line of defence for schedules that reorder streams, not the only one.
    assert explore(all_gather_programs(2, 4, back_pressure=False), {}) is None
    # one staging buffer is not enough, with or without the two-call back-pressure
    for bp in (False, True):
        out = explore(all_gather_programs(2, 4, back_pressure=bp, parities=1), {})
        assert out is not None and "violation" in out


# ----------------------------------------------------------------------------- GEMM -> reduce-scatter
def reduce_scatter_programs(world: int, calls: int, arrivals: int = 2, clear_before_release: bool = True,
                            back_pressure: bool = True, parities: int = 2, clear: bool = True):
    """kb_gemm_rs epilogue + kb_rs_reduce (tp_native._gemm_rs): a producer stores its partial rows into
    the owner's slab for this source, then adds its arrivals to the owner's counter; the owner waits for
    `arrivals` from every source, sums, clears the counters and only then releases the slabs (`done`
    epoch on every peer); a producer starts call c only after every owner released call c - 2."""
    progs = []
    for r in range(world):
        p: list[Step] = []
        for c in range(1, calls + 1):
            par = c % parities
            if back_pressure and c > 2:
                p.append(("wait", lambda m, c=c, r=r: all(g(m, ("rs_done", r, o)) >= c - 2 for o in range(world))))
            for o in range(world):
                for a in range(arrivals):               # one arrival per epilogue warp: data, then the counter
                    p.append(("do", lambda m, o=o, par=par, r=r, c=c, a=a: m.__setitem__(("slab", o, par, r, a), c)))
                    p.append(("do", lambda m, o=o, par=par, r=r:
                              m.__setitem__(("cnt", o, par, r), g(m, ("cnt", o, par, r)) + 1)))
            # the owner half, on the same stream after the producer half
            p.append(("wait", lambda m, par=par, r=r: all(g(m, ("cnt", r, par, s)) >= arrivals for s in range(world))))
            for s in range(world):
                for a in range(arrivals):
                    p.append(("do", lambda m, s=s, par=par, r=r, c=c, a=a:
                              None if g(m, ("slab", r, par, s, a)) == c else
                              f"call {c} summed rows of call {g(m, ('slab', r, par, s, a))} from source {s}"))
            clear_steps = [("do", lambda m, s=s, par=par, r=r: m.__setitem__(("cnt", r, par, s), 0)) for s in range(world)]
            release = [("do", lambda m, q=q, r=r, c=c: m.__setitem__(("rs_done", q, r), c)) for q in range(world)]
            if not clear:
                clear_steps = []
            p.extend(clear_steps + release if clear_before_release else release + clear_steps)
        progs.append(p)
    return progs


@pytest.mark.parametrize("world,calls", [(2, 4), (3, 3)])
def test_reduce_scatter_slabs_and_counters(world, calls):
    assert explore(reduce_scatter_programs(world, calls, arrivals=2 if world == 2 else 1), {}) is None


def test_reduce_scatter_model_shows_what_each_rule_is_for():
    # With two slab sets and each rank's producer and owner halves in program order, the order of
    # "clear the counters" and "release the slabs", and the release wait itself, are second lines of
    # defence: the same chain of dependencies as in the all-gather keeps call c + 2 behind call c.
    assert explore(reduce_scatter_programs(2, 5, arrivals=1, clear_before_release=False), {}) is None
    assert explore(reduce_scatter_programs(2, 4, arrivals=1, back_pressure=False), {}) is None
    # what is needed: the second slab set, and counters that start each use at zero
    out = explore(reduce_scatter_programs(2, 4, arrivals=1, parities=1), {})
    assert out is not None and "violation" in out
    out = explore(reduce_scatter_programs(2, 4, arrivals=1, clear=False), {})
    assert out is not None and "violation" in out


# ----------------------------------------------------------------------------- push all-reduce (decode)
def push_allreduce_programs(world: int, calls: int, parities: int = 2):
    """kb_allreduce_push (serve/tp.py): call e pushes this rank's partial into slot e % 2 of every
    peer, raises the epoch flag there, waits for every source's flag and sums.  There is no explicit
    release: a rank can push call e + 2 only after it completed call e + 1, which needed every
    peer's push of e + 1, which that peer issues after it finished summing call e."""
    progs = []
    for r in range(world):
        p: list[Step] = []
        for e in range(1, calls + 1):
            par = e % parities
            for q in range(world):
                p.append(("do", lambda m, q=q, par=par, r=r, e=e: m.__setitem__(("recv", q, par, r), e)))
            for q in range(world):
                p.append(("do", lambda m, q=q, r=r, e=e: m.__setitem__(("flag", q, r), e)))
            p.append(("wait", lambda m, r=r, e=e: all(g(m, ("flag", r, s)) >= e for s in range(world))))
            for s in range(world):
                p.append(("do", lambda m, s=s, par=par, r=r, e=e:
                          None if g(m, ("recv", r, par, s)) == e else
                          f"call {e} summed the partial of call {g(m, ('recv', r, par, s))} from rank {s}"))
        progs.append(p)
    return progs


@pytest.mark.parametrize("world,calls", [(2, 6), (3, 4)])
def test_push_allreduce_two_parities_suffice(world, calls):
    assert explore(push_allreduce_programs(world, calls), {}) is None


def test_push_allreduce_model_finds_the_reuse_with_one_slot():
    out = explore(push_allreduce_programs(2, 4, parities=1), {})
    assert out is not None and "violation" in out


# ----------------------------------------------------------------------------- bounded waits
def test_a_rank_that_never_arrives_is_a_deadlock_in_the_model_and_a_timeout_in_the_kernels():
    """The model has no clock: a missing rank shows up as a deadlock.  The kernels turn exactly that
    state into status 4 after their limit (tests/test_ops_gpu.py covers the device side)."""
    progs = all_gather_programs(2, 2)
    progs[1] = []                                    # rank 1 never runs
    out = explore(progs, {})
    assert out is not None and "deadlock" in out


# ----------------------------------------------------------------------------- programmatic dependent launches
def dependent_launch_programs(k2_waits: bool = True, k3_reads_early: bool = False, k3_prefetches_weight: bool = True):
    """Three kernels on one stream, each launched as a programmatic dependent of the one before it (csrc/common.cuh:
    kb_launch_dep / kb_dep_trigger / kb_dep_wait; the decode graphs of serve/engine.py).  A kernel may START once its
    predecessor has triggered, and its wait returns once the predecessor has COMPLETED.  K1 produces x, K2 turns x into
    y, K3 reads y and x (x only through K2's completion: K3 waits for K2 alone) and may fetch a constant weight early.
    Each kernel is one program here; "every thread waits" is modelled by the wait being a step of the kernel itself."""
    k1: list[Step] = [("do", lambda m: m.__setitem__("trig1", 1)),
                      ("do", lambda m: m.__setitem__("x", 1)),                 # the value K1 is there to produce
                      ("do", lambda m: m.__setitem__("done1", 1))]
    k2: list[Step] = [("wait", lambda m: g(m, "trig1") == 1),                 # launch condition
                      ("do", lambda m: m.__setitem__("trig2", 1))]            # trigger first: K3 may start at once
    if k2_waits:
        k2.append(("wait", lambda m: g(m, "done1") == 1))
        k2.append(("do", lambda m: None if g(m, "x") == 1 else "K2 read x before K1 wrote it"))
    k2 += [("do", lambda m: m.__setitem__("y", 1)), ("do", lambda m: m.__setitem__("done2", 1))]
    k3: list[Step] = [("wait", lambda m: g(m, "trig2") == 1)]
    if k3_prefetches_weight:
        k3.append(("do", lambda m: None if g(m, "w", 7) == 7 else "the weight changed under the prefetch"))   # nothing ever writes w
    if k3_reads_early:
        k3.append(("do", lambda m: None if g(m, "y") == 1 else "K3 read y before K2 wrote it"))
    k3 += [("wait", lambda m: g(m, "done2") == 1),
           ("do", lambda m: None if g(m, "y") == 1 else "K3 read y before K2 wrote it"),
           ("do", lambda m: None if g(m, "x") == 1 else "K3 read x before K1 wrote it")]
    return [k1, k2, k3]


def test_dependent_launches_are_safe_when_every_kernel_waits():
    assert explore(dependent_launch_programs(), {}) is None


def test_dependent_launch_model_shows_what_each_rule_is_for():
    # data of the predecessor read before the wait: stale
    out = explore(dependent_launch_programs(k3_reads_early=True), {})
    assert out is not None and "K3 read y before" in out
    # a kernel in the middle that does not wait (it happens not to need its predecessor's data) breaks the chain for
    # the kernel after it, which waits for the middle one only
    out = explore(dependent_launch_programs(k2_waits=False), {})
    assert out is not None and "K3 read x before" in out
