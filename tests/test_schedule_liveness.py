"""Liveness of the engine's work schedules, checked on the host.

The chunk kernel has no grid-wide barrier in its layer loop: GEMM CTAs walk a static list of units and wait, unit by
unit, for the stage counter of the activations they consume; row CTAs walk a fixed sequence of attentions and residual
operations and wait for the counters of the GEMMs that feed them.  A schedule is only usable if those two fixed orders
can never wait for each other in a circle.  This test replays both orders for every batch size on the schedule that
``pi05_schedule_plan`` returns (no GPU involved): agents advance whenever the counter they wait for has reached its
target, and the replay must run to completion.

The orders restated here are those of ``act_producer`` / ``epilogue`` (which counter a unit waits for and which it
bumps) and of ``row_cta`` (the three sequences of row work) in ``csrc/pi05_chunk_kernel.cuh``.
"""
import pytest

from pi05_megakernel_b200 import _lib, build

QKV, O, GU, DOWN = range(4)
ROW_CTAS = 25
TUNING = ("PI05_OBS_PER_MMA", "PI05_LATENCY_SCHEDULE", "PI05_ONE_STREAM", "PI05_ROW_GROUPS", "PI05_KEY_GROUPS",
          "PI05_GROUPED_FROM", "PI05_STREAMS_FROM", "PI05_ENTRIES_PER_PHASE")


def replay(batch: int, npass: int, env: dict | None = None) -> int:
    """Returns the number of scheduler sweeps the replay needed; raises AssertionError on a circular wait."""
    entries, plan = _lib.schedule_plan(148, batch, 128)
    gn, ngroups, split = plan["obs_per_mma"], plan["groups"], plan["stream_split"]
    units = plan["units"]
    named = any(e[3] >= 0 for e in entries)
    count: dict = {}                                  # (event, observation) -> value

    def reached(ev, ob, target):
        return count.get((ev, ob), 0) >= target

    def bump(ev, ob, by=1):
        count[(ev, ob)] = count.get((ev, ob), 0) + by

    def obs_of(group):
        return range(group * gn, min(batch, (group + 1) * gn))

    def gemm_cta(lst):
        cycles = npass + (1 if split else 0)
        for cyc in range(cycles):
            for _, gemm, lag, group, tile, _k0, _nk in lst:
                ps = cyc - lag
                if ps < 0 or ps >= npass:
                    continue
                for g in (range(ngroups) if group < 0 else [group]):
                    need = {QKV: ("ana", ROW_CTAS), O: ("att", ROW_CTAS), GU: ("anf", ROW_CTAS),
                            DOWN: ("gu", units["gate_up"])}[gemm]
                    for ob in obs_of(g):              # the MMAs of a group start when all its observations are in
                        while not reached(need[0], ob, need[1] * (ps + 1)):
                            yield
                    out = {QKV: "kv" if tile >= 16 else "q", O: "o", GU: "gu", DOWN: "down"}[gemm]
                    for ob in obs_of(g):
                        bump(out, ob)

    def attention(ob, ps):
        while not reached("q", ob, (units["qkv"] - 4) * (ps + 1)):
            yield
        while not reached("kv", ob, 4 * (ps + 1)):
            yield
        bump("att", ob, ROW_CTAS)                     # one agent stands for the 25 row CTAs of its group

    def residual(ob, ps, first):
        ev, n = ("o", units["o"]) if first else ("down", units["down"])
        while not reached(ev, ob, n * (ps + 1)):
            yield
        bump("anf" if first else "ana", ob, ROW_CTAS)

    def row_group(group, ngrp):
        mine = list(range(group, batch, ngrp))
        for ob in mine:
            bump("ana", ob, ROW_CTAS)                 # the first norm, before the layer loop
        if split:
            for cyc in range(npass + 1):
                for op in range(6):
                    stream = (0x2C >> op) & 1
                    ps = cyc - 1 if op == 2 else cyc
                    if ps < 0 or ps >= npass:
                        continue
                    for ob in mine:
                        if (0 if ob // gn < split else 1) != stream:
                            continue
                        if op in (0, 3):
                            yield from attention(ob, ps)
                        else:
                            yield from residual(ob, ps, op in (1, 5))
            return
        for ps in range(npass):
            if named:                                  # throughput schedule, one stream: all attentions first
                for ob in mine:
                    yield from attention(ob, ps)
                for ob in mine:
                    yield from residual(ob, ps, True)
            else:                                      # attention of one observation, residual of the one before
                for k in range(len(mine) + 1):
                    if k < len(mine):
                        yield from attention(mine[k], ps)
                    if k >= 1:
                        yield from residual(mine[k - 1], ps, True)
            for ob in mine:
                yield from residual(ob, ps, False)

    per_cta: dict = {}
    for e in entries:
        per_cta.setdefault(e[0], []).append(e)
    agents = [gemm_cta(lst) for lst in per_cta.values()]
    agents += [row_group(g, plan["row_groups"]) for g in range(plan["row_groups"])]
    sweeps = 0
    while agents:
        sweeps += 1
        before = dict(count)
        alive = []
        for a in agents:
            try:
                next(a)
                alive.append(a)
            except StopIteration:
                pass
        assert len(alive) < len(agents) or count != before, f"circular wait at batch {batch}: {len(alive)} agents stuck"
        agents = alive
    for ob in range(batch):                           # every observation went through every pass
        assert count[("ana", ob)] == ROW_CTAS * (npass + 1) and count[("down", ob)] == units["down"] * npass
    return sweeps


@pytest.mark.parametrize("batch", list(range(1, 17)))
def test_default_schedules_cannot_deadlock(batch, monkeypatch):
    build.build()
    for name in TUNING:
        monkeypatch.delenv(name, raising=False)
    replay(batch, npass=4)


@pytest.mark.parametrize("env", [{"PI05_OBS_PER_MMA": "2"}, {"PI05_ONE_STREAM": "1"}, {"PI05_LATENCY_SCHEDULE": "1"},
                                 {"PI05_GROUPED_FROM": "2", "PI05_STREAMS_FROM": "2"}, {"PI05_ROW_GROUPS": "2"},
                                 {"PI05_OBS_PER_MMA": "2", "PI05_ONE_STREAM": "1", "PI05_ENTRIES_PER_PHASE": "3"}])
@pytest.mark.parametrize("batch", [2, 3, 5, 7, 8, 12])
def test_tuned_schedules_cannot_deadlock(batch, env, monkeypatch):
    build.build()
    for name in TUNING:
        monkeypatch.delenv(name, raising=False)
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    replay(batch, npass=3)
