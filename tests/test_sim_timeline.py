"""CPU tests of the schedule simulator and the trace analysis (no GPU: the trace rows are simulated or made up)."""
import numpy as np
import pytest

import etx_megakernel_b200  # noqa: F401
from etx_megakernel_b200.models import qwen as Q
from etx_megakernel_b200.passes import compile_graph
from etx_megakernel_b200.runtime.timeline import Timeline, main
from etx_megakernel_b200.sim import simulate


def _plan(name="qwen3-30b-a3b", layers=2, **kw):
    d = Q.load_dims(name, layers=layers)
    g, pool, _ = Q.build_graph(d, lambda n: 0x7F0000000000, 1072, **kw)
    return compile_graph(g, "b200", {"POOL": len(pool.bytes())})


def test_simulated_step_runs_every_task_once_and_predicts_the_measured_step():
    plan = _plan()
    r = simulate(plan)
    assert not r.deadlock and len(r.done) == len(plan.tasks) == sum(1 for s in r.segments if s.kind == "task")
    # a 2-layer Qwen3-30B-A3B step measured 245-290 us on B200; the annotations come from those stamps
    assert 200.0 < r.makespan_us < 300.0, r.summary()
    assert 0.0 < r.utilisation <= 1.0 and abs(r.busy_us - sum(r.per_grid_us.values())) < 1e-6
    # every task starts after all its producers are done
    for tid, t in enumerate(plan.tasks):
        for ev in plan.inst.task_in[(t.grid, t.coord)]:
            for p in plan.inst.producers[ev]:
                assert r.done[plan.task_index[p]] <= r.ready[tid]
    # the unfused phase structure has more phases and is predicted slower
    assert simulate(_plan(fused_attn=False, fold_topk=False)).makespan_us > r.makespan_us


def test_simulator_reports_a_deadlock_with_the_blocked_tasks():
    plan = _plan("qwen3-8b", layers=1)
    q = plan.static_queues[(0, 0)]
    q[0], q[-1] = q[-1], q[0]                                   # a consumer queued ahead of its producer
    r = simulate(plan)
    assert r.deadlock and any("waits for" in b for b in r.blocked) and "DEADLOCK" in r.summary()
    with pytest.raises(ValueError, match="deadlocked"):
        Timeline.from_sim(plan, r)


def test_timeline_tables_and_critical_path():
    plan = _plan()
    r = simulate(plan)
    tl = Timeline.from_sim(plan, r)
    assert abs(tl.span_us - r.makespan_us) < 1e-9
    rows = {x["grid"]: x for x in tl.by_grid()}
    assert rows["moe_up_0"]["tasks"] == 148 and rows["lm_head"]["tasks"] == 148
    assert rows["qkv_1"]["last_ready"] > rows["moe_down_0"]["last_done"]
    steps, totals = tl.critical_path()
    whole = sum(v["body"] + v["dependency"] + v["queue"] for v in totals.values()) + steps[-1].gap_us
    assert abs(whole - tl.span_us) < 1e-6                       # the path telescopes to the span
    assert steps[0].grid == "argmax" and steps[-1].grid == "prologue" and steps[-1].via == "start"
    assert "critical path" in tl.text()


def test_raw_rows_follow_the_nine_int64_layout(tmp_path):
    plan = _plan("qwen3-8b", layers=1)
    n = len(plan.tasks)
    rows = np.zeros((n, 8), np.uint64)                          # a made-up device trace: 1 us per task, back to back per worker
    for (dev, w), q in plan.static_queues.items():
        for i, tid in enumerate(q):
            rows[tid] = [10_000 + 1000 * i, 10_200 + 1000 * i, 11_000 + 1000 * i, w, 10_300 + 1000 * i, 0, 0, 0]
    tl = Timeline.from_trace(plan, rows)
    raw = tl.raw_rows()
    assert raw.shape == (n, 9) and raw.dtype == np.int64
    t = plan.tasks[5]
    assert raw[5, 0] == plan.type_ids[t.grid] and raw[5, 1] == t.coord[0] and raw[5, 8] == rows[5, 3]
    assert raw[5, 5] == rows[5, 0] and raw[5, 6] == rows[5, 1] and raw[5, 7] == rows[5, 2]
    assert abs(tl.by_grid()[0]["wait"] - 0.2) < 1e-9 and abs(tl.by_grid()[0]["marks"][0] - 0.1) < 1e-9
    tl.write_raw(tmp_path / "trace.bin")
    assert (tmp_path / "trace.bin").stat().st_size == n * 72
    assert main(["--layers", "1", "--sim", "--model", "qwen3-8b"]) == 0
