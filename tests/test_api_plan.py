"""CPU tests of the public planning surface: plan(PlanRequest) -> PlannedWorkload, simulate(planned)."""
import json

import pytest

import etx_megakernel_b200  # noqa: F401
from etx_megakernel_b200 import api


def test_model_request_plans_and_simulates():
    req = api.PlanRequest(api.model("qwen3-30b-a3b", config={"layers": 2, "maxlen": 1072}))
    pw = api.plan(req)
    assert pw.report["tasks"] == 1872 and pw.report["workers"] == 148 and pw.report["grids"]["moe_up_0"] == 148
    assert pw.report["verify"] == [] and pw.machine["name"] == "b200" and all(m == "static" for m in pw.report["modes"].values())
    again = api.PlannedWorkload.from_dict(json.loads(json.dumps(pw.to_dict())))
    assert again.identity == pw.identity and api.plan(req).identity == pw.identity          # detached, reproducible records
    sim = api.simulate(pw, seed=3)
    assert sim.backend == "simulation" and not sim.deadlock and sim.plan_identity == pw.identity and sim.seed == 3
    assert 200 < sim.metrics["makespan_us"] < 300 and 0 < sim.metrics["utilisation"] <= 1


def test_declarative_graph_request_and_refusals():
    cfg = {"tensors": [{"name": "impargs", "shape": [64], "role": "weight", "bytes_per_elem": 1}],
           "events": [{"name": "E0", "shape": [1], "wait_count": 4}],
           "grids": [{"name": "a", "grid": [4], "body": {"symbol": "nop"}, "args": ["impargs"], "out_edges": {"E0": "i->(0)"}},
                     {"name": "b", "grid": [1], "body": {"symbol": "nop"}, "args": ["impargs"], "in_edges": {"E0": "i->(0)"}}]}
    pw = api.plan(api.PlanRequest(api.graph("two_phase", config=cfg), options={"workers": 4}))
    assert pw.report["tasks"] == 5 and pw.report["workers"] == 4 and pw.report["grids"] == {"a": 4, "b": 1}
    assert not api.simulate(pw).deadlock
    with pytest.raises(ValueError, match="unknown packaged target"):
        api.plan(api.PlanRequest(api.graph("g", config=cfg), target="gfx942"))
    with pytest.raises(ValueError, match="unknown planner options"):
        api.plan(api.PlanRequest(api.graph("g", config=cfg), options={"relay_budget": 3}))
    with pytest.raises(ValueError, match="nonnegative integers"):
        api.PlanRequest(api.graph("g", config=cfg), bindings={"N": -1})
    with pytest.raises(ValueError, match="at least one grid"):
        api.plan(api.PlanRequest(api.graph("g", config={"tensors": cfg["tensors"]})))
    with pytest.raises(ValueError, match="unknown model configuration"):
        api.plan(api.PlanRequest(api.model("qwen3-8b", config={"layers": 1, "tp": 8})))
    with pytest.raises(ValueError, match="finite JSON"):
        api.model("m", config={"x": float("nan")})
    with pytest.raises(TypeError):
        api.simulate("not a plan")
