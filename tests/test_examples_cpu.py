"""The example programs run end to end on CPU processors (threads) and agree with eager PyTorch."""
import importlib
import os
import sys

import pytest

EX = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples")


def _load(name):
    sys.path.insert(0, EX)
    try:
        for m in ("common", name):
            sys.modules.pop(m, None)
        return importlib.import_module(name)
    finally:
        sys.path.remove(EX)


@pytest.mark.parametrize("name,kinds", [("parallel", {"reduce"}), ("pl", {"reduce"}), ("cp", {"broadcast"}),
                                        ("ep", {"alltoall"}), ("engines", {"permute"}), ("crossing", {"reduce"})])
def test_compiled_examples(name, kinds):
    rep = _load(name).main(["--small", "--nodes", "2"])
    assert rep["ok"] and rep["signature_ok"], rep
    assert kinds <= set(rep["by_kind"]), rep["by_kind"]


def test_parallel_example_archive_round_trip_and_unequal_shares():
    rep = _load("parallel").main(["--small", "--nodes", "2", "--archive", "--units", "3,1"])
    assert rep["ok"], rep


def test_planner_workload_moves_columns_to_the_fast_rank():
    rep = _load("planner_workload").main(["--ticks", "60", "--bots", "96", "--ff", "1024", "--slow", "1,3"])
    assert sum(rep["columns"]) == 1024 and rep["columns"][0] > rep["columns"][1], rep


def test_hybrid_train_example_solo_cpu():
    losses = _load("hybrid_train").main(["--small", "--steps", "4"])
    assert losses[-1] < losses[0]


@pytest.mark.parametrize("flags", [[], ["--inference", "--grid", "2,2,1"]])
def test_hybrid_job_as_one_compiled_program(flags):
    """Pipeline x context x tensor on a grid of CPU threads: one compiled step, the numbers of eager PyTorch."""
    rep = _load("hybrid_compiled").main(["--small"] + flags)
    assert rep["ok"] and rep["signature_ok"] and rep["gathering_fallbacks"] == 0, rep
    assert rep["by_verb"].get("send_recv", 0) >= 1
    if flags:
        assert rep["fused"]["ring_attention"] == 4, rep
