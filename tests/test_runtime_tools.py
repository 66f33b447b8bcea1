import torch
import torch.nn as nn

from ml_experiments_b200.runtime import Canary, OpTimer, bitwise_repeatable, check_nan, instrument_module, scheduled_profiler, set_debug_nan


def test_op_timer_and_instrumentation(tmp_path):
    model = nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 4))
    timer = OpTimer(device="cpu")
    undo = instrument_module(model, timer)
    for _ in range(3):
        model(torch.randn(2, 8))
    undo()
    model(torch.randn(2, 8))
    assert timer.calls == {"0": 3, "1": 3, "2": 3} and set(timer.totals_ms()) == {"0", "1", "2"} and "x3" in timer.table()
    with scheduled_profiler(str(tmp_path / "t"), rank=2, wait=1, warmup=1, active=1) as prof:
        for _ in range(4):
            model(torch.randn(2, 8))
            prof.step()
    assert (tmp_path / "t-rank2-chrome-trace.json.gz").exists()


def test_debug_helpers():
    set_debug_nan(True)
    try:
        check_nan(torch.ones(3), "ok")
        try:
            check_nan(torch.tensor([1.0, float("nan")]), "bad")
            raise AssertionError("expected a RuntimeError")
        except RuntimeError as e:
            assert "bad" in str(e) and "nan=1" in str(e)
    finally:
        set_debug_nan(False)
    check_nan(torch.tensor([float("nan")]), "ignored when off")
    c = Canary(10, device="cpu", pad=4)
    c.tensor.fill_(1.0)
    c.check()
    c._buf[1] = 0.0
    try:
        c.check()
        raise AssertionError("expected a RuntimeError")
    except RuntimeError:
        pass
    x = torch.randn(100)
    assert bitwise_repeatable(lambda: x.cumsum(0)) and not bitwise_repeatable(lambda: torch.randn(3))
