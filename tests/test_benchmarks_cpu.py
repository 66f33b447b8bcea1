"""The CPU benchmark entry point (SpanFinder, 16 x 512 planted-span batches) runs and both arms see the same data."""
import pytest

from ml_experiments_b200.benchmarks import spanfinder_cpu as B


def test_spanfinder_cpu_benchmark_runs():
    out = B.main(["--impl", "ours", "--steps", "3", "--warmup", "1"])
    line = out["ours"]
    assert line["params"] == 53954 and line["value"] > 0 and line["final_loss"] == line["final_loss"]


@pytest.mark.skipif(B.reference_root() is None, reason="no copy of the reference package next to the repository")
def test_reference_arm_trains_on_the_same_tensors():
    out = B.main(["--impl", "both", "--steps", "3", "--warmup", "1"])
    # same seed, same batches, same model definition: the two arms start from the same loss
    assert abs(out["ours"]["first_loss"] - out["reference"]["first_loss"]) < 1e-5
