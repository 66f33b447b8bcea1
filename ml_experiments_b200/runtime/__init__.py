"""Host-side runtime around the training step: failure detection (heartbeats, step watchdog), host-level fault injection
for tests, restart-from-checkpoint, tracing / per-operator timing, and debugging aids (NaN probes, canaries, determinism).
The reference has none of the first three (a failing rank hangs its peers in NCCL) and only ad-hoc versions of the rest."""
from .debug import Canary, bitwise_repeatable, check_nan, set_debug_nan, set_deterministic  # noqa: F401
from .failure import Heartbeat, RankFailure, StepWatchdog, run_with_recovery  # noqa: F401
from .fault_injection import DroppingStore, FaultPlan, InjectedFault  # noqa: F401
from .tracing import OpTimer, instrument_module, nvtx_range, scheduled_profiler  # noqa: F401
