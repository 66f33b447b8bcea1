"""Per-configuration benchmark entry points (device-timed, max over ranks); bench.py at the repository root is the headline."""
