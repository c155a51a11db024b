"""Benchmark harness: the result contract, the observer, the host-load meter, the noise-aware comparator and the
runner that drives this package's public API.  ``python -m benchmarks.harness --help`` lists the commands."""
