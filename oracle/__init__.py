"""CPU checker for the packed-KV decode path.  Test infrastructure: only the
test-suite, the smoke entry and the benchmark's CPU-baseline leg import it."""
