"""Device-timed micro-benchmarks (CUDA events, L2 flushed between iterations) and roofline helpers."""
