"""Benchmarks a user can run on their own box: kernels against the measured roofline, chunked logprobs,
and an HTTP load test of the inference server (reference: R/benchmarks/*.py)."""
