"""Reference arm of the benchmark (see ref_harness.py)."""

# Both arms of bench.py print this string as their ``metric``: what is measured is the same quantity on the same
# model shape and workload; how each arm times it is in the separate ``timing`` key.
METRIC = "decode tok/s (batch 1, greedy); prefill tok/s and p50 TTFT alongside"
