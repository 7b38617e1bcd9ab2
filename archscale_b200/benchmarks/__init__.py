"""Measurement entry points, kept apart from the operators they time.

* ``python -m archscale_b200.benchmarks.kernels [names…]`` — CUDA-event timings of the hand-written kernels on the
  shapes of the flagship configurations, with achieved bandwidth / FLOP rate against the measured peaks.
* ``python -m archscale_b200.benchmarks.reference_bars [names…]`` — the same shapes on what the reference calls
  (its Triton files loaded by path from ``$ARCHSCALE_REFERENCE_DIR``, flash_attn, QuACK).
* ``python -m archscale_b200.benchmarks.profile_cases <case>`` — one small launch sequence per kernel, sized for a
  profiler capture (a few launches, inputs just above the L2 size).
"""
