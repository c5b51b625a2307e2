"""Step profiling without external tools: ``capture`` records one steady-state training step per rank with
the CUPTI-based torch profiler, ``analyze`` turns the traces into stream/overlap/kernel-class tables."""
