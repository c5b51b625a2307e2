"""Stand-alone developer tools that ship with the framework (memory estimator, profile analysis, loss-curve compare)."""
