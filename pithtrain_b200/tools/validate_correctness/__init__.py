"""Loss-curve regression check: run the same short job on two builds, then compare the rank-0 logs."""
