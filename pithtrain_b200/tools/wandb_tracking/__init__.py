"""Helpers around Weights & Biases runs of this trainer (list, compare a metric across runs, fetch run files)."""
