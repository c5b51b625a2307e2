"""Parallel runtime: 4-D mesh, flat-sharded parameters, symmetric memory, expert-parallel dispatch."""
