"""Training infrastructure: distributed setup, training setup, optimizers, checkpointing, data, logging."""
