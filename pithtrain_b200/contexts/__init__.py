"""Process-global runtime state, one module per concern (distributed, training, logging).

Values are set once by the matching ``setup_*`` function and read in-line everywhere else, the same
pattern as pithtrain/contexts/__init__.py:1-7 of the reference.
"""
from . import distributed, logging, training  # noqa: F401
