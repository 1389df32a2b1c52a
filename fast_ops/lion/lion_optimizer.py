"""Module path of the reference (fast_ops/lion/lion_optimizer.py)."""
from fast_ops_b200.lion.lion_optimizer import Lion, lion_update  # noqa: F401
