"""CPU oracle for the attention forward and the Lion step.

TEST INFRASTRUCTURE ONLY.  Imported by tests/, by the smoke check and by the CPU-baseline
leg of bench.py as the checker / timed CPU reference.  The product package
(fast_ops_b200) never imports it.
"""
from .oracle import (  # noqa: F401
    attention_bwd,
    attention_ex,
    attention_fwd,
    build,
    dropout_mask,
    lion_step,
    num_threads,
    set_num_threads,
)
