"""Drop-in module paths of jfc4050/fast-ops, served by fast_ops_b200.

`from fast_ops.flash_attention.flash_attention import multi_head_attention` and
`from fast_ops.lion.lion_optimizer import Lion` resolve to the B200 implementations.
"""
