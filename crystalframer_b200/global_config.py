"""Process-wide switch of the reference (models/global_config.py): 0 = pure PyTorch pooling and
attention in the callers, >=1 = fused pooling, >=2 = fused attention.  This package implements
the fused operators only, so the value is kept for interface parity and must stay >= 2."""
REPRODUCIBLITY_STATE = 2
