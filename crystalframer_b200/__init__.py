"""crystalframer_b200: B200 (sm_100a) implementation of CrystalFramer's periodic lattice-sum
attention path behind the reference's own module and autograd-Function interfaces.

``cuda_funcs``  drop-in autograd Functions (reference: models/cuda_funcs)
``attention``   CrystalformerMultiheadAttentionCUDA (reference: models/indexed_lattice_multi_head_attention_cuda.py)
``encoder``     pair list, lattice geometry, encoder stack (reference: models/indexed_latticeformer_encoder.py)
``pooling``     per-crystal pooling (reference: models/pooling.py)
``synth``       seeded synthetic crystal batches

The compute lives in ``libcfb200.so`` (C ABI in ``include/cfb200.h``); importing the operator
modules without that library raises -- there is no CPU or PyTorch fallback.
"""
__version__ = "0.1.0"
