"""spgt_b200: sm_100a kernels for the SpGT (Speed Galerkin Transformer) Darcy inference forward.

The kernels live in libspgt_b200.so behind the C ABI of include/spgt_b200.h; this package is the host-side
mirror of the reference's op and module interface (extension/bind, network/sp_layer.py, network/sp_model.py).
"""
__version__ = '0.1.0'
