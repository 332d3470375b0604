"""fsgs: B200 (sm_100a) kernels for Fast-SP-GS's surfel-rendering hot path behind the reference's operator API.

``fsgs.ops``       the reference's nine operator names over the C ABI of ``libfsgs.so``
``fsgs.install``   makes the reference's own Python (``fast_2d_gs.renderer``, ``utils.cdist_top``,
                   ``fast_2d_gs.sparse_gaussian_adam``) bind to these operators, unmodified
``fsgs.renderer``  ``GS_2D_fast_render`` with the reference's signature and result dictionary
``fsgs.optim``     ``SparseGaussianAdam`` (single fused launch)
``fsgs.dist``      one-view-per-GPU sharding with NCCL all-reduce of per-Gaussian gradients
"""
from .install import install  # noqa: F401
