"""B200-native implementation of the dflash-mlx target-verify hot path.

Mirrors the reference's module names: ``verify_qmm``, ``verify_linear``, ``kernels``,
``recurrent_rollback_cache``.  Tensors are ``torch.Tensor`` on a CUDA device; the compute is
hand-written sm_100a CUDA behind the C ABI in ``include/dflash_b200.h``.
"""
__version__ = "0.1.0"
