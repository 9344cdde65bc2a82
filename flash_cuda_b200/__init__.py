"""flash_cuda_b200 — a B200-native (sm_100a) FlashAttention forward behind the `fwd` /
`get_scheduler_metadata` torch-op boundary, with a plain C ABI underneath (include/fa_b200.h).

  flash_cuda_b200.ops    the torch ops (drop-in boundary)
  flash_cuda_b200.capi   ctypes binding of the C ABI
  flash_cuda_b200.build  in-tree build of both shared libraries
"""
__all__ = ["ops", "capi", "build"]
