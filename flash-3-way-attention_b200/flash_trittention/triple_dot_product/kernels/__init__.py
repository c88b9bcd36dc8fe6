"""Mask helpers of the triple-dot-product variant (the device kernels live in the CUDA library)."""
