"""B200-native kernels behind train-gpt's FP8 hot path.

`fp8.block_scaled_matmul(a, b, block_k=128)` and `kernels.rms_norm(x, scale, eps)` keep
the reference's signatures (train-gpt fp8.py:30-36, kernels.py:55-56); `ops` exposes the
individual kernels; `_lib` is the ctypes binding of the C ABI.
"""
__all__ = ["fp8", "kernels", "ops", "model"]
