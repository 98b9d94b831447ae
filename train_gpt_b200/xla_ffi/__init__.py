"""XLA FFI layer over the C ABI: `xla_ffi.cc` (one handler per kernel entry point), `jax_shim.py`
(train-gpt's fp8.py / kernels.py surface on `jax.ffi`), `build.py` (compiles the handlers where
jaxlib's FFI headers exist).  Nothing here is imported by the PyTorch-hosted package."""
