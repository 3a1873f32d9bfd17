"""Native sources (CUDA kernels, C++ host runtime), their build and their Python bindings."""
