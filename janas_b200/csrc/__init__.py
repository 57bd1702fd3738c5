"""CUDA kernels for sm_100a (sources), their build and their Python wrappers."""
