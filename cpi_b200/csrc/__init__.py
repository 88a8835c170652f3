"""CUDA sources of the kernel library (sm_100a), its build script and its ctypes bindings."""
