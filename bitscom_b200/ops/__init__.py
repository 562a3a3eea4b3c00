"""Python entry points of the hand-written sm_100a kernels (ctypes over C symbols)."""
