"""Graph-level operators (NumPy oracle path + sm_100a kernel path per op)."""
