"""Data-parallel training: communicators, fused all-reduce + optimizer, parameter-server shards."""
