"""Python faces of the native runtime: capped pool, CUDA-graph replay, schedule
log / happens-before checker, planner core."""
