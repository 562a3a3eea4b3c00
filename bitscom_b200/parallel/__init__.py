"""Multi-GPU machinery: symmetric memory, fused collectives, hooks, schedules."""
