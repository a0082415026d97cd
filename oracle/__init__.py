"""CPU oracle for the quantised-matvec / qwen3moe routed-expert path.

TEST INFRASTRUCTURE ONLY: the tests, the smoke check and the benchmark's CPU-baseline leg
may import this package; the product package never does.
"""
from .binding import Oracle, build, load  # noqa: F401
