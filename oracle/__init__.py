"""CPU oracle for the conv hot path: test infrastructure only (tests, smoke, cpu_baseline)."""
from .oracle import *  # noqa: F401,F403
