"""CPU parity oracle (test infrastructure).

Only the tests, the smoke check and the CPU-baseline legs of the benchmark
import this package.  Nothing under ``nml_b200`` may depend on it.
"""
from .oracle import *  # noqa: F401,F403
