"""CPU oracle for the CD-SSM scan path: test infrastructure, not product code.

Only tests/, the smoke check and the bench's CPU-baseline leg may import this package.
"""
from .oracle import *  # noqa: F401,F403
