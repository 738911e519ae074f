"""Test support that ships with the package: the scripted multi-rank harness."""
from .harness import RankHarness  # noqa: F401
