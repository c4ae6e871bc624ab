"""The seeded inputs of the benchmark configurations live in the package
(``lego_b200/configs.py``) so that bench.py runs without the test tree; the tests
import them under this name."""
from lego_b200.configs import *  # noqa: F401,F403
from lego_b200.configs import GROUPED_CHOICES  # noqa: F401
