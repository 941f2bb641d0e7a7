"""The loader of the unchanged reference modules lives in oracle/reference_loader.py; this name is kept for
the tests and the golden generator that import it from here."""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir, os.pardir, "oracle"))
from reference_loader import *  # noqa: F401,F403,E402
from reference_loader import REFERENCE_ROOT, _cache  # noqa: F401,E402
