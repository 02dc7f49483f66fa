"""The option tables under the name that the reference's scripts import (``from options import make_parser,
backward_compatible``): re-exported from ``nmtgminor_b200.options``.  (reference: options.py)"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from nmtgminor_b200.options import *  # noqa: F401,F403
from nmtgminor_b200.options import backward_compatible, make_parser  # noqa: F401
