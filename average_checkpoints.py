#!/usr/bin/env python
"""python average_checkpoints.py average -models a.pt b.pt -output avg.pt [-method mean|gmean] | best -prefix model -top 5
(reference: tools/average_checkpoints.py, average_checkpoints_auto.py, tools/get_best.py)"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from nmtgminor_b200.tools.checkpoints import main

if __name__ == "__main__":
    main()
