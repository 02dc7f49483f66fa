#!/usr/bin/env python
"""stdin -> stdout translation loop configured by a key-value file:  python online.py <config>   (reference: online.py:1-18)"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from nmtgminor_b200.inference.online import stdin_loop

if __name__ == "__main__":
    stdin_loop(sys.argv[1])
