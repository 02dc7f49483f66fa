#!/usr/bin/env python
"""HTTP translation server with request batching:  python serve_online.py <config> [host] [port]
(counterpart of the reference's flask_online.py / flask_mt.py; uses the standard library's HTTP server)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from nmtgminor_b200.inference.online import serve

if __name__ == "__main__":
    host = sys.argv[2] if len(sys.argv) > 2 else "127.0.0.1"
    port = int(sys.argv[3]) if len(sys.argv) > 3 else 5000
    server, _ = serve(sys.argv[1], host, port)
    print("serving on %s:%d" % (host, port), flush=True)
    server.serve_forever()
