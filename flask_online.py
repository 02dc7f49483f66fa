#!/usr/bin/env python
"""python flask_online.py <host> <port> [model.conf]
The serving entry point under the reference's name and argument order.  Routes: POST /predictions/<in>,<out> (fields
``text`` or ``pcm_s16le``, optional ``prefix``) -> {"hypo": ...}; GET /models/<in>,<out> -> the configuration.  Runs on the
standard library's threaded HTTP server with the request batching of ``nmtgminor_b200/inference/online.py`` (Flask is not
needed).  (reference: flask_mt.py, flask_online.py)"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from nmtgminor_b200.inference.online import serve

if __name__ == "__main__":
    if len(sys.argv) < 3:
        sys.exit(__doc__)
    host, port = sys.argv[1], int(sys.argv[2])
    conf = sys.argv[3] if len(sys.argv) > 3 else "model.conf"
    server, _ = serve(conf, host, port)
    print("serving %s on %s:%d" % (conf, host, port), flush=True)
    server.serve_forever()
