"""Serving shims: a translator configured from a key-value text file, a stdin loop, and a small HTTP server that
batches concurrent requests.

``OnlineTranslator(config_path)`` reads lines ``key value`` (``model``, ``beam_size``, ``gpu``, ``bpe_codes`` ignored here,
``src_lang`` / ``tgt_lang``, ``max_sent_length``, ``batch_size`` ...), builds a ``Translator`` and exposes
``translate(text)`` / ``translate_batch(texts)`` / ``set_language``.  ``serve`` starts a ``ThreadingHTTPServer``
(POST /translate with JSON ``{"text": "..."}`` or ``{"texts": [...]}``); a worker thread drains the request queue and
translates up to ``max_batch`` requests at once.  Flask is not required.

Reference: onmt/online_translator.py:17-605 (``TranslatorParameter`` :19, ``OnlineTranslator`` :137, ASR variant :341),
online.py:1-18, flask_online.py / flask_mt.py (request queue, batches of 16).
"""
from __future__ import annotations

import json
import queue
import sys
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from types import SimpleNamespace
from typing import List

from ..options import make_translate_parser
from .translator import Translator


class TranslatorParameter:
    """Translation options read from a ``key value`` file on top of the ``translate.py`` defaults."""

    def __init__(self, path: str):
        opt = make_translate_parser().parse_args(["-model", "none", "-src", "none"])
        opt.gpu, opt.verbose = -1, False
        with open(path) as fh:
            for line in fh:
                parts = line.strip().split(None, 1)
                if len(parts) != 2 or parts[0].startswith("#"):
                    continue
                k, v = parts
                cur = getattr(opt, k, None)
                if isinstance(cur, bool):
                    v = v.lower() in ("1", "true", "yes")
                elif isinstance(cur, int):
                    v = int(v)
                elif isinstance(cur, float):
                    v = float(v)
                setattr(opt, k, v)
        self.opt = opt


class OnlineTranslator:
    def __init__(self, config_path: str):
        self.param = TranslatorParameter(config_path)
        self.translator = Translator(self.param.opt)
        self.src_lang = getattr(self.param.opt, "src_lang", "src")
        self.tgt_lang = getattr(self.param.opt, "tgt_lang", "tgt")
        self.lock = threading.Lock()

    def set_language(self, src_lang: str, tgt_lang: str):
        self.src_lang, self.tgt_lang = src_lang, tgt_lang

    def translate_batch(self, texts: List[str], prefix: List[str] = None) -> List[str]:
        toks = [t.split() for t in texts]
        with self.lock:
            pred, *_ = self.translator.translate(toks, prefix=[p.split() for p in prefix] if prefix else None)
        return [" ".join(p[0]) for p in pred]

    def translate(self, text: str, prefix: str = None) -> str:
        return self.translate_batch([text], [prefix] if prefix else None)[0]


class _BatchingWorker(threading.Thread):
    def __init__(self, translator: OnlineTranslator, max_batch: int = 16):
        super().__init__(daemon=True)
        self.translator, self.max_batch = translator, max_batch
        self.q: "queue.Queue" = queue.Queue()

    def submit(self, text: str):
        slot = SimpleNamespace(text=text, result=None, done=threading.Event())
        self.q.put(slot)
        return slot

    def run(self):
        while True:
            slots = [self.q.get()]
            while len(slots) < self.max_batch:
                try:
                    slots.append(self.q.get_nowait())
                except queue.Empty:
                    break
            try:
                outs = self.translator.translate_batch([s.text for s in slots])
            except Exception as exc:  # noqa: BLE001 - reported to the callers
                outs = ["ERROR: %r" % (exc,)] * len(slots)
            for s, o in zip(slots, outs):
                s.result = o
                s.done.set()


def parse_request_fields(content_type: str, body: bytes) -> dict:
    """Fields of a POST body: JSON, or ``multipart/form-data`` (values as bytes; file parts included) as the clients of
    the reference's Flask servers send it (``pcm_s16le``, ``text``, ``prefix``, ``priority``)."""
    ctype = (content_type or "").lower()
    if ctype.startswith("multipart/form-data"):
        from email.parser import BytesParser
        msg = BytesParser().parsebytes(b"Content-Type: " + content_type.encode() + b"\r\n\r\n" + body)
        return {part.get_param("name", header="content-disposition"): part.get_payload(decode=True) for part in msg.get_payload()
                if part.get_param("name", header="content-disposition")}
    if body:
        try:
            return json.loads(body)
        except ValueError:
            from urllib.parse import parse_qs
            return {k: v[0] for k, v in parse_qs(body.decode("utf-8", "replace")).items()}
    return {}


def serve(config_path: str, host: str = "127.0.0.1", port: int = 5000, max_batch: int = 16):
    """HTTP server with request batching.  Routes: ``POST /`` with JSON ``{"text": ...}`` / ``{"texts": [...]}``; and the
    routes of the reference's Flask servers (flask_mt.py / flask_online.py:163-215):
    ``POST /predictions/<input_language>,<output_language>`` with the fields ``text`` (machine translation) or
    ``pcm_s16le`` (raw 16-bit mono audio for speech models) and optionally ``prefix`` -> ``{"hypo": ...}``, and
    ``GET /models/<input_language>,<output_language>`` -> the configuration the server runs."""
    translator = OnlineTranslator(config_path)
    worker = _BatchingWorker(translator, max_batch)
    worker.start()
    with open(config_path) as fh:
        config_text = fh.read()

    class Handler(BaseHTTPRequestHandler):
        def _reply(self, obj, code=200):
            out = json.dumps(obj).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(out)))
            self.end_headers()
            self.wfile.write(out)

        def do_GET(self):
            if self.path.startswith("/models/"):
                return self._reply({"version": config_text})
            self._reply({"error": "unknown route"}, 404)

        def do_POST(self):
            raw = self.rfile.read(int(self.headers.get("Content-Length", 0)) or 0)
            body = parse_request_fields(self.headers.get("Content-Type", ""), raw)
            if self.path.startswith("/predictions/"):
                langs = self.path[len("/predictions/"):].split(",")
                if len(langs) == 2:
                    translator.set_language(langs[0], langs[1])
                text = lambda v: v.decode("utf-8", "replace") if isinstance(v, (bytes, bytearray)) else v
                prefix = text(body.get("prefix")) or None
                try:
                    if body.get("pcm_s16le") is not None:
                        import numpy as np
                        import torch
                        wav = torch.from_numpy(np.frombuffer(body["pcm_s16le"], dtype="<i2").astype("float32") / 32768.0)
                        with translator.lock:
                            pred, *_ = translator.translator.translate([wav.view(-1, 1)], prefix=[prefix.split()] if prefix else None)
                        hypo = " ".join(pred[0][0])
                    else:
                        hypo = translator.translate(text(body.get("text", "")), prefix)
                    return self._reply({"hypo": hypo})
                except Exception as exc:      # a bad request must not take the server down
                    return self._reply({"hypo": "", "status": 400, "error": str(exc)}, 400)
            texts = body.get("texts") or [body.get("text", "")]
            slots = [worker.submit(t) for t in texts]
            for s in slots:
                s.done.wait()
            self._reply({"translations": [s.result for s in slots]})

        def log_message(self, *a):
            pass

    server = ThreadingHTTPServer((host, port), Handler)
    return server, worker


def stdin_loop(config_path: str):
    t = OnlineTranslator(config_path)
    for line in sys.stdin:
        print(t.translate(line.strip()), flush=True)
