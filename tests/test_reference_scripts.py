"""The entry points that exist under the reference's script names: checkpoint averaging by file name, language surgery,
vocabulary extraction, text normalisation, auto-encoder training / scoring, the serving routes."""
import json
import os
import subprocess
import sys
import threading
import urllib.request

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PY = sys.executable


def _run(*args, cwd=ROOT):
    r = subprocess.run([PY] + list(args), cwd=cwd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    return r.stdout


@pytest.fixture(scope="module")
def trained(tmp_path_factory):
    """A tiny multilingual model trained for a few updates through the command line, with two checkpoints."""
    d = tmp_path_factory.mktemp("ref_scripts")
    import random
    rng = random.Random(0)
    for split, n in (("train", 200), ("valid", 20)):
        with open(d / ("%s.src" % split), "w") as fs, open(d / ("%s.tgt" % split), "w") as ft:
            for _ in range(n):
                L = rng.randint(3, 9)
                words = ["w%d" % rng.randint(0, 30) for _ in range(L)]
                fs.write(" ".join(words) + "\n")
                ft.write(" ".join(reversed(words)) + "\n")
    _run("preprocess.py", "-train_src", str(d / "train.src"), "-train_tgt", str(d / "train.tgt"), "-valid_src", str(d / "valid.src"),
         "-valid_tgt", str(d / "valid.tgt"), "-save_data", str(d / "data"), "-format", "raw", "-join_vocab", "-train_src_lang", "en", "-train_tgt_lang", "de", "-valid_src_lang", "en", "-valid_tgt_lang", "de")
    _run("train.py", "-data", str(d / "data"), "-data_format", "raw", "-save_model", str(d / "model"), "-model", "multilingual_translator",
         "-multilingual_factorized_weights", "-multilingual_adapter", "-adapter_bottleneck_size", "8", "-model_size", "32", "-inner_size", "64",
         "-n_heads", "2", "-layers", "1", "-batch_size_words", "200", "-epochs", "2", "-optim", "adam", "-learning_rate", "0.001",
         "-update_method", "regular", "-dropout", "0.0", "-seed", "3")
    ckpts = sorted(p for p in os.listdir(d) if p.startswith("model_ppl_"))
    assert len(ckpts) >= 2
    return d, [str(d / c) for c in ckpts]


def test_average_checkpoints_auto_and_sample_lm_averaging(trained):
    d, ckpts = trained
    out = str(d / "avg.pt")
    _run("average_checkpoints_auto.py", "-models", str(d), "-top", "2", "-output", out)
    a, b, avg = (torch.load(p, weights_only=False)["model"] for p in (ckpts[0], ckpts[1], out))
    k = next(k for k in a if a[k].is_floating_point())
    assert torch.allclose(avg[k], (a[k] + b[k]) / 2, atol=1e-6)
    out2 = str(d / "avg2.pt")
    _run("sample_lm.py", "-models", "|".join(ckpts[:2]), "-output", out2)
    assert torch.allclose(torch.load(out2, weights_only=False)["model"][k], avg[k], atol=1e-6)


def test_extend_weight_and_rematch_language_embedding(trained):
    d, ckpts = trained
    out = str(d / "ext.pt")
    _run("extend_weight.py", "-model", ckpts[0], "-n_languages", "5", "-output", out)
    old, new = torch.load(ckpts[0], weights_only=False), torch.load(out, weights_only=False)
    n_old = len(old["dicts"]["langs"])
    grown = [k for k in old["model"] if torch.is_tensor(old["model"][k]) and old["model"][k].dim() > 0
             and new["model"][k].shape[0] == 5 and old["model"][k].shape[0] == n_old]
    assert any(k.endswith(".r") for k in grown) and any("lang_embed" in k for k in grown)
    k = next(k for k in grown if k.endswith(".r"))
    assert torch.equal(new["model"][k][:n_old], old["model"][k])
    assert any(".adapters.4." in k for k in new["model"]) and not any(".adapters.4." in k for k in old["model"])
    # the extended state loads into a model built for five languages
    from nmtgminor_b200.models.factory import build_model
    from nmtgminor_b200.options import backward_compatible
    from nmtgminor_b200.train.checkpoint import load_model_state
    dicts = dict(new["dicts"])
    dicts["langs"] = {"l%d" % i: i for i in range(5)}
    model = build_model(backward_compatible(new["opt"]), dicts)
    load_model_state(model, new["model"], strict=True)
    # language tables follow another checkpoint's language order
    other = dict(old)
    other["dicts"] = dict(old["dicts"])
    other["dicts"]["langs"] = {lang: (n_old - 1 - i) for lang, i in old["dicts"]["langs"].items()}
    torch.save(other, d / "other.pt")
    _run("rematch_language_embedding.py", "-model_src", ckpts[0], "-model_tgt", str(d / "other.pt"), "-model_out", str(d / "rematched.pt"))
    re = torch.load(d / "rematched.pt", weights_only=False)
    k = next(k for k in old["model"] if "lang_embed" in k)
    assert torch.equal(re["model"][k][n_old - 1], old["model"][k][0]) and re["dicts"]["langs"] == other["dicts"]["langs"]


def test_extract_vocab_and_normalize_text(trained, tmp_path):
    d, _ = trained
    out = str(tmp_path / "ids.pt")
    _run("extract_vocab.py", "-dict", str(d / "data.train.pt"), "-text", "%s|%s" % (d / "valid.src", d / "valid.tgt"), "-output", out)
    counts = torch.load(out, weights_only=False)
    n_words = sum(len(l.split()) for f in ("valid.src", "valid.tgt") for l in open(d / f))
    assert sum(counts.values()) == n_words and list(counts.values()) == sorted(counts.values())
    text = tmp_path / "t.txt"
    text.write_text("Hello,  World!\n“Quoted” ‘text’ here.\n!!! ???\n")
    _run("normalize_text.py", str(text), "en", "2")
    assert open(str(text) + ".norm").read().splitlines() == ["hello world", "quoted 'text' here", ""]
    _run("normalize_text.py", str(text), "en", "1", "1")
    assert open(str(text) + ".norm.clean").read().splitlines() == ["hello world", "quoted 'text' here"]


def test_autoencoder_train_and_eval(trained, tmp_path):
    d, ckpts = trained
    _run("autoencoder.py", "-data", str(d / "data"), "-data_format", "raw", "-load_from", ckpts[0], "-save_model", str(tmp_path / "ae"),
         "-auto_encoder_hidden_size", "8", "-epochs", "2", "-batch_size_words", "200", "-learning_rate", "0.001")
    ae = str(tmp_path / "ae_e2.pt")
    assert os.path.exists(ae)
    out = str(tmp_path / "scores.txt")
    _run("eval_autoencoder.py", "-model", ckpts[0], "-autoencoder", ae, "-src", str(d / "valid.src"), "-output", out)
    scores = [float(x) for x in open(out)]
    assert len(scores) == 20 and all(s >= 0 for s in scores)


def test_serving_routes_of_the_reference(trained, tmp_path):
    from nmtgminor_b200.inference.online import parse_request_fields, serve
    d, ckpts = trained
    conf = tmp_path / "model.conf"
    conf.write_text("model %s\nbeam_size 2\nmax_sent_length 12\n" % ckpts[0])
    server, _ = serve(str(conf), "127.0.0.1", 0)
    port = server.server_address[1]
    threading.Thread(target=server.serve_forever, daemon=True).start()
    try:
        req = urllib.request.Request("http://127.0.0.1:%d/predictions/en,de" % port, data=json.dumps({"text": "w1 w2 w3"}).encode(),
                                     headers={"Content-Type": "application/json"})
        hypo = json.loads(urllib.request.urlopen(req, timeout=60).read())["hypo"]
        assert isinstance(hypo, str)
        ver = json.loads(urllib.request.urlopen("http://127.0.0.1:%d/models/en,de" % port, timeout=60).read())
        assert "beam_size 2" in ver["version"]
        old = json.loads(urllib.request.urlopen(urllib.request.Request(
            "http://127.0.0.1:%d/" % port, data=json.dumps({"texts": ["w1 w2", "w3"]}).encode()), timeout=60).read())
        assert len(old["translations"]) == 2
    finally:
        server.shutdown()
    boundary = "XyZ"
    body = ("--XyZ\r\nContent-Disposition: form-data; name=\"text\"\r\n\r\nhello there\r\n--XyZ\r\nContent-Disposition: form-data; "
            "name=\"pcm_s16le\"; filename=\"a\"\r\nContent-Type: application/octet-stream\r\n\r\n\x01\x00\x02\x00\r\n--XyZ--\r\n").encode("latin-1")
    fields = parse_request_fields("multipart/form-data; boundary=%s" % boundary, body)
    assert fields["text"] == b"hello there" and fields["pcm_s16le"] == b"\x01\x00\x02\x00"
