import json
import threading
import urllib.request

import pytest
import torch

from nmtgminor_b200.data.synthetic import synthetic_dict
from nmtgminor_b200.inference.online import OnlineTranslator, serve
from nmtgminor_b200.inference.scoring import PerplexityScorer, Rescorer, StreamTranslator
from nmtgminor_b200.models.factory import build_model
from nmtgminor_b200.options import default_options, make_translate_parser
from nmtgminor_b200.tools.checkpoints import average_checkpoints, best_checkpoints, extend_vocabulary, rematch_embeddings
from nmtgminor_b200.train.checkpoint import save_checkpoint


@pytest.fixture(scope="module")
def ckpt(tmp_path_factory):
    torch.manual_seed(0)
    d = synthetic_dict(40)
    opt = default_options(["-model_size", "32", "-layers", "1", "-n_heads", "1", "-inner_size", "64", "-ffn_activation", "relu",
                           "-tie_weights", "-join_embedding"])
    base = tmp_path_factory.mktemp("ck")
    paths = []
    for i, ppl in enumerate((9.0, 5.0, 7.0)):
        torch.manual_seed(i)
        m = build_model(opt, {"src": d, "tgt": d})
        p = str(base / ("model_ppl_%.6f_e%d.00.pt" % (ppl, i + 1)))
        save_checkpoint(p, m, {"src": d, "tgt": d}, opt, float(i + 1))
        paths.append(p)
    return base, paths, d


def _topt(path, **kw):
    o = make_translate_parser().parse_args(["-model", path, "-src", "x", "-gpu", "-1", "-beam_size", "2", "-max_sent_length", "6"])
    for k, v in kw.items():
        setattr(o, k, v)
    return o


def test_average_and_best(ckpt):
    base, paths, _ = ckpt
    best = best_checkpoints(str(base / "model"), 2)
    assert "5.000000" in best[0] and "7.000000" in best[1]
    out = average_checkpoints(paths, str(base / "avg.pt"))
    states = [torch.load(p, weights_only=False)["model"] for p in paths]
    avg = torch.load(out, weights_only=False)["model"]
    k = "encoder.word_lut.weight"
    assert torch.allclose(avg[k], sum(s[k] for s in states) / 3, atol=1e-6)


def test_ensemble_scorer_rescorer_stream(ckpt):
    _, paths, d = ckpt
    src = [["w1", "w2", "w3"], ["w4", "w5"]]
    ens = PerplexityScorer(_topt("|".join(paths[:2])))
    pred, ids, scores, *_ = ens.translate(src)
    assert len(pred) == 2 and all(isinstance(s[0], float) for s in scores)
    single = PerplexityScorer(_topt(paths[0]))
    sc, ppl = single.score(src, [["w2", "w3"], ["w5"]])
    assert len(sc) == 2 and ppl > 1
    ranked = Rescorer(_topt(paths[0])).rescore(src[:1], [[["w2"], ["w3", "w4"], ["w9"]]])
    assert ranked[0][0][1] >= ranked[0][-1][1]
    st = StreamTranslator(_topt(paths[0]), context_tokens=2)
    a = st.translate_segment(src[0])
    b = st.translate_segment(src[1])
    assert isinstance(a, list) and isinstance(b, list)


def test_online_translator_and_http_server(ckpt, tmp_path):
    _, paths, _ = ckpt
    cfg = tmp_path / "online.conf"
    cfg.write_text("model %s\nbeam_size 2\ngpu -1\nmax_sent_length 5\n" % paths[0])
    t = OnlineTranslator(str(cfg))
    assert isinstance(t.translate("w1 w2 w3"), str)
    server, _ = serve(str(cfg), "127.0.0.1", 0)
    port = server.server_address[1]
    th = threading.Thread(target=server.serve_forever, daemon=True)
    th.start()
    req = urllib.request.Request("http://127.0.0.1:%d/translate" % port, data=json.dumps({"texts": ["w1 w2", "w3"]}).encode(),
                                 headers={"Content-Type": "application/json"})
    out = json.loads(urllib.request.urlopen(req, timeout=60).read())
    server.shutdown()
    assert len(out["translations"]) == 2


def test_vocabulary_tools(ckpt):
    _, paths, d = ckpt
    state = torch.load(paths[0], weights_only=False)["model"]
    n = state["encoder.word_lut.weight"].shape[0]
    extend_vocabulary(state, ["encoder.word_lut.weight", "generator.0.linear.bias"], n + 5)
    assert state["encoder.word_lut.weight"].shape[0] == n + 5 and state["generator.0.linear.bias"].shape[0] == n + 5
    d2 = synthetic_dict(20)
    d2.add("brand_new")
    w = rematch_embeddings(state["decoder.word_lut.weight"], d, d2)
    assert torch.equal(w[d2.lookup("w3")], state["decoder.word_lut.weight"][d.lookup("w3")])
