"""The per-sentence ``Beam`` API, the candidate-selection strategies and the two translators built on them."""
import math

import pytest
import torch

from nmtgminor_b200.data.synthetic import synthetic_dict
from nmtgminor_b200.inference.legacy_search import (Beam, BeamSearch, DiverseBeamSearch, GlobalStreamTranslator,
                                                    LegacyTranslator, Sampling)
from nmtgminor_b200.inference.scoring import PerplexityScorer
from nmtgminor_b200.models.factory import build_model
from nmtgminor_b200.options import default_options, make_translate_parser
from nmtgminor_b200.train.checkpoint import save_checkpoint


@pytest.fixture(scope="module")
def ckpt(tmp_path_factory):
    torch.manual_seed(3)
    d = synthetic_dict(30)
    opt = default_options(["-model_size", "32", "-layers", "1", "-n_heads", "1", "-inner_size", "64", "-ffn_activation", "relu",
                           "-tie_weights", "-join_embedding"])
    m = build_model(opt, {"src": d, "tgt": d})
    p = str(tmp_path_factory.mktemp("ck") / "model_ppl_5.000000_e1.00.pt")
    save_checkpoint(p, m, {"src": d, "tgt": d}, opt, 1.0)
    return p, d


def _topt(path, **kw):
    o = make_translate_parser().parse_args(["-model", path, "-src", "x", "-gpu", "-1", "-beam_size", "3", "-max_sent_length", "7",
                                            "-n_best", "3"])
    for k, v in kw.items():
        setattr(o, k, v)
    return o


def test_beam_backpointers():
    """Three steps over a hand-made distribution: the back-pointers must reproduce the best path."""
    V, K = 6, 2
    beam = Beam(K, bos_id=2, eos_id=3, pad_id=0)
    lk = torch.full((K, V), -10.0)
    lk[0, 4], lk[0, 5] = -0.1, -0.2
    beam.advance(lk.clone())
    assert beam.get_current_state().tolist() == [4, 5] and beam.get_current_origin().tolist() == [0, 0]
    lk = torch.full((K, V), -10.0)
    lk[0, 5] = -3.0          # continuation of "4" is bad
    lk[1, 4] = -0.1          # continuation of "5" is good: the second hypothesis overtakes
    beam.advance(lk)
    assert beam.get_current_origin().tolist()[0] == 1
    lk = torch.full((K, V), -10.0)
    lk[:, 3] = -0.01         # EOS
    done = beam.advance(lk)
    assert done and beam.done
    hyp, _ = beam.get_hyp(0)
    assert hyp == [5, 4, 3]
    score, idx = beam.get_best()
    assert math.isclose(float(score), -0.2 - 0.1 - 0.01, rel_tol=1e-5) and int(idx) == 0


def test_search_strategies_shapes_and_rules():
    torch.manual_seed(0)
    B, K, V = 2, 4, 11
    lp = torch.log_softmax(torch.randn(B, K, V), -1)
    scores = torch.randn(B, K, 3)
    s, t, b = BeamSearch().step(2, lp, scores)
    ref = (lp + scores[:, :, 1:2]).view(B, -1).topk(2 * K, 1)
    assert torch.equal(t, ref[1] % V) and torch.equal(b, ref[1] // V) and torch.allclose(s, ref[0])
    s0, t0, b0 = BeamSearch().step(0, lp, None)
    assert int(b0.max()) == 0                                   # only the first beam is alive at step 0
    # diverse: groups may not pick the same word for free
    d = DiverseBeamSearch(num_groups=2, diversity_strength=100.0)
    sd, td, bd = d.step(1, lp, scores)
    g0, g1 = td[:, 0::2], td[:, 1::2]
    assert all(int(g1[i, 0]) not in g0[i].tolist() for i in range(B))
    assert set((bd[:, 0::2] % 2).flatten().tolist()) == {0} and set((bd[:, 1::2] % 2).flatten().tolist()) == {1}
    # sampling: top-k = 1 is greedy
    smp = Sampling(sampling_topk=1)
    ss, ts, bs = smp.step(1, lp, scores)
    assert torch.equal(ts, lp.argmax(-1)) and torch.equal(bs, torch.arange(K).repeat(B, 1))
    smp = Sampling(sampling_topp=0.5)
    ss, ts, bs = smp.step(1, lp, scores)
    assert ts.shape == (B, K) and bool(torch.isfinite(ss).all())


def test_legacy_translator_is_consistent_with_fast_search(ckpt):
    path, d = ckpt
    src = [["w1", "w2", "w3", "w4"], ["w5", "w6"], ["w7"]]
    fast = PerplexityScorer(_topt(path))
    legacy = LegacyTranslator(_topt(path))
    pf, idf, sf, *_ = fast.translate(src)
    pl, idl, sl, *_ = legacy.translate(src)
    for i in range(len(src)):
        # every legacy hypothesis carries the model's own score of its tokens
        for toks, score in zip(pl[i], sl[i]):
            gold, _ = fast.score([src[i]], [toks])
            assert math.isclose(gold[0], score, rel_tol=1e-4, abs_tol=1e-4)
        # both searches agree on the best hypothesis of these short sentences
        assert pl[i][0] == pf[i][0]
        assert math.isclose(sl[i][0], sf[i][0], rel_tol=1e-4, abs_tol=1e-4)


def test_global_stream_translator_carries_scores(ckpt):
    path, d = ckpt
    g = GlobalStreamTranslator(_topt(path), context_tokens=2)
    segs = [["w1", "w2", "w3"], ["w4", "w5"], ["w6", "w7", "w8"]]
    outs = [g.translate_segment(s) for s in segs]
    assert len(g.document()) == 3 and g.document()[-1] == outs[-1]
    assert int(g.prev_lengths[0]) == sum(len(o) + 1 for o in g.document())
    # cumulative scores are sorted and only decrease as segments are added
    sc = g.prev_scores.tolist()
    finite = [x for x in sc if math.isfinite(x)]
    assert finite == sorted(finite, reverse=True)
    first = GlobalStreamTranslator(_topt(path), context_tokens=2)
    first.translate_segment(segs[0])
    assert float(first.prev_scores[0]) > float(g.prev_scores[0])
    # without context the first segment equals the plain translator's output
    plain = PerplexityScorer(_topt(path))
    pred, *_ = plain.translate([segs[0]])
    assert pred[0][0] == g.document()[0]
    g.reset_stream()
    assert g.prev_hyps[0] == [] and float(g.prev_scores[0]) == 0.0
