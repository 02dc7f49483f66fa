"""-mirror_loss / -reconstruct: the backward decoder, the state-matching term and the source reconstruction decoder."""
import torch

from nmtgminor_b200.data.dataset import collate
from nmtgminor_b200.data.synthetic import synthetic_dict
from nmtgminor_b200.models.factory import build_model
from nmtgminor_b200.models.layers import PackedSeqs
from nmtgminor_b200.options import default_options

ARGS = ["-model_size", "32", "-layers", "1", "-n_heads", "1", "-inner_size", "64", "-ffn_activation", "relu", "-dropout", "0",
        "-attn_dropout", "0", "-word_dropout", "0", "-emb_dropout", "0", "-label_smoothing", "0"]


def _model(extra):
    torch.manual_seed(0)
    d = synthetic_dict(30)
    m = build_model(default_options(ARGS + extra), {"src": d, "tgt": d})
    m.train()
    return m


SRC = [torch.tensor([5, 6, 7, 8]), torch.tensor([9, 10]), torch.tensor([4, 5, 6])]
TGT = [torch.tensor([2, 11, 12, 13, 3]), torch.tensor([2, 14, 3]), torch.tensor([2, 15, 16, 17, 18, 3])]


def test_flip_index_reverses_each_sequence():
    m = _model(["-mirror_loss", "1"])
    cu = torch.tensor([0, 3, 5, 9], dtype=torch.int32)
    seqs = PackedSeqs(torch.arange(12), torch.zeros(12, dtype=torch.long), cu, 4)
    assert m._flip_index(seqs, 12).tolist() == [2, 1, 0, 4, 3, 8, 7, 6, 5, 9, 10, 11]


def test_mirror_terms_match_sentence_by_sentence():
    m = _model(["-mirror_loss", "0.5"])
    whole = m(collate(SRC, TGT, padded=True, packed=True))
    rev = mir = nmt = 0.0
    for s, t in zip(SRC, TGT):
        one = m(collate([s], [t], padded=True, packed=True))
        # single sentence: the reversal is a plain flip, so the backward decoder's input can be written down directly
        labels, inputs = t[1:], t[:-1]
        rev_in = PackedSeqs(labels.flip(0), torch.arange(len(labels)), torch.tensor([0, len(labels)], dtype=torch.int32), len(labels))
        src = one["src"]
        rev_hidden = m.mirror_decoder(rev_in, one["context_packed"], src)
        logits = m.mirror_generator(rev_hidden).float()
        rev_ref = torch.nn.functional.cross_entropy(logits, inputs.flip(0), reduction="sum")
        mir_ref = (m.mirror_g(one["hidden_packed"][:len(labels)]) - rev_hidden.flip(0)).pow(2).sum() / 32
        assert torch.allclose(one["rev_loss"], rev_ref, rtol=1e-4, atol=1e-4)
        assert torch.allclose(one["mirror_loss"], mir_ref, rtol=1e-4, atol=1e-4)
        rev, mir, nmt = rev + float(rev_ref), mir + float(mir_ref), nmt + float(one["nmt_loss"].sum())
    assert abs(float(whole["rev_loss"]) - rev) < 1e-3 * max(1.0, rev)
    assert abs(float(whole["mirror_loss"]) - mir) < 1e-3 * max(1.0, mir)
    assert abs(float(whole["loss"].sum()) - (nmt + rev + 0.5 * mir)) < 1e-3 * (nmt + rev + mir)
    whole["loss"].sum().backward()
    assert m.mirror_g.weight.grad.abs().sum() > 0
    assert all(p.grad is not None for p in m.mirror_decoder.parameters() if p.requires_grad)


def test_reconstruction_decoder_trains_and_is_off_in_eval():
    m = _model(["-reconstruct"])
    out = m(collate(SRC, TGT, padded=True, packed=True))
    assert "rec_loss" in out and float(out["rec_loss"]) > 0
    assert abs(float(out["loss"].sum()) - float(out["nmt_loss"].sum()) - float(out["rec_loss"])) < 1e-3
    out["loss"].sum().backward()
    assert m.rec_linear.weight.grad.abs().sum() > 0
    # the reconstruction labels are the source itself: a uniform model scores log(V) per source word
    n_src = sum(len(s) for s in SRC)
    assert 0.3 * n_src * torch.log(torch.tensor(34.0)) < float(out["rec_loss"]) < 3.0 * n_src * torch.log(torch.tensor(34.0))
    m.eval()
    with torch.no_grad():
        ev = m(collate(SRC, TGT, padded=True, packed=True))
    assert "rec_loss" not in ev and "nmt_loss" not in ev
