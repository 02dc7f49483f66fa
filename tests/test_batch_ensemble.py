"""Batch-ensemble weights: member selection per sentence in training, member averaging in evaluation, model conversion."""
import torch

from nmtgminor_b200.data.dataset import collate
from nmtgminor_b200.data.synthetic import synthetic_dict
from nmtgminor_b200.models.factory import build_model
from nmtgminor_b200.models.layers import FeedForward, PackedSeqs
from nmtgminor_b200.modules.batch_ensemble import (BatchEnsembleFeedForward, BatchEnsembleLinear, convert_to_batch_ensemble,
                                                   members_of_rows)
from nmtgminor_b200.options import default_options


def test_linear_matches_the_definition():
    torch.manual_seed(0)
    lin = BatchEnsembleLinear(6, 5, 3, init="normal")
    x = torch.randn(7, 6)
    rows = torch.tensor([0, 0, 1, 1, 1, 2, 2])
    lin.train()
    y = lin(x, row_members=rows)
    for i in range(7):
        e = int(rows[i])
        w_e = lin.weight * (lin.s[e][:, None] * lin.r[e][None, :])
        assert torch.allclose(y[i], x[i] @ w_e.t() + lin.bias, atol=1e-5)
    lin.eval()
    avg = lin(x)
    ref = sum(x @ (lin.weight * (lin.s[e][:, None] * lin.r[e][None, :])).t() for e in range(3)) / 3 + lin.bias
    assert torch.allclose(avg, ref, atol=1e-5)
    # padded [T, B, in]: sentence b -> member b mod E
    lin.train()
    xp = torch.randn(4, 5, 6)
    yp = lin(xp)
    assert torch.allclose(yp[:, 4], lin(xp[:, 4], row_members=torch.full((4,), 4 % 3)), atol=1e-5)


def test_members_of_rows():
    cu = torch.tensor([0, 2, 5, 6, 9], dtype=torch.int32)
    assert members_of_rows(cu, 9, 3).tolist() == [0, 0, 1, 1, 1, 2, 0, 0, 0]
    assert members_of_rows(cu, 9, 3, torch.tensor([2, 2, 0, 1])).tolist() == [2, 2, 2, 2, 2, 0, 1, 1, 1]


def test_feed_forward_members_and_average():
    torch.manual_seed(1)
    ffn = FeedForward(8, 16, 0.0, "relu")
    be = BatchEnsembleFeedForward(ffn, 2, init="normal")
    assert be.fc1 is ffn.fc1
    x = torch.randn(6, 8)
    seqs = PackedSeqs(torch.zeros(6, dtype=torch.long), torch.zeros(6, dtype=torch.long), torch.tensor([0, 2, 6], dtype=torch.int32), 4)
    be.train()
    y = be(x, residual=x, seqs=seqs)

    def member(e, rows):
        h = torch.relu(((rows * be.r_in[e]) @ ffn.fc1.weight.t()) * be.s_in[e] + ffn.fc1.bias)
        return ((h * be.r_out[e]) @ ffn.fc2.weight.t()) * be.s_out[e] + ffn.fc2.bias

    assert torch.allclose(y[:2], x[:2] + member(0, x[:2]), atol=1e-5)
    assert torch.allclose(y[2:], x[2:] + member(1, x[2:]), atol=1e-5)
    be.eval()
    ev = be(x, residual=x)
    assert torch.allclose(ev, x + 0.5 * (member(0, x) + member(1, x)), atol=1e-5)
    forced = be(x, residual=None, seqs=seqs, members=torch.tensor([1, 1]))
    assert torch.allclose(forced, member(1, x), atol=1e-5)


def test_model_conversion_and_freezing():
    torch.manual_seed(0)
    d = synthetic_dict(30)
    opt = default_options(["-model_size", "32", "-layers", "2", "-n_heads", "1", "-inner_size", "64", "-ffn_activation", "relu",
                           "-batch_ensemble", "3", "-dropout", "0", "-attn_dropout", "0", "-word_dropout", "0", "-emb_dropout", "0"])
    m = build_model(opt, {"src": d, "tgt": d})
    blocks = [x for x in m.modules() if isinstance(x, BatchEnsembleFeedForward)]
    assert len(blocks) == 4 and all(b.n_ensembles == 3 for b in blocks)
    b = collate([torch.tensor([5, 6, 7]), torch.tensor([8, 9])], [torch.tensor([2, 8, 9, 3]), torch.tensor([2, 4, 3])],
                padded=True, packed=True)
    m.train()
    out = m(b)
    out["loss"].sum().backward()
    g = blocks[0].r_in.grad
    assert g[0].abs().sum() > 0 and g[1].abs().sum() > 0 and g[2].abs().sum() == 0      # two sentences -> members 0 and 1
    m.eval()
    with torch.no_grad():
        assert torch.isfinite(m(b)["loss"]).all()
    plain = build_model(default_options(["-model_size", "32", "-layers", "1", "-n_heads", "1", "-inner_size", "64"]), {"src": d, "tgt": d})
    n = convert_to_batch_ensemble(plain, 2, init="ones", freeze_shared=True)
    assert n == 2
    trainable = [k for k, p in plain.named_parameters() if p.requires_grad]
    assert trainable and all(k.rsplit(".", 1)[-1] in ("r_in", "s_in", "r_out", "s_out") for k in trainable)
