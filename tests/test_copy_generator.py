"""-copy_generator: the mixed generate / copy output distribution, its training loss and its use in beam search."""
import math

import torch

from nmtgminor_b200.data.dataset import collate
from nmtgminor_b200.data.synthetic import synthetic_dict
from nmtgminor_b200.inference.beam_search import BeamConfig, beam_search
from nmtgminor_b200.models.factory import build_model
from nmtgminor_b200.modules.copy_generator import CopyGenerator
from nmtgminor_b200.options import default_options


def test_distribution_is_normalised_and_copies_source_words():
    torch.manual_seed(0)
    g = CopyGenerator(8, 12)
    h, ctx = torch.randn(2, 3, 8), torch.randn(2, 4, 8)
    src = torch.tensor([[5, 6, 5, 0], [7, 8, 9, 10]])
    pad = src == 0
    logp = g(h, ctx, src, pad)
    assert logp.shape == (2, 3, 12) and torch.allclose(logp.exp().sum(-1), torch.ones(2, 3), atol=1e-5)
    # by hand for one position
    z = torch.sigmoid(g.linear_copy(h[0, 1]))
    p_gen = torch.softmax(g.linear(h[0, 1]), -1) * (1 - z)
    a = torch.softmax((ctx[0, :3] @ h[0, 1]), -1) * z
    want = p_gen.clone()
    want[5] += a[0] + a[2]
    want[6] += a[1]
    assert torch.allclose(logp[0, 1].exp(), want, atol=1e-6)
    # a gate forced open puts all the mass on source words
    g.linear_copy.bias.data.fill_(50.0)
    p = g(h, ctx, src, pad, log=False)
    assert float(p[1, :, [7, 8, 9, 10]].sum(-1).min()) > 0.999


def test_model_trains_and_decodes_with_the_copy_generator():
    torch.manual_seed(0)
    d = synthetic_dict(30)
    opt = default_options(["-model_size", "32", "-layers", "1", "-n_heads", "1", "-inner_size", "64", "-ffn_activation", "relu",
                           "-tie_weights", "-join_embedding", "-copy_generator", "-dropout", "0", "-attn_dropout", "0",
                           "-word_dropout", "0", "-emb_dropout", "0", "-label_smoothing", "0.1"])
    m = build_model(opt, {"src": d, "tgt": d})
    assert m.copy_generator.linear.weight is m.generator.weight and not m.supports_logits_step
    src = [torch.tensor([5, 6, 7, 8]), torch.tensor([9, 10])]
    tgt = [torch.tensor([2, 5, 6, 7, 8, 3]), torch.tensor([2, 9, 10, 3])]       # the task: copy the source
    b = collate(src, tgt, padded=True, packed=True, round_to=1)
    m.train()
    opt_ = torch.optim.Adam(m.parameters(), lr=5e-3)
    first = None
    for _ in range(60):
        opt_.zero_grad()
        out = m(b)
        loss = out["loss"].sum()
        first = first if first is not None else float(loss)
        loss.backward()
        opt_.step()
    assert float(loss) < 0.5 * first and math.isfinite(float(loss))
    m.eval()
    with torch.no_grad():
        hyps = beam_search(m, b, BeamConfig(beam_size=2, max_len=8, bos=2, eos=3, pad=0))
    assert hyps[0][0].tokens[:4] == [5, 6, 7, 8] and hyps[1][0].tokens[:2] == [9, 10]
