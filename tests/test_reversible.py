import torch

from nmtgminor_b200.models.layers import PackedSeqs
from nmtgminor_b200.models.reversible import ReversibleStack


def _seqs(lengths):
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32)
    n = int(cu[-1])
    pos = torch.cat([torch.arange(l) for l in lengths])
    return PackedSeqs(torch.zeros(n, dtype=torch.long), pos, cu, max(lengths))


def test_reversible_stack_matches_plain_autograd():
    torch.manual_seed(0)
    src, tgt = _seqs([5, 3, 7]), _seqs([4, 6, 2])
    enc = ReversibleStack(2, 32, 2, 64, dropout=0.0, attn_dropout=0.0).train()
    dec = ReversibleStack(2, 32, 2, 64, dropout=0.0, attn_dropout=0.0, causal=True, cross=True).train()
    xs = torch.randn(15, 32)
    xt = torch.randn(12, 32)
    grads = []
    for plain in (True, False):
        for m in (enc, dec):
            m.zero_grad()
        a, b = xs.clone().requires_grad_(), xt.clone().requires_grad_()
        mem = enc(a, src, plain=plain)
        out = dec(b, tgt, mem, src, plain=plain)
        (out * torch.linspace(-1, 1, 32)).sum().backward()
        grads.append([a.grad.clone(), b.grad.clone()] + [p.grad.clone() for p in list(enc.parameters()) + list(dec.parameters())])
    for g_plain, g_rev in zip(*grads):
        assert torch.allclose(g_plain, g_rev, atol=2e-5, rtol=1e-4)
    # the reconstruction inside backward recovered the layer inputs
    x1, x2 = dec.layers[0]._last_inputs
    assert torch.allclose(x1, xt, atol=1e-4) and torch.allclose(x2, xt, atol=1e-4)


def test_reversible_flags_build_a_trainable_decodable_transformer():
    from nmtgminor_b200.data.synthetic import synthetic_dict, token_budget_batches
    from nmtgminor_b200.inference.beam_search import BeamConfig, beam_search
    from nmtgminor_b200.models.transformer import Transformer
    from nmtgminor_b200.options import default_options
    torch.manual_seed(0)
    d = synthetic_dict(60)
    opt = default_options(["-model_size", "32", "-layers", "2", "-n_heads", "2", "-inner_size", "64", "-ffn_activation", "relu",
                           "-tie_weights", "-join_embedding", "-src_reversible", "-tgt_reversible", "-dropout", "0.1"])
    model = Transformer(opt, {"src": d, "tgt": d}).train()
    assert model.encoder.reversible is not None and model.decoder.reversible is not None
    batch = token_budget_batches(60, 4, 10, 120, 1, seed=1, padded=True)[0]
    out = model(batch)
    out["loss"].backward()
    assert all(p.grad is not None for p in model.decoder.reversible.parameters())
    model.eval()
    hyps = beam_search(model, batch, BeamConfig(beam_size=2, max_len=5))
    assert len(hyps) == batch.size
