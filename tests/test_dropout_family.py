import torch

from nmtgminor_b200 import constants as C
from nmtgminor_b200.data.synthetic import synthetic_dict, token_budget_batches
from nmtgminor_b200.models.transformer import Transformer
from nmtgminor_b200.modules import dropout as D
from nmtgminor_b200.options import default_options


def test_variational_dropout_shares_mask_over_time():
    torch.manual_seed(0)
    x = torch.ones(7, 3, 16)
    y = D.variational_dropout(x, 0.5, True)
    assert torch.equal(y[0], y[6]) and set(y.unique().tolist()) <= {0.0, 2.0}
    cu = torch.tensor([0, 3, 4, 9], dtype=torch.int32)
    yp = D.variational_dropout(torch.ones(12, 8), 0.5, True, cu=cu)     # 3 rows of static padding
    assert torch.equal(yp[0], yp[2]) and torch.equal(yp[4], yp[8])
    assert torch.equal(D.variational_dropout(x, 0.5, False), x)


def test_word_dropout_and_embedded_dropout():
    torch.manual_seed(0)
    tokens = torch.randint(4, 50, (200,))
    new, scale = D.word_dropout_tokens(tokens, 50, 0.3)
    dropped = new != tokens
    assert dropped.any() and abs(scale - 1 / 0.7) < 1e-6
    # a word type is dropped everywhere or nowhere
    for w in tokens[dropped].unique():
        assert bool((new[tokens == w] == C.PAD).all())
    emb = torch.nn.Embedding(50, 8, padding_idx=0)
    out = D.embedded_dropout(emb, tokens, 0.3)
    zero_rows = out.abs().sum(-1) == 0
    assert zero_rows.any() and not zero_rows.all()


def test_switchout_keeps_special_tokens():
    torch.manual_seed(0)
    words = torch.randint(4, 100, (6, 12))
    words[:, 0] = C.BOS
    words[:, -1] = C.EOS
    words[3, 6:] = C.PAD
    out = D.switchout(words, 100, tau=0.1)
    special = (words == C.BOS) | (words == C.EOS) | (words == C.PAD)
    assert torch.equal(out[special], words[special])
    assert (out != words).any() and int(out.max()) < 100
    cu = torch.tensor([0, 5, 12], dtype=torch.int32)
    packed = torch.randint(4, 100, (14,))
    packed[12:] = C.PAD
    changed = False
    for _ in range(20):
        outp = D.switchout_packed(packed, cu, 100, tau=0.05)
        assert torch.equal(outp[12:], packed[12:])
        changed |= bool((outp != packed).any())
    assert changed


def test_static_dropout_replays_mask():
    m = D.StaticDropout(0.5).train()
    x = torch.ones(4, 8)
    a = m(x, resample=True)
    assert torch.equal(a, m(x)) and not torch.equal(a, x)


def _model(extra):
    torch.manual_seed(0)
    d = synthetic_dict(60)
    opt = default_options(["-model_size", "32", "-layers", "2", "-n_heads", "2", "-inner_size", "64", "-ffn_activation", "relu",
                           "-tie_weights", "-join_embedding", "-dropout", "0.1"] + extra)
    return Transformer(opt, {"src": d, "tgt": d}).train()


def test_transformer_with_regularisation_options_trains():
    batch = token_budget_batches(60, 4, 10, 120, 1, seed=1, padded=False)[0]
    for extra in (["-variational_dropout"], ["-word_dropout", "0.2"], ["-switchout", "0.5"]):
        out = _model(extra)(batch)
        out["loss"].backward()
        assert torch.isfinite(out["loss"])


def test_checkpointing_gives_identical_gradients():
    batch = token_budget_batches(60, 4, 10, 120, 1, seed=1, padded=False)[0]
    grads = []
    for extra in ([], ["-checkpointing", "2"]):
        m = _model(extra + ["-dropout", "0.0", "-attn_dropout", "0.0", "-emb_dropout", "0.0"])
        out = m(batch)
        out["loss"].backward()
        grads.append(torch.cat([p.grad.reshape(-1) for p in m.parameters() if p.grad is not None]))
    assert torch.allclose(grads[0], grads[1], atol=1e-6)
