import torch

from nmtgminor_b200.data.synthetic import synthetic_dict, token_budget_batches
from nmtgminor_b200.models.efficient_attention import LSHAttention, MaxOut, PerceiverBottleneck, PerformerAttention, softmax_kernel
from nmtgminor_b200.models.efficient_attention import gaussian_orthogonal_random_matrix
from nmtgminor_b200.models.transformer import Transformer
from nmtgminor_b200.options import default_options
from nmtgminor_b200.parallel.flat import FlatParameterStore
from nmtgminor_b200.train import finetune as FT


def _model(seed=0):
    torch.manual_seed(seed)
    d = synthetic_dict(60)
    opt = default_options(["-model_size", "32", "-layers", "1", "-n_heads", "2", "-inner_size", "64", "-ffn_activation", "relu",
                           "-tie_weights", "-join_embedding", "-dropout", "0.0", "-attn_dropout", "0.0", "-emb_dropout", "0.0"])
    return Transformer(opt, {"src": d, "tgt": d})


def test_lora_trains_only_adapters_and_merges():
    model = _model()
    batch = token_budget_batches(60, 4, 10, 120, 1, seed=1, padded=False)[0]
    model.eval()
    base_loss = model(batch)["loss"].item()
    replaced = FT.apply_lora(model, r=4, alpha=8)
    assert replaced and all(("lora_" in n) == p.requires_grad for n, p in model.named_parameters())
    assert abs(model(batch)["loss"].item() - base_loss) < 1e-4          # B starts at zero
    model.train()
    opt = torch.optim.Adam([p for p in model.parameters() if p.requires_grad], lr=0.05)
    for _ in range(10):
        opt.zero_grad()
        model(batch)["loss"].backward()
        opt.step()
    model.eval()
    tuned = model(batch)["loss"].item()
    assert tuned < base_loss
    assert FT.merge_lora(model) == len(replaced)
    assert abs(model(batch)["loss"].item() - tuned) < 1e-2 * abs(tuned)


def test_flat_ema_and_distillation():
    model = _model()
    store = FlatParameterStore(model, "cpu")
    ema = FT.FlatEMA(store, decay=0.5)
    before = store.master.clone()
    store.master.add_(1.0)
    ema.update()
    assert torch.allclose(ema.shadow, before + 0.5)
    ema.swap_in()
    assert torch.allclose(store.master, before + 0.5)
    ema.swap_out()
    assert torch.allclose(store.master, before + 1.0)
    student, teacher = _model(1), _model(2)
    batch = token_budget_batches(60, 4, 10, 120, 1, seed=1, padded=False)[0]
    loss = FT.distill_step(student, teacher.eval(), batch, alpha=0.7)
    loss.backward()
    assert torch.isfinite(loss) and any(p.grad is not None for p in student.parameters())
    same = FT.distillation_loss(torch.randn(5, 7), torch.randn(5, 7), torch.tensor([1, 2, 0, 3, 4]), alpha=1.0)
    logits = torch.randn(5, 7)
    assert FT.distillation_loss(logits, logits, torch.tensor([1, 2, 0, 3, 4]), alpha=1.0).abs() < 1e-5 < same


def test_batch_ensemble_members_differ():
    torch.manual_seed(0)
    be = FT.BatchEnsembleLinear(8, 6, members=2)
    x = torch.randn(1, 8).repeat(4, 1)
    y = be(x)
    assert torch.allclose(y[0], y[1]) and not torch.allclose(y[0], y[3])


def test_performer_approximates_softmax_attention():
    torch.manual_seed(0)
    proj = gaussian_orthogonal_random_matrix(512, 16)
    q, k = 0.5 * torch.randn(1, 1, 6, 16), 0.5 * torch.randn(1, 1, 6, 16)
    approx = softmax_kernel(q, proj, True) @ softmax_kernel(k, proj, False).transpose(-1, -2)
    approx = approx / approx.sum(-1, keepdim=True)
    exact = torch.softmax(q @ k.transpose(-1, -2) / 4.0, -1)
    assert (approx - exact).abs().max() < 0.08
    att = PerformerAttention(32, 2, causal=True)
    x = torch.randn(2, 9, 32)
    y = att(x)
    y2 = att(torch.cat([x[:, :5], torch.randn(2, 4, 32)], 1))
    assert torch.allclose(y[:, :5], y2[:, :5], atol=2e-3)                 # causal (up to the eps of the feature map)


def test_lsh_perceiver_maxout_shapes_and_masks():
    torch.manual_seed(0)
    x = torch.randn(2, 12, 32)
    pad = torch.zeros(2, 12, dtype=torch.bool)
    pad[1, 8:] = True
    assert LSHAttention(32, 2)(x, pad).shape == x.shape
    lat = PerceiverBottleneck(32, 2, n_latents=5, layers=1).eval()
    a = lat(x, pad)
    x2 = x.clone()
    x2[1, 8:] = 100.0
    assert a.shape == (2, 5, 32) and torch.allclose(a, lat(x2, pad), atol=1e-4)       # padded frames are ignored
    assert MaxOut(32, 7, 3)(x).shape == (2, 12, 7)


def test_distillation_wrapper_trains_through_the_engine():
    from nmtgminor_b200.train.engine import TrainEngine
    student, teacher = _model(1), _model(2)
    wrapper = FT.DistillationWrapper(student, teacher, alpha=0.5)
    assert all(not p.requires_grad for p in teacher.parameters())
    assert len(list(wrapper.parameters())) == len(list(student.parameters()))
    opt = default_options(["-model_size", "32", "-layers", "1", "-n_heads", "2", "-inner_size", "64", "-optim", "adam", "-learning_rate",
                           "0.01", "-update_method", "regular"])
    eng = TrainEngine(wrapper, opt, device="cpu")
    batch = token_budget_batches(60, 4, 10, 120, 1, seed=1, padded=False)[0]
    first = eng.train_step(batch)[0].item()
    for _ in range(8):
        last = eng.train_step(batch)[0].item()
    assert last < first
    wrapper.eval()
    assert "loss" in wrapper(batch)


def test_reformer_layer_and_chunked_forward():
    from nmtgminor_b200.models.efficient_attention import ReformerEncoderLayer, apply_chunking_to_forward
    torch.manual_seed(0)
    lin = torch.nn.Linear(8, 8)
    x = torch.randn(2, 10, 8)
    assert torch.allclose(apply_chunking_to_forward(3, 1, lin, x), lin(x), atol=1e-6)       # ragged last slice
    assert torch.equal(apply_chunking_to_forward(0, 1, lin, x), lin(x))
    layer = ReformerEncoderLayer(32, 4, 64, dropout=0.0, ffn_chunk=4).eval()
    whole = ReformerEncoderLayer(32, 4, 64, dropout=0.0, ffn_chunk=0).eval()
    whole.load_state_dict(layer.state_dict())
    h = torch.randn(2, 12, 32)
    assert torch.allclose(layer(h), whole(h), atol=1e-5)
    pad = torch.zeros(2, 12, dtype=torch.bool)
    pad[1, 8:] = True
    out = layer(h, pad)
    h2 = h.clone()
    h2[1, 8:] = 0.0
    assert torch.allclose(out[1, :8], layer(h2, pad)[1, :8], atol=1e-5)                      # padded frames are not attended to
    drop = ReformerEncoderLayer(32, 4, 64, death_rate=1.0 - 1e-9).train()
    assert torch.equal(drop(h), h)
