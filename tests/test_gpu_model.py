"""End-to-end: the fused bf16 Transformer on the GPU against the fp32 PyTorch path of the same model."""
import copy

import pytest
import torch

from nmtgminor_b200 import ops
from nmtgminor_b200.data.synthetic import synthetic_dict, token_budget_batches
from nmtgminor_b200.models.transformer import Transformer
from nmtgminor_b200.options import default_options
from nmtgminor_b200.parallel.flat import FlatParameterStore
from nmtgminor_b200.train.engine import TrainEngine

pytestmark = pytest.mark.gpu


def _opt(extra=()):
    return default_options(["-model_size", "256", "-layers", "2", "-n_heads", "4", "-inner_size", "1024", "-tie_weights",
                            "-join_embedding", "-ffn_activation", "relu", "-label_smoothing", "0.1", "-optim", "adam",
                            "-learning_rate", "1e-3", "-update_method", "regular", "-dropout", "0.0", "-attn_dropout", "0.0",
                            "-emb_dropout", "0.0", "-weight_decay", "0.01"] + list(extra))


def test_fused_model_matches_fp32_reference():
    torch.manual_seed(0)
    d = synthetic_dict(2000)
    opt = _opt()
    cpu_model = Transformer(opt, {"src": d, "tgt": d})
    gpu_model = copy.deepcopy(cpu_model)
    batch = token_budget_batches(2000, 5, 40, 600, 1, seed=3, static=True, padded=False)[0]
    out = cpu_model(batch)
    out["loss"].backward()
    store = FlatParameterStore(gpu_model, "cuda")
    for b in gpu_model.buffers():
        b.data = b.data.cuda()
    gbatch = copy.deepcopy(batch).cuda("cuda", hot_only=True)
    gout = gpu_model(gbatch)
    gout["loss"].backward()
    torch.cuda.synchronize()
    assert ops.check_status() == 0
    n = batch.tgt_size
    assert abs(gout["loss"].item() - out["loss"].item()) / n < 3e-2, (gout["loss"].item() / n, out["loss"].item() / n)
    worst = 0.0
    for (name, p), (_, q) in zip(cpu_model.named_parameters(), gpu_model.named_parameters()):
        if p.grad is None:
            continue
        g = q.main_grad.float().cpu()
        denom = p.grad.abs().max().item() + 1e-6
        err = (g - p.grad).abs().max().item() / denom
        worst = max(worst, err)
        assert err < 0.12, "gradient of %s: relative max error %.3f" % (name, err)
    print("worst relative gradient error", worst)


@pytest.mark.parametrize("graph", [False, True])
def test_engine_trains(graph):
    torch.manual_seed(1)
    d = synthetic_dict(2000)
    opt = _opt(["-dropout", "0.1", "-attn_dropout", "0.1"])
    model = Transformer(opt, {"src": d, "tgt": d})
    eng = TrainEngine(model, opt, device="cuda", cuda_graph=graph)
    batches = [b.pin_memory() for b in token_budget_batches(2000, 5, 40, 1024, 4, seed=5, static=True, padded=False)]
    first = last = None
    for it in range(30):
        b = batches[it % len(batches)]
        loss, _ = eng.train_step(b)
        val = loss.item() / b.tgt_size
        first = val if first is None else first
        last = val
    assert ops.check_status() == 0
    assert last < first - 0.5, "loss did not go down: %.3f -> %.3f" % (first, last)


def test_graph_capture_waits_for_the_third_batch_of_a_class_when_asked():
    """Trainers that stream a token-budget data set capture a shape class at its third batch: rare classes stay eager."""
    torch.manual_seed(1)
    d = synthetic_dict(2000)
    opt = _opt(["-dropout", "0.1", "-attn_dropout", "0.1"])
    model = Transformer(opt, {"src": d, "tgt": d})
    eng = TrainEngine(model, opt, device="cuda", cuda_graph=True)
    eng.capture_after = 3
    a, b = [x.pin_memory() for x in token_budget_batches(2000, 5, 40, 1024, 2, seed=5, static=True, padded=False)]
    sizes = []
    for batch in (a, a, b, a, a, b, b, b):
        eng.train_step(batch)
        sizes.append(len(eng._graphs))
    same_class = eng._seen.keys().__len__() == 1
    assert sizes == ([0, 0, 1, 1, 1, 1, 1, 1] if same_class else [0, 0, 0, 1, 1, 1, 2, 2])
    assert ops.check_status() == 0
    # a full cache that may not evict leaves new classes to the eager path
    eng.max_graphs, eng.evict_graphs = len(eng._graphs), False
    c = token_budget_batches(2000, 5, 40, 2048, 1, seed=9, static=True, padded=False)[0].pin_memory()
    before = len(eng._graphs)
    for _ in range(4):
        eng.train_step(c)
    assert len(eng._graphs) == before


def test_checkpointing_replays_fused_dropout_masks():
    """Recomputed layers must regenerate the dropout masks of the first pass: gradients match the plain run."""
    d = synthetic_dict(2000)
    batch = token_budget_batches(2000, 5, 40, 600, 1, seed=3, static=True, padded=False)[0]
    grads, losses = [], []
    for extra in ([], ["-checkpointing", "2"]):
        torch.manual_seed(0)
        opt = _opt(["-dropout", "0.1", "-attn_dropout", "0.1", "-emb_dropout", "0.1"] + extra)
        model = Transformer(opt, {"src": d, "tgt": d}).train()
        store = FlatParameterStore(model, "cuda")
        for b in model.buffers():
            b.data = b.data.cuda()
        ops.manual_seed(77)
        ops.reset_stream_counter()
        out = model(copy.deepcopy(batch).cuda("cuda", hot_only=True))
        out["loss"].backward()
        torch.cuda.synchronize()
        grads.append(store.grad.clone())
        losses.append(out["loss"].item())
    assert ops.check_status() == 0
    assert abs(losses[0] - losses[1]) < 1e-3 * abs(losses[0])
    denom = grads[0].abs().max().item()
    assert (grads[0] - grads[1]).abs().max().item() / denom < 2e-2


def test_chunked_generator_loss_matches_unchunked():
    """Rows processed 512 at a time through one scratch buffer give the loss and gradients of the one-shot path."""
    d = synthetic_dict(2000)
    batch = token_budget_batches(2000, 5, 40, 1500, 1, seed=4, static=True, padded=False)[0]
    res = []
    for extra in ([], ["-generator_chunk_rows", "512"]):
        torch.manual_seed(0)
        model = Transformer(_opt(extra), {"src": d, "tgt": d}).train()
        store = FlatParameterStore(model, "cuda")
        for b in model.buffers():
            b.data = b.data.cuda()
        out = model(copy.deepcopy(batch).cuda("cuda", hot_only=True), grad_scale=1.0)
        out["loss"].backward()
        torch.cuda.synchronize()
        res.append((out["loss"].item(), out["correct"].item(), store.grad.clone(), out["row_loss"].clone()))
    assert ops.check_status() == 0
    assert abs(res[0][0] - res[1][0]) < 1e-3 * abs(res[0][0]) and res[0][1] == res[1][1]
    assert torch.allclose(res[0][3], res[1][3], atol=1e-3)
    denom = res[0][2].abs().max().item()
    assert (res[0][2] - res[1][2]).abs().max().item() / denom < 2e-2


def test_forward_is_bitwise_deterministic_for_a_seed():
    """Same seed, same batch: dropout masks, attention and GEMM results repeat bit for bit (the forward pass has no
    atomics); a different seed changes the masks."""
    d = synthetic_dict(2000)
    batch = token_budget_batches(2000, 5, 40, 600, 1, seed=3, static=True, padded=False)[0]
    torch.manual_seed(0)
    model = Transformer(_opt(["-dropout", "0.2", "-attn_dropout", "0.1", "-emb_dropout", "0.1"]), {"src": d, "tgt": d}).train()
    FlatParameterStore(model, "cuda")
    for b in model.buffers():
        b.data = b.data.cuda()
    gb = copy.deepcopy(batch).cuda("cuda", hot_only=True)
    outs = []
    for seed in (11, 11, 12):
        ops.manual_seed(seed)
        ops.reset_stream_counter()
        with torch.no_grad():
            out = model(gb)
        outs.append((out["loss"].clone(), out["row_loss"].clone()))
    torch.cuda.synchronize()
    assert torch.equal(outs[0][1], outs[1][1]) and torch.allclose(outs[0][0], outs[1][0], rtol=1e-5)   # the sum uses atomics
    assert not torch.equal(outs[0][1], outs[2][1])
    assert ops.ext().bounds_violations() in (-1, 0)


def test_lora_adapters_train_on_the_fused_path_and_leave_frozen_weights_alone():
    from nmtgminor_b200.train import finetune as ft
    from nmtgminor_b200.train.engine import TrainEngine
    torch.manual_seed(0)
    d = synthetic_dict(2000)
    opt = _opt(["-weight_decay", "0.1"])
    model = Transformer(opt, {"src": d, "tgt": d})
    replaced = ft.apply_lora(model, r=8, alpha=16)
    assert replaced
    eng = TrainEngine(model, opt, device="cuda", cuda_graph=False)
    store = eng.store
    n_train = sum(p.numel() for p in model.parameters() if p.requires_grad)
    assert 0 < store.trainable_total < store.total and eng.optim.exp_avg.numel() == store.trainable_total
    assert store.trainable_total < n_train * 2 + 64 * len(replaced) * 4
    frozen_before = store.master[store.trainable_total:].clone()
    batches = [b.pin_memory() for b in token_budget_batches(2000, 5, 40, 1024, 2, seed=5, static=True)]
    losses = []
    for it in range(12):
        loss, _ = eng.train_step(batches[it % 2])
        losses.append(loss.item() / batches[it % 2].tgt_size)
    torch.cuda.synchronize()
    assert ops.check_status() == 0
    assert torch.equal(store.master[store.trainable_total:], frozen_before)      # no update, no weight decay
    assert losses[-1] < losses[0]


@pytest.mark.parametrize("graph", [False, True])
def test_every_step_draws_new_dropout_masks(graph):
    """With a learning rate of zero the parameters never move, so two steps on the same batch differ only through
    their dropout masks: equal losses would mean the masks repeat from step to step."""
    torch.manual_seed(1)
    d = synthetic_dict(2000)
    opt = _opt(["-dropout", "0.3", "-attn_dropout", "0.1", "-learning_rate", "0.0"])
    model = Transformer(opt, {"src": d, "tgt": d})
    eng = TrainEngine(model, opt, device="cuda", cuda_graph=graph)
    batch = token_budget_batches(2000, 5, 40, 1024, 1, seed=5, static=True, padded=False)[0].pin_memory()
    losses = [eng.train_step(batch)[0].item() for _ in range(4)]
    assert len(set(losses)) == len(losses), "dropout masks repeat: %r" % (losses,)
    # accumulation micro-batches get their own masks too
    a = eng.train_step(batch, update=False)[0].item()
    b = eng.train_step(batch, update=True)[0].item()
    assert a != b


def test_rng_state_round_trip_restores_the_device_seed_word():
    from nmtgminor_b200.train.checkpoint import restore_rng_state, rng_state
    word = ops.ext().get_seed_tensor(torch.cuda.current_device())
    ops.advance_device_seed(by=5)
    saved = rng_state()
    want = int(word.item())
    ops.advance_device_seed(by=3)
    assert int(word.item()) == want + 3
    restore_rng_state(saved)
    assert int(word.item()) == want
