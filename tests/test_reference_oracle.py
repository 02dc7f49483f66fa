"""Step-for-step comparison with the installed reference on the CPU (tiny Transformer, fp32).

The reference package under ``baseline/_ref`` builds its own model; its state dict is loaded into this framework's
Transformer through the checkpoint key map, both see the same equal-length batch (on ragged batches the reference's
loss mixes up the B x T and T x B layouts of its mask, so only equal lengths are comparable), and the summed loss
and every parameter gradient must agree.  Skipped when the reference is not installed."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

VOCAB = 500


def _reference_runner():
    from bench_reference import ReferenceRunner, reference_available
    ok, why = reference_available()
    if not ok:
        pytest.skip(why)
    try:
        return ReferenceRunner(VOCAB, "cpu", tiny=True, argv_extra=["-dropout", "0.0", "-attn_dropout", "0.0", "-emb_dropout", "0.0",
                                                                   "-word_dropout", "0.0", "-death_rate", "0.0"])
    except Exception as exc:  # noqa: BLE001
        pytest.skip("the reference did not build here: %r" % (exc,))


def _ours():
    from nmtgminor_b200.data.synthetic import synthetic_dict
    from nmtgminor_b200.models.transformer import Transformer
    from nmtgminor_b200.options import default_options
    opt = default_options(["-model", "transformer", "-layers", "2", "-model_size", "256", "-n_heads", "4", "-inner_size", "1024",
                           "-dropout", "0.0", "-attn_dropout", "0.0", "-emb_dropout", "0.0", "-ffn_activation", "relu", "-tie_weights",
                           "-join_embedding", "-label_smoothing", "0.1"])
    d = synthetic_dict(VOCAB)
    return Transformer(opt, {"src": d, "tgt": d})


def test_loss_and_gradients_match_the_reference_on_an_equal_length_batch():
    from nmtgminor_b200.data.dataset import collate
    from nmtgminor_b200.train.checkpoint import load_model_state, transformer_to_reference
    runner = _reference_runner()
    ref_model = runner.raw_model
    ref_model.train()
    ours = _ours()
    missing, unexpected = load_model_state(ours, {k: v.detach().clone() for k, v in ref_model.state_dict().items()})
    assert not missing, missing
    ours.train()

    rng = np.random.RandomState(0)
    n, ls, lt = 6, 11, 9
    src = [torch.from_numpy(rng.randint(4, VOCAB, size=ls).astype(np.int64)) for _ in range(n)]
    tgt = [torch.from_numpy(np.concatenate([[2], rng.randint(4, VOCAB, size=lt), [3]]).astype(np.int64)) for _ in range(n)]

    # reference: its own collate, forward, loss
    from onmt.data.dataset import rewrap
    rb = rewrap(runner.collate(src, tgt))
    targets = rb.get("target_output")
    tgt_mask = rb.get("target_input_selfattn_mask")
    outputs = ref_model(rb, streaming=False, target_mask=tgt_mask, zero_encoder=False, mirror=False, streaming_state=None, nce=False,
                        pretrained_layer_states=None, adv_ptb_grad=False, checkpointing_ffn=False, checkpointing_cross_attn=False,
                        checkpointing_self_attn=False, ctc_loss_function=None, ctc_labels=targets, grad_scaler=None, ctc_coeff=0.0)
    outputs["tgt_mask"] = tgt_mask
    loss_dict = runner.loss_function(outputs, targets, model=ref_model)
    ref_loss = loss_dict["loss"]
    ref_model.zero_grad()
    ref_loss.backward()

    out = ours(collate(src, tgt, padded=False, packed=True))
    our_loss = out["loss"].sum()
    ours.zero_grad()
    our_loss.backward()
    assert abs(float(our_loss) - float(ref_loss)) < 1e-4 * abs(float(ref_loss)), (float(our_loss), float(ref_loss))

    # gradients, compared in the reference's naming (fused projections are split by the key map)
    ref_grads = {k: p.grad for k, p in ref_model.named_parameters() if p.grad is not None}
    our_grads = transformer_to_reference({k: (p.grad if p.grad is not None else torch.zeros_like(p))
                                          for k, p in ours.state_dict(keep_vars=True).items()})     # tied weights under every name
    checked = 0
    for k, g in ref_grads.items():
        if k not in our_grads:
            continue
        a, b = our_grads[k], g.detach().float()
        scale = b.abs().max().item() + 1e-8
        assert (a - b).abs().max().item() < 2e-4 * scale + 1e-6, "gradient of %s differs: %g (scale %g)" % (k, (a - b).abs().max().item(), scale)
        checked += 1
    assert checked >= 20, "only %d gradients were comparable" % checked


def test_our_checkpoint_loads_into_the_reference_model():
    """The other direction of the key map: a state dict saved by this framework restores the reference's model."""
    from nmtgminor_b200.train.checkpoint import model_state_for_saving
    runner = _reference_runner()
    ours = _ours()
    saved = model_state_for_saving(ours)
    ref_model = runner.raw_model
    want = set(k for k in ref_model.state_dict() if "positional_encoder" not in k and not k.endswith("decoder.mask"))
    assert want <= set(saved.keys()) | {k for k in want if "time_transformer" in k}, sorted(want - set(saved.keys()))[:5]
    ref_model.load_state_dict(saved, strict=False)
    back = ref_model.state_dict()
    for k in ("encoder.layer_modules.0.multihead.fc_query.function.linear.weight", "generator.0.linear.weight",
              "decoder.layer_modules.1.feedforward.function.fc_2.linear.bias"):
        assert torch.allclose(back[k], saved[k])
