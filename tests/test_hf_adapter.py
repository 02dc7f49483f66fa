"""Hugging Face style interface (input_features / labels -> loss, logits) around a speech-to-text model."""
import pytest
import torch

from nmtgminor_b200.data.synthetic import synthetic_dict
from nmtgminor_b200.models.factory import build_model
from nmtgminor_b200.options import default_options
from nmtgminor_b200.train.hf_adapter import HFSeq2SeqAdapter, SpeechSeq2SeqCollator, make_trainer, train_steps


def _adapter():
    torch.manual_seed(0)
    d = synthetic_dict(40)
    opt = default_options(["-model", "speech_transformer", "-encoder_type", "audio", "-input_size", "8", "-model_size", "32",
                           "-layers", "1", "-n_heads", "1", "-inner_size", "64", "-dropout", "0", "-attn_dropout", "0",
                           "-word_dropout", "0", "-emb_dropout", "0", "-label_smoothing", "0"])
    return HFSeq2SeqAdapter(build_model(opt, {"tgt": d}), pad_id=0, bos_id=2)


def _features(seed=0):
    g = torch.Generator().manual_seed(seed)
    return [{"input_features": torch.randn(8, 48, generator=g), "labels": torch.tensor([5, 6, 7, 3])},
            {"input_features": torch.randn(8, 32, generator=g), "labels": torch.tensor([9, 3])}]


def test_collator_and_forward():
    batch = SpeechSeq2SeqCollator()(_features())
    assert batch["input_features"].shape == (2, 8, 48) and batch["labels"].tolist() == [[5, 6, 7, 3], [9, 3, -100, -100]]
    assert batch["attention_mask"].sum(-1).tolist() == [48, 32]
    ad = _adapter().eval()
    out = ad(**batch, return_logits=True)
    assert out.n_tokens == 6 and out.logits.shape[:2] == (2, 4)
    # the loss is the mean cross-entropy of the labelled tokens under the returned logits
    lp = torch.log_softmax(out.logits.float(), -1)
    y = batch["labels"]
    nll = -(lp.gather(-1, y.clamp(min=0)[..., None]).squeeze(-1) * (y != -100)).sum() / 6
    assert torch.allclose(out.loss, nll, atol=1e-4)
    assert out[0] is out.loss and out["logits"] is out.logits


def test_plain_training_loop_learns():
    ad = _adapter()
    batch = SpeechSeq2SeqCollator()(_features())
    losses = train_steps(ad, [batch] * 25, lr=5e-3)
    assert losses[-1] < 0.6 * losses[0]


def test_trainer_factory_reports_the_missing_dependency():
    try:
        import accelerate  # noqa: F401
    except ImportError:
        with pytest.raises(ImportError, match="accelerate"):
            make_trainer(_adapter(), [], output_dir="/tmp/unused")
