"""wav2vec 2.0 feature / code extraction tools: wav list -> Kaldi ark / scp and per-frame discrete units."""
import numpy as np
import pytest
import torch

from nmtgminor_b200.data.audio import read_ark_matrix, read_scp, write_wav
from nmtgminor_b200.models.speech_encoders import Wav2Vec2Encoder
from nmtgminor_b200.tools.extract import _batches, encoder_frames, extract_codes, extract_tdnn, load_speech_encoder
from nmtgminor_b200.tools.kmeans import learn_kmeans

CONV = [(16, 10, 5), (16, 3, 2), (16, 2, 2)]


def _fairseq_checkpoint(path, with_quantizer=True):
    """A fairseq-format pre-training checkpoint of a tiny encoder with random weights."""
    torch.manual_seed(0)
    from nmtgminor_b200.models.pretrained_io import wav2vec2_to_reference
    enc = Wav2Vec2Encoder(dim=32, layers=2, heads=2, ffn=64, dropout=0.0, attn_dropout=0.0, conv_layers=CONV, conv_bias=True,
                          pos_kernel=8, pos_groups=4)
    model = wav2vec2_to_reference(enc.state_dict(), 2) if callable(wav2vec2_to_reference) else enc.state_dict()
    if with_quantizer:
        model["quantizer.vars"] = torch.rand(1, 2 * 5, 4)
        model["quantizer.weight_proj.weight"] = torch.randn(10, 16)
        model["quantizer.weight_proj.bias"] = torch.zeros(10)
    cfg = {"encoder_embed_dim": 32, "encoder_layers": 2, "encoder_attention_heads": 2, "encoder_ffn_embed_dim": 64,
           "layer_norm_first": True, "extractor_mode": "layer_norm", "conv_bias": True, "latent_groups": 2, "conv_pos": 8, "conv_pos_groups": 4,
           "conv_feature_layers": "[(16, 10, 5)] + [(16, 3, 2)] + [(16, 2, 2)]"}
    torch.save({"cfg": {"model": cfg}, "model": model}, path)
    return enc


def _wavs(tmp_path, lens=(4000, 2500, 3100)):
    rng = np.random.RandomState(0)
    lines = []
    for i, n in enumerate(lens):
        p = tmp_path / ("u%d.wav" % i)
        write_wav(str(p), (rng.randn(n) * 0.1).astype(np.float32), 16000)
        lines.append("utt%d %s" % (i, p))
    lines.append("utt_seg %s 0.05 0.15" % (tmp_path / "u0.wav"))
    lst = tmp_path / "wav.list"
    lst.write_text("\n".join(lines) + "\n")
    return str(lst)


def test_batches_respect_the_sample_budget():
    items = [("a", torch.zeros(10)), ("b", torch.zeros(30)), ("c", torch.zeros(20)), ("d", torch.zeros(5))]
    groups = [u for u, _ in _batches(items, 60)]
    assert groups == [["a", "b"], ["c", "d"]]


def test_tdnn_features_to_ark_scp(tmp_path):
    ck = str(tmp_path / "w2v.pt")
    ref_enc = _fairseq_checkpoint(ck)
    lst = _wavs(tmp_path)
    ark, scp = str(tmp_path / "o.ark"), str(tmp_path / "o.scp")
    n = extract_tdnn(ck, lst, ark, scp, batch_samples=9000)
    assert n == 4
    index = read_scp(scp)
    assert list(index.keys()) == ["utt0", "utt1", "utt2", "utt_seg"]
    enc, quant = load_speech_encoder(ck)
    assert quant is not None and quant.groups == 2 and quant.entries == 5
    for utt, (path, off) in index.items():
        m = read_ark_matrix(path, off)
        assert m.shape[1] == 16 and m.shape[0] > 0
    # batching does not change an utterance's features, and the loaded weights are the checkpoint's
    from nmtgminor_b200.tools.extract import read_wav_list
    waves = dict(read_wav_list(lst))
    alone = encoder_frames(enc, [waves["utt1"]])[0]
    path, off = index["utt1"]
    assert np.allclose(read_ark_matrix(path, off), alone.numpy(), atol=1e-4)
    ref_enc.eval()
    with torch.no_grad():
        direct = ref_enc.extractor(waves["utt1"][None])[0]
    assert torch.allclose(alone, direct[:alone.shape[0]], atol=1e-4)
    assert abs(waves["utt_seg"].numel() - 1600) <= 2
    # the dump verifies against a recomputation with other batch boundaries; a changed model does not
    from nmtgminor_b200.tools.extract import verify_tdnn
    checked, worst = verify_tdnn(ck, lst, scp, batch_samples=100000, atol=1e-4)
    assert checked == 4 and worst < 1e-4
    import subprocess, sys, os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "verify_wav2vec2_feat.py"), "-model", ck, "-src", lst, "-scp", scp],
                       capture_output=True, text=True)
    assert r.returncode == 0 and "4 utterances match" in r.stdout, r.stdout + r.stderr
    other = str(tmp_path / "w2v_other.pt")
    state = torch.load(ck, weights_only=False)
    k = next(k for k in state["model"] if "feature_extractor" in k and state["model"][k].dim() == 3)
    state["model"][k] = state["model"][k] * 1.5
    torch.save(state, other)
    with pytest.raises(AssertionError, match="differs from the stored features"):
        verify_tdnn(other, lst, scp)
    # states after one Transformer layer
    n = extract_tdnn(ck, lst, ark, scp, layer=1)
    path, off = read_scp(scp)["utt0"]
    assert read_ark_matrix(path, off).shape[1] == 32


def test_codes_from_quantiser_and_kmeans(tmp_path):
    ck = str(tmp_path / "w2v.pt")
    _fairseq_checkpoint(ck)
    lst = _wavs(tmp_path)
    out = str(tmp_path / "codes.txt")
    assert extract_codes(ck, lst, out) == 4
    rows = [l.split() for l in open(out)]
    assert rows[0][0] == "utt0" and all(":" in c for c in rows[0][1:])
    g0 = {int(c.split(":")[0]) for r in rows for c in r[1:]}
    assert g0 <= set(range(5))
    enc, _ = load_speech_encoder(ck)
    from nmtgminor_b200.tools.extract import read_wav_list
    feats = encoder_frames(enc, [w for _, w in read_wav_list(lst)])
    km = learn_kmeans(feats, 3, epochs=2)
    kp = str(tmp_path / "km.pt")
    torch.save(km.state_dict(), kp)
    assert extract_codes(ck, lst, out, kmeans_path=kp) == 4
    rows = [l.split() for l in open(out)]
    assert len(rows[1]) - 1 == feats[1].shape[0] and {int(c) for c in rows[1][1:]} <= {0, 1, 2}
