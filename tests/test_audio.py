import numpy as np
import torch

from nmtgminor_b200.data.audio import (Augmenter, LanguageModelDataset, SCPDataset, WavDataset, fbank, mel_filterbank, read_ark_matrix,
                                       read_scp, read_wav, stack_frames, whisper_log_mel, write_ark_matrix, write_wav)
from nmtgminor_b200.data.dataset import collate


def test_wav_roundtrip_and_segments(tmp_path):
    sr = 16000
    t = np.arange(sr) / sr
    wav = 0.5 * np.sin(2 * np.pi * 440 * t)
    p = str(tmp_path / "a.wav")
    write_wav(p, wav, sr)
    x, got_sr = read_wav(p)
    assert got_sr == sr and len(x) == sr and np.abs(x - wav).max() < 1e-3
    seg, _ = read_wav(p, 0.25, 0.5)
    assert len(seg) == sr // 4
    ds = WavDataset([(p, 0.0, 0.5, sr), (p, 0.5, 1.0, sr)], wav_processor=None)
    assert ds[0].shape == (sr // 2, 1) and abs(float(ds[0].mean())) < 1e-3
    feats = WavDataset([(p, 0.0, 1.0, sr)], wav_processor="fbank", num_mel_bin=40)[0]
    assert feats.shape[1] == 40 and 95 <= feats.shape[0] <= 100
    b = collate([ds[0], ds[1][:4000]], [torch.tensor([2, 5, 3]), torch.tensor([2, 6, 7, 3])], src_type="audio")
    assert b.get("source").shape == (sr // 2, 2, 2) and int(b.get("source")[:, 1, 0].sum()) == 4000


def test_kaldi_ark_scp(tmp_path):
    ark, scp = str(tmp_path / "f.ark"), str(tmp_path / "f.scp")
    mats = {"utt1": np.random.randn(7, 40).astype(np.float32), "utt2": np.random.randn(3, 40).astype(np.float32)}
    with open(ark, "wb") as fh, open(scp, "w") as sf:
        for k, m in mats.items():
            off = write_ark_matrix(fh, k, m)
            sf.write("%s %s:%d\n" % (k, ark, off))
    entries = read_scp(scp)
    assert list(entries) == ["utt1", "utt2"]
    for k, (f, off) in entries.items():
        assert np.array_equal(read_ark_matrix(f, off), mats[k])
    ds = SCPDataset(list(entries.values()), concat=4)
    assert ds[0].shape == (2, 160) and ds[1].shape == (1, 160)
    assert torch.equal(stack_frames(torch.arange(6.0).view(3, 2), 2), torch.tensor([[0., 1, 2, 3], [4, 5, 0, 0]]))


def test_whisper_log_mel_and_filterbank_shapes():
    fb = mel_filterbank(80, 400, 16000)
    assert fb.shape == (80, 201) and (fb >= 0).all() and (fb.sum(1) > 0).all()
    wav = torch.randn(16000 * 2) * 0.1
    mel = whisper_log_mel(wav)
    assert mel.shape == (3000, 80) and torch.isfinite(mel).all()
    assert mel.max() - mel.min() <= 2.0 + 1e-4           # clamp to (max - 8) / 4 range
    f = fbank(wav, 40)
    assert f.shape[1] == 40 and 195 <= f.shape[0] <= 200


def test_spec_augment_masks_without_changing_shape():
    x = torch.ones(200, 40)
    y = Augmenter(F=8, mf=2, T=40, mt=2, input_size=40, seed=0).augment(x)
    assert y.shape == x.shape and (y == 0).any() and (y == 1).any()
    assert torch.equal(x, torch.ones(200, 40))


def test_language_model_dataset_blocks():
    ds = LanguageModelDataset(torch.arange(4, 104), batch_size_sents=4, seq_length=8)
    b = ds.get_batch(0)
    assert b.get("target_input").shape == (8, 4) and torch.equal(b.get("target_output")[:-1], b.get("target_input")[1:])
    assert len(ds) == 3
