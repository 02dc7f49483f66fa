"""Audio input: wav segments, Kaldi ark/scp matrices, filterbank and Whisper log-mel features, SpecAugment.

No external audio library is required: PCM wav files are read with the standard ``wave`` module (the reference uses
``soundfile``, onmt/data/audio_utils.py:322-490), Kaldi binary float matrices with a small parser (the reference vendors
a ``kaldiio`` subset, onmt/data/kaldiio/*), and features are computed with torch FFTs (``torchaudio.compliance.kaldi``
is used for filterbanks when it is importable).  ``WavDataset`` / ``SCPDataset`` expose ``[frames, feat]`` tensors that
``data.dataset.collate`` turns into the padded ``[T, B, 1 + feat]`` layout.

Reference: onmt/data/wav_dataset.py:13-158, onmt/data/scp_dataset.py:10, onmt/data/whisper_audio.py:9,
onmt/speech/Augmenter.py:8-66.
"""
from __future__ import annotations

import math
import struct
import wave
from collections import OrderedDict
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch


# ---------------------------------------------------------------------------------------------------
# wav
# ---------------------------------------------------------------------------------------------------
def read_wav(path: str, start: float = 0.0, end: float = 0.0, dtype=np.float32) -> Tuple[np.ndarray, int]:
    """PCM wav -> mono float waveform in [-1, 1] and its sample rate; ``start`` / ``end`` in seconds (0 = whole file)."""
    with wave.open(path, "rb") as w:
        sr, n, width, ch = w.getframerate(), w.getnframes(), w.getsampwidth(), w.getnchannels()
        s = int(round(start * sr))
        e = int(round(end * sr)) if end and end > 0 else n
        s, e = max(0, min(s, n)), max(0, min(e, n))
        w.setpos(s)
        raw = w.readframes(max(e - s, 0))
    if width == 2:
        x = np.frombuffer(raw, dtype="<i2").astype(dtype) / 32768.0
    elif width == 4:
        x = np.frombuffer(raw, dtype="<i4").astype(dtype) / 2147483648.0
    elif width == 1:
        x = (np.frombuffer(raw, dtype=np.uint8).astype(dtype) - 128.0) / 128.0
    else:
        raise ValueError("unsupported sample width %d in %s" % (width, path))
    if ch > 1:
        x = x.reshape(-1, ch).mean(axis=1)
    return x, sr


def write_wav(path: str, samples: np.ndarray, sample_rate: int = 16000) -> None:
    pcm = np.clip(np.asarray(samples) * 32767.0, -32768, 32767).astype("<i2")
    with wave.open(path, "wb") as w:
        w.setnchannels(1)
        w.setsampwidth(2)
        w.setframerate(sample_rate)
        w.writeframes(pcm.tobytes())


# ---------------------------------------------------------------------------------------------------
# Kaldi ark / scp (binary float / double matrices, uncompressed)
# ---------------------------------------------------------------------------------------------------
def write_ark_matrix(fh, key: str, mat: np.ndarray) -> int:
    """Append one matrix; returns the byte offset that an scp entry should point to."""
    fh.write((key + " ").encode())
    offset = fh.tell()
    mat = np.ascontiguousarray(mat, dtype=np.float32)
    fh.write(b"\0BFM ")
    fh.write(b"\4" + struct.pack("<i", mat.shape[0]))
    fh.write(b"\4" + struct.pack("<i", mat.shape[1]))
    fh.write(mat.tobytes())
    return offset


def read_ark_matrix(path: str, offset: int) -> np.ndarray:
    with open(path, "rb") as fh:
        fh.seek(offset)
        if fh.read(2) != b"\0B":
            raise ValueError("%s:%d is not a binary Kaldi object" % (path, offset))
        token = b""
        while True:
            c = fh.read(1)
            if c == b" ":
                break
            token += c
        if token not in (b"FM", b"DM"):
            raise ValueError("unsupported Kaldi matrix type %r (compressed matrices are not handled)" % token)
        assert fh.read(1) == b"\4"
        rows = struct.unpack("<i", fh.read(4))[0]
        assert fh.read(1) == b"\4"
        cols = struct.unpack("<i", fh.read(4))[0]
        dt = np.float32 if token == b"FM" else np.float64
        data = np.frombuffer(fh.read(rows * cols * np.dtype(dt).itemsize), dtype=dt)
    return data.reshape(rows, cols).astype(np.float32)


def read_scp(path: str) -> "OrderedDict[str, Tuple[str, int]]":
    out = OrderedDict()
    with open(path) as fh:
        for line in fh:
            if not line.strip():
                continue
            key, loc = line.strip().split(None, 1)
            f, off = loc.rsplit(":", 1)
            out[key] = (f, int(off))
    return out


class SCPDataset(torch.utils.data.Dataset):
    """Lazy list of Kaldi matrices addressed by ``(ark path, offset)``; optional frame stacking (``concat``)."""

    def __init__(self, entries: Sequence[Tuple[str, int]], concat: int = 1):
        self.entries, self.concat = list(entries), concat

    def __len__(self):
        return len(self.entries)

    def __getitem__(self, i):
        f, off = self.entries[i]
        return stack_frames(torch.from_numpy(read_ark_matrix(f, off)), self.concat)


def stack_frames(feats: torch.Tensor, concat: int) -> torch.Tensor:
    """[T, F] -> [ceil(T / concat), F * concat] (zero padded), the ``-concat`` input reduction."""
    if concat <= 1:
        return feats
    T, F = feats.shape
    pad = (-T) % concat
    if pad:
        feats = torch.cat([feats, feats.new_zeros(pad, F)], 0)
    return feats.reshape(-1, F * concat)


# ---------------------------------------------------------------------------------------------------
# features
# ---------------------------------------------------------------------------------------------------
def mel_filterbank(n_mels: int, n_fft: int, sample_rate: int, f_min: float = 0.0, f_max: Optional[float] = None,
                   htk: bool = False) -> torch.Tensor:
    """Triangular mel filters ``[n_mels, n_fft // 2 + 1]`` (Slaney scale and area normalisation unless ``htk``)."""
    f_max = f_max or sample_rate / 2.0

    def hz_to_mel(f):
        f = np.asarray(f, dtype=np.float64)
        if htk:
            return 2595.0 * np.log10(1.0 + f / 700.0)
        lin = f / (200.0 / 3)
        log_region = f >= 1000.0
        return np.where(log_region, 15.0 + np.log(np.maximum(f, 1e-10) / 1000.0) / (np.log(6.4) / 27.0), lin)

    def mel_to_hz(m):
        m = np.asarray(m, dtype=np.float64)
        if htk:
            return 700.0 * (10.0 ** (m / 2595.0) - 1.0)
        return np.where(m >= 15.0, 1000.0 * np.exp((np.log(6.4) / 27.0) * (m - 15.0)), m * (200.0 / 3))

    mels = np.linspace(hz_to_mel(f_min), hz_to_mel(f_max), n_mels + 2)
    hz = mel_to_hz(mels)
    fft_freqs = np.linspace(0, sample_rate / 2.0, n_fft // 2 + 1)
    fb = np.zeros((n_mels, n_fft // 2 + 1))
    for i in range(n_mels):
        lo, ce, hi = hz[i], hz[i + 1], hz[i + 2]
        up = (fft_freqs - lo) / max(ce - lo, 1e-10)
        down = (hi - fft_freqs) / max(hi - ce, 1e-10)
        fb[i] = np.maximum(0.0, np.minimum(up, down))
        if not htk:
            fb[i] *= 2.0 / max(hi - lo, 1e-10)
    return torch.from_numpy(fb.astype(np.float32))


def whisper_log_mel(wav: torch.Tensor, n_mels: int = 80, sample_rate: int = 16000, n_fft: int = 400, hop: int = 160,
                    pad_to_seconds: float = 30.0) -> torch.Tensor:
    """Whisper front-end: pad / trim to 30 s, STFT (Hann 400 / hop 160), mel power, log10, clamp to max - 8, (x + 4) / 4.
    Returns ``[frames, n_mels]`` (3000 frames for 30 s)."""
    wav = torch.as_tensor(wav, dtype=torch.float32)
    if pad_to_seconds:
        n = int(pad_to_seconds * sample_rate)
        wav = wav[:n] if wav.numel() >= n else torch.cat([wav, wav.new_zeros(n - wav.numel())])
    spec = torch.stft(wav, n_fft, hop, window=torch.hann_window(n_fft), return_complex=True)
    power = spec[..., :-1].abs() ** 2
    mel = mel_filterbank(n_mels, n_fft, sample_rate) @ power
    log = torch.clamp(mel, min=1e-10).log10()
    log = torch.maximum(log, log.max() - 8.0)
    return ((log + 4.0) / 4.0).t().contiguous()


def fbank(wav: torch.Tensor, n_mels: int = 80, sample_rate: int = 16000, frame_length_ms: float = 25.0,
          frame_shift_ms: float = 10.0, dither: float = 0.0) -> torch.Tensor:
    """Kaldi-style log mel filterbank energies ``[frames, n_mels]``."""
    wav = torch.as_tensor(wav, dtype=torch.float32)
    try:
        import torchaudio.compliance.kaldi as kaldi
        return kaldi.fbank(wav.unsqueeze(0) * 32768.0, num_mel_bins=n_mels, sample_frequency=sample_rate,
                           frame_length=frame_length_ms, frame_shift=frame_shift_ms, dither=dither)
    except Exception:  # noqa: BLE001 - torchaudio missing or incompatible: own implementation
        win = int(sample_rate * frame_length_ms / 1000)
        hop = int(sample_rate * frame_shift_ms / 1000)
        n_fft = 1 << (win - 1).bit_length()
        if wav.numel() < win:
            return wav.new_zeros(0, n_mels)
        frames = wav.unfold(0, win, hop) * 32768.0
        frames = frames - frames.mean(-1, keepdim=True)
        frames = torch.cat([frames[:, :1], frames[:, 1:] - 0.97 * frames[:, :-1]], 1) * torch.hamming_window(win, periodic=False)
        power = torch.fft.rfft(frames, n_fft).abs() ** 2
        mel = power @ mel_filterbank(n_mels, n_fft, sample_rate, 20.0, None, htk=True).t()
        return torch.clamp(mel, min=1.1920929e-07).log()


class Augmenter:
    """SpecAugment on a ``[frames, feat]`` matrix: ``F`` / ``T`` = maximum widths of the frequency / time masks,
    ``mf`` / ``mt`` = number of masks (no time warping)."""

    def __init__(self, F: int = 8, mf: int = 2, T: int = 64, max_t: float = 0.2, mt: int = 2, input_size: int = 40, concat: int = 1,
                 seed: Optional[int] = None):
        self.F, self.mf, self.T, self.max_t, self.mt = F, mf, T, max_t, mt
        self.input_size, self.concat = input_size, concat
        self.rng = np.random.RandomState(seed)

    def augment(self, feats: torch.Tensor) -> torch.Tensor:
        x = feats.clone()
        T, D = x.shape
        base = D // max(self.concat, 1)
        for _ in range(self.mf):
            f = int(self.rng.randint(0, self.F + 1))
            f0 = int(self.rng.randint(0, max(base - f, 1)))
            for c in range(max(self.concat, 1)):
                x[:, c * base + f0:c * base + f0 + f] = 0
        max_t = max(1, min(self.T, int(self.max_t * T)))
        for _ in range(self.mt):
            t = int(self.rng.randint(0, max_t + 1))
            t0 = int(self.rng.randint(0, max(T - t, 1)))
            x[t0:t0 + t] = 0
        return x


class WavDataset(torch.utils.data.Dataset):
    """Utterances given as ``(path, start, end, sample_rate)``; returns raw waveforms ``[samples, 1]`` or features.

    ``wav_processor``: ``None`` / ``'raw'`` (waveform, optionally mean/variance normalised), ``'fbank'``, ``'whisper'``.
    A small LRU cache keeps recently read files so segments of the same recording do not re-read it."""

    def __init__(self, entries: Sequence[Tuple[str, float, float, int]], wav_processor: Optional[str] = None, num_mel_bin: int = 80,
                 normalize: bool = True, cache_size: int = 64, augmenter: Optional[Augmenter] = None):
        self.entries = list(entries)
        self.proc = wav_processor or "raw"
        self.n_mels, self.normalize = num_mel_bin, normalize
        self.cache: "OrderedDict[str, Tuple[np.ndarray, int]]" = OrderedDict()
        self.cache_size = cache_size
        self.augmenter = augmenter

    def __len__(self):
        return len(self.entries)

    def _load(self, path):
        if path in self.cache:
            self.cache.move_to_end(path)
            return self.cache[path]
        data = read_wav(path)
        self.cache[path] = data
        if len(self.cache) > self.cache_size:
            self.cache.popitem(last=False)
        return data

    def __getitem__(self, i):
        path, start, end, sr = self.entries[i][:4]
        wav, file_sr = self._load(path)
        s = int(round(start * file_sr))
        e = int(round(end * file_sr)) if end and end > 0 else len(wav)
        x = torch.from_numpy(np.ascontiguousarray(wav[s:e]))
        if self.proc == "raw":
            if self.normalize and x.numel() > 1:
                x = (x - x.mean()) / (x.std() + 1e-7)
            return x.unsqueeze(-1)
        feats = whisper_log_mel(x, self.n_mels, file_sr) if self.proc == "whisper" else fbank(x, self.n_mels, file_sr)
        return self.augmenter.augment(feats) if self.augmenter is not None else feats


class LanguageModelDataset(torch.utils.data.Dataset):
    """One long token stream cut into ``[batch, seq_len]`` blocks (inputs and next-token targets), for ``train_language_model``.
    Reference: onmt/data/lm_dataset.py:53."""

    def __init__(self, tokens: torch.Tensor, batch_size_sents: int, seq_length: int):
        n = tokens.numel() // batch_size_sents
        self.data = tokens[:n * batch_size_sents].view(batch_size_sents, n)
        self.seq_length = seq_length
        self.num_batches = max((n - 1 + seq_length - 1) // seq_length, 0)

    def __len__(self):
        return self.num_batches

    def get_batch(self, i):
        from .dataset import collate
        s = i * self.seq_length
        e = min(s + self.seq_length + 1, self.data.shape[1])
        rows = [self.data[b, s:e] for b in range(self.data.shape[0])]
        return collate(None, rows, round_to=1)

    __getitem__ = get_batch
