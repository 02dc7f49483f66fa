#!/usr/bin/env python
"""Frame features of a speech encoder checkpoint for unit discovery (k-means, quantisation):

    reader = FeatureReader("wav2vec2.pt", layer=12, use_cuda=False)
    feats = reader.get_feats("utt.wav")            # [frames, dim]

    python neural_feature_reader.py <checkpoint> <wav list: '<id> <path>' per line> <out.pt> [layer]

(reference: neural_feature_reader.py: FeatureReader.read_audio / get_feats)"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from nmtgminor_b200.tools.extract import encoder_frames, load_speech_encoder, read_wav_list


class FeatureReader:
    def __init__(self, checkpoint_path, layer=None, max_chunk=1600000, use_cuda=True, fp16=False, bf16=False, **_unused):
        self.device = "cuda" if (use_cuda and torch.cuda.is_available()) else "cpu"
        self.encoder, self.quantizer = load_speech_encoder(checkpoint_path, self.device)
        self.layer = layer
        self.max_chunk = max_chunk

    def read_audio(self, path, ref_len=None, channel_id=None):
        from nmtgminor_b200.data.audio import read_wav
        wav, _rate = read_wav(path)
        wav = torch.as_tensor(wav, dtype=torch.float32)
        if wav.dim() == 2:
            wav = wav[:, channel_id or 0] if wav.shape[1] < wav.shape[0] else wav[channel_id or 0]
        return wav.reshape(-1)

    @torch.no_grad()
    def get_feats(self, file_path, ref_len=None, channel_id=None):
        wav = self.read_audio(file_path, ref_len, channel_id)
        chunks = [wav[i:i + self.max_chunk] for i in range(0, wav.numel(), self.max_chunk)]
        feats = encoder_frames(self.encoder, chunks, self.layer, self.device)
        return torch.cat([f.float().cpu() for f in feats], 0)


if __name__ == "__main__":
    if len(sys.argv) < 4:
        sys.exit(__doc__)
    layer = int(sys.argv[4]) if len(sys.argv) > 4 else None
    enc, _ = load_speech_encoder(sys.argv[1], "cuda" if torch.cuda.is_available() else "cpu")
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    out = [encoder_frames(enc, [wav], layer, dev)[0].float().cpu() for _uid, wav in read_wav_list(sys.argv[2])]
    torch.save(out, sys.argv[3])
    print("wrote %d feature matrices to %s" % (len(out), sys.argv[3]))
