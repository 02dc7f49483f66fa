"""Audio corpora end to end on the CPU: utterance lists -> preprocess (-asr) -> training data sets -> a model step."""
import importlib.util
import os

import numpy as np
import torch

from nmtgminor_b200.data.audio import write_ark_matrix, write_wav
from nmtgminor_b200.data.binarizer import binarize_speech_file

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _wav_corpus(tmp_path, n=6):
    rng = np.random.default_rng(0)
    lines, text = [], []
    for i in range(n):
        path = str(tmp_path / ("utt%d.wav" % i))
        write_wav(path, (rng.standard_normal(4000 + 500 * i) * 0.1).astype(np.float32), 16000)
        lines.append("utt%d %s" % (i, path) if i % 2 else "utt%d %s 0.0 0.2" % (i, path))     # every other one is a segment
        text.append(" ".join("w%d" % ((i + j) % 7) for j in range(3 + i % 3)))
    src, tgt = tmp_path / "train.wavlist", tmp_path / "train.txt"
    src.write_text("\n".join(lines) + "\n")
    tgt.write_text("\n".join(text) + "\n")
    return str(src), str(tgt)


def test_wav_lists_are_indexed_not_copied(tmp_path):
    src, _ = _wav_corpus(tmp_path)
    out = binarize_speech_file(src, "wav")
    assert len(out["data"]) == 6 and out["data"][1][1:] == (0.0, 0.0, 16000)
    assert out["sizes"][0] == 3200 and out["sizes"][1] == 4500          # 0.2 s segment; whole file
    frames = binarize_speech_file(src, "wav", num_mel_bin=80)["sizes"]
    assert frames[0] == 20 and frames[1] == 28


def test_kaldi_scp_lists(tmp_path):
    ark = str(tmp_path / "feats.ark")
    lines = []
    with open(ark, "wb") as fh:
        for i in range(3):
            off = write_ark_matrix(fh, "utt%d" % i, np.random.rand(10 + i, 8).astype(np.float32))
            lines.append("utt%d %s:%d" % (i, ark, off))
    scp = tmp_path / "feats.scp"
    scp.write_text("\n".join(lines) + "\n")
    out = binarize_speech_file(str(scp), "scp", concat=4)
    assert out["sizes"] == [3, 3, 3] and out["data"][2][0] == ark


def test_preprocess_asr_then_train_step(tmp_path):
    src, tgt = _wav_corpus(tmp_path)
    pre = _load("preprocess")
    save = str(tmp_path / "data" / "asr")
    pre.main(["-asr", "-asr_format", "wav", "-format", "wav", "-train_src", src, "-train_tgt", tgt, "-valid_src", src, "-valid_tgt", tgt,
              "-save_data", save, "-tgt_seq_length", "64"])
    for suffix in (".dict.pt", ".wav_path.pt", ".train.tgt.bin", ".train.tgt.idx", ".train.src_sizes.npy", ".valid.tgt_sizes.npy"):
        assert os.path.exists(save + suffix), suffix
    index = torch.load(save + ".wav_path.pt", weights_only=False)
    assert len(index["train"]) == 6 and index["train"][0][0].endswith("utt0.wav")

    td = _load("train_distributed")
    from nmtgminor_b200.models.factory import build_model
    from nmtgminor_b200.options import make_parser
    enc = tmp_path / "enc.json"
    enc.write_text('{"encoder_embed_dim": 32, "encoder_layers": 1, "encoder_attention_heads": 2, "encoder_ffn_embed_dim": 64}')
    opt = make_parser().parse_args(["-data", save, "-data_format", "wav", "-model", "wav2vec2_transformer", "-enc_config_file", str(enc),
                                    "-model_size", "32", "-layers", "1", "-n_heads", "2", "-inner_size", "64", "-batch_size_words", "64",
                                    "-batch_size_frames", "20000", "-save_model", str(tmp_path / "m")])
    dicts, train, valid = td.load_data(opt)
    assert opt.encoder_type == "audio" and len(train) >= 1 and valid is not None
    batch = train.get_batch(0)
    source = batch.get("source")
    assert source.dim() == 3 and source.shape[-1] == 2            # [frames, batch, marker + waveform]
    model = build_model(opt, dicts)
    out = model(batch)
    assert torch.isfinite(out["loss"]).all()
    out["loss"].backward()


def test_multi_dataset_directories(tmp_path):
    """``-multi_dataset``: one directory per corpus, language ids from the table in the dictionary file."""
    def corpus(name, n, off):
        s, t = tmp_path / (name + ".src"), tmp_path / (name + ".tgt")
        s.write_text("\n".join(" ".join("a%d" % ((i + j + off) % 9) for j in range(4 + i % 3)) for i in range(n)) + "\n")
        t.write_text("\n".join(" ".join("b%d" % ((i + j + off) % 9) for j in range(3 + i % 4)) for i in range(n)) + "\n")
        return str(s), str(t)
    s0, t0 = corpus("ende", 12, 0)
    s1, t1 = corpus("enfr", 8, 3)
    pre = _load("preprocess")
    save = str(tmp_path / "multi" / "corpus")
    pre.main(["-multi_dataset", "-format", "mmap", "-train_src", s0 + "|" + s1, "-train_tgt", t0 + "|" + t1, "-valid_src", s0, "-valid_tgt", t0,
              "-train_src_lang", "en|en", "-train_tgt_lang", "de|fr", "-valid_src_lang", "en", "-valid_tgt_lang", "de", "-save_data", save])
    root = os.path.dirname(save)
    assert sorted(d for d in os.listdir(root) if os.path.isdir(os.path.join(root, d))) == ["train.0.en-de", "train.1.en-fr", "valid.0.en-de"]
    td = _load("train_distributed")
    from nmtgminor_b200.options import make_parser
    opt = make_parser().parse_args(["-data", save, "-data_format", "mmap", "-multi_dataset", "-batch_size_words", "64", "-save_model", str(tmp_path / "m")])
    dicts, train, valid = td.load_data(opt)
    assert dicts["langs"] == {"en": 0, "de": 1, "fr": 2}
    assert len(train) == 2 and len(valid) == 1
    b = train[1].get_batch(0)
    assert int(b.get("target_lang")[0]) == 2 and int(b.get("source_lang")[0]) == 0


def test_external_tokenizer_from_a_local_directory(tmp_path):
    """``-external_tokenizer <dir>``: ids come from a Hugging Face tokenizer stored locally."""
    tokenizers = __import__("pytest").importorskip("tokenizers")
    from transformers import PreTrainedTokenizerFast
    from nmtgminor_b200.data.binarizer import binarize_file, load_external_tokenizer
    vocab = {"<pad>": 0, "<unk>": 1, "<s>": 2, "</s>": 3, "hello": 4, "world": 5}
    tk = tokenizers.Tokenizer(tokenizers.models.WordLevel(vocab, unk_token="<unk>"))
    tk.pre_tokenizer = tokenizers.pre_tokenizers.Whitespace()
    PreTrainedTokenizerFast(tokenizer_object=tk, unk_token="<unk>", pad_token="<pad>").save_pretrained(str(tmp_path / "tok"))
    ext = load_external_tokenizer(str(tmp_path / "tok"))
    assert ext("hello world foo") == [4, 5, 1]
    f = tmp_path / "t.txt"
    f.write_text("hello world\nworld\n")
    out = binarize_file(str(f), None, None, None, None, 1, external=ext)
    assert [t.tolist() for t in out["data"]] == [[4, 5], [5]] and out["sizes"] == [2, 1]
