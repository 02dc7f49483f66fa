#!/usr/bin/env python
"""Training entry point: one process per GPU.

    python train_distributed.py -data <prefix> -data_format raw|bin|mmap|wav|scp -save_model <path> -gpus 0 1 2 3 ...

Loads the preprocessed corpus, builds token-budget ``Dataset`` objects, then either runs the trainer in this
process (one GPU / CPU) or spawns one process per listed GPU (``torch.multiprocessing.spawn``), each of which
joins a NCCL process group over 127.0.0.1.  When launched under ``torchrun`` (RANK / WORLD_SIZE in the
environment) no processes are spawned and the environment's rank is used.
Reference flow: train_distributed.py:118-727.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import numpy as np
import torch

from nmtgminor_b200.constants import Constants
from nmtgminor_b200.data.dataset import Dataset
from nmtgminor_b200.data.mmap_dataset import MMapIndexedDataset
from nmtgminor_b200.options import make_parser


def _dataset_from(split, opt, dicts, training):
    if split is None or (split.get("src") is None and split.get("tgt") is None):
        return None
    if getattr(opt, "model", "") in ("transformer_xl_lm", "TransformerXL") and split.get("src") is None and split.get("tgt") is not None:
        # language-model training: the target side is one long token stream cut into [-batch_size_sents, -lm_seq_length] blocks
        from nmtgminor_b200.data.audio import LanguageModelDataset
        stream = torch.cat([torch.as_tensor(t).view(-1) for t in split["tgt"]])
        return LanguageModelDataset(stream, opt.batch_size_sents if opt.batch_size_sents > 0 else 32, int(getattr(opt, "lm_seq_length", 128)))
    audio = getattr(opt, "encoder_type", "text") != "text"
    augmenter = None
    if training and audio and getattr(opt, "augment_speech", False):
        # -augment_speech: SpecAugment on the feature matrices, widths from -sa_f / -sa_t (reference:
        # train_distributed.py:186-200 -> onmt/speech/Augmenter.py)
        from nmtgminor_b200.data.audio import Augmenter
        augmenter = Augmenter(F=int(getattr(opt, "sa_f", 8)), T=int(getattr(opt, "sa_t", 64)),
                              input_size=int(getattr(opt, "input_size", 40) or 40), concat=int(getattr(opt, "concat", 1) or 1),
                              seed=int(getattr(opt, "seed", 9999)))
    # captured CUDA graphs need batches whose shapes repeat: round packed capacities to a few sizes (text batches)
    static = training and not audio and _use_cuda_graph(opt)
    return Dataset(split.get("src"), split.get("tgt"), split.get("src_sizes"), split.get("tgt_sizes"), split.get("src_lang"),
                   split.get("tgt_lang"), split.get("src_atb"), split.get("tgt_atb"),
                   batch_size_words=opt.batch_size_words, batch_size_frames=getattr(opt, "batch_size_frames", 10 ** 12),
                   batch_size_sents=opt.batch_size_sents if opt.batch_size_sents > 0 else 10 ** 9,
                   multiplier=opt.batch_size_multiplier, data_type=getattr(opt, "encoder_type", "text") if getattr(opt, "encoder_type", "text") != "text" else "text",
                   max_src_len=opt.max_src_length if training else 10 ** 9, max_tgt_len=(opt.max_tgt_length + 2) if training else 10 ** 9,
                   cleaning=training, verbose=True, aux_tgt_data=split.get("aux_tgt"), augmenter=augmenter, static_shapes=static,
                   concat=training and bool(getattr(opt, "concat_dataset", False)), concat_seed=int(getattr(opt, "seed", 1234) or 1234))


def _use_cuda_graph(opt) -> bool:
    """The training step is replayed from CUDA graphs by default on a GPU; ``-no_cuda_graph``, gradient accumulation
    (``-update_frequency`` > 1, ``-batch_size_update``) and random layer skipping switch it off."""
    from nmtgminor_b200.parallel.sharded import skips_layers
    gpu = bool(getattr(opt, "gpus", None)) and opt.gpus not in ([], [-1]) and torch.cuda.is_available()
    return (gpu and not getattr(opt, "no_cuda_graph", False) and int(getattr(opt, "update_frequency", 1) or 1) <= 1
            and int(getattr(opt, "batch_size_update", -1) or -1) <= 0 and not skips_layers(opt))


def load_multi_datasets(opt):
    """``-multi_dataset``: one data set per directory ``train.<i>.<langs>/data.*`` / ``valid.<i>.<langs>/data.*`` next to
    ``<data>.dict.pt`` (reference: train_distributed.py:487-545); returns lists that the trainer iterates jointly."""
    from nmtgminor_b200.data.audio import SCPDataset, WavDataset
    dicts = torch.load(opt.data + ".dict.pt", map_location="cpu", weights_only=False)
    root = os.path.dirname(os.path.abspath(opt.data))
    fmt = opt.data_format
    found = {"train": {}, "valid": {}}
    for d in os.listdir(root):
        parts = d.split(".")
        if os.path.isdir(os.path.join(root, d)) and parts[0] in found and len(parts) > 1 and parts[1].isdigit():
            found[parts[0]][int(parts[1])] = os.path.join(root, d)
    if fmt in ("wav", "scp", "scpmem") and getattr(opt, "encoder_type", "text") == "text":
        opt.encoder_type = "audio"

    def one(d, training):
        mm = lambda name: MMapIndexedDataset(os.path.join(d, name)) if MMapIndexedDataset.exists(os.path.join(d, name)) else None
        if fmt in ("wav", "scp", "scpmem"):
            entries = torch.load(os.path.join(d, "data.scp_path.pt"), map_location="cpu", weights_only=False)
            proc = getattr(opt, "wav_processor", None)
            src = (WavDataset(entries, proc if proc in ("fbank", "whisper") else None, getattr(opt, "num_mel_bin", 0) or 80)
                   if fmt == "wav" else SCPDataset(entries, getattr(opt, "concat", 1) or 1))
        else:
            src = mm("data.src")
        sizes = lambda name: np.load(os.path.join(d, name)) if os.path.exists(os.path.join(d, name)) else None
        split = {"src": src, "tgt": mm("data.tgt"), "src_lang": mm("data.src_lang"), "tgt_lang": mm("data.tgt_lang"),
                 "src_atb": mm("data.src_atb"), "tgt_atb": mm("data.tgt_atb"),
                 "src_sizes": sizes("data.src_sizes.npy"), "tgt_sizes": sizes("data.tgt_sizes.npy")}
        return _dataset_from(split, opt, dicts, training)
    # -train_sets / -valid_sets pick data sets by their directory index (all of them when empty); -train_set_orders
    # gives the order in which the chosen training sets are visited; -dataset_index starts a continual-learning run at
    # that position of the list (reference: train_distributed.py:470-545)
    want_train = list(getattr(opt, "train_sets", []) or []) or sorted(found["train"])
    want_valid = list(getattr(opt, "valid_sets", []) or []) or sorted(found["valid"])
    orders = list(getattr(opt, "train_set_orders", []) or [])
    if orders:
        assert len(orders) == len(want_train), "-train_set_orders needs one position per training set"
        want_train = [i for _, i in sorted(zip(orders, want_train))]
    start = int(getattr(opt, "dataset_index", 0) or 0)
    if start > 0:
        want_train = want_train[start:]
    missing = [i for i in want_train if i not in found["train"]] + [i for i in want_valid if i not in found["valid"]]
    if missing:
        raise FileNotFoundError("data set directories with index %s not found under %s" % (missing, root))
    train = [one(found["train"][i], True) for i in want_train]
    valid = [one(found["valid"][i], False) for i in want_valid]
    return dicts, train, (valid or None)


def load_data(opt):
    fmt = opt.data_format
    if getattr(opt, "multi_dataset", False):
        return load_multi_datasets(opt)
    if fmt in ("raw", "bin"):
        blob = torch.load(opt.data + ".train.pt", map_location="cpu", weights_only=False)
        dicts = blob["dicts"]
        train, valid = blob["train"], blob.get("valid")
    elif fmt in ("mmap", "mmem"):
        dicts = torch.load(opt.data + ".dict.pt", map_location="cpu", weights_only=False)

        def side(split):
            out = {}
            for s in ("src", "tgt", "src_lang", "tgt_lang"):
                prefix = "%s.%s.%s" % (opt.data, split, s)
                out[s] = MMapIndexedDataset(prefix) if MMapIndexedDataset.exists(prefix) else None
            for s in ("src", "tgt"):
                f = "%s.%s.%s_sizes.npy" % (opt.data, split, s)
                out[s + "_sizes"] = np.load(f) if os.path.exists(f) else None
            return out
        train, valid = side("train"), side("valid")
    elif fmt in ("wav", "scp", "scpmem"):
        from nmtgminor_b200.data.audio import SCPDataset, WavDataset
        dicts = torch.load(opt.data + ".dict.pt", map_location="cpu", weights_only=False)
        index = torch.load(opt.data + (".wav_path.pt" if fmt == "wav" else ".scp_path.pt"), map_location="cpu", weights_only=False)
        if getattr(opt, "encoder_type", "text") == "text":
            opt.encoder_type = "audio"

        def side(split):
            entries = index.get(split)
            if not entries:
                return None
            if fmt == "wav":
                replace = getattr(opt, "wav_path_replace", None)
                if replace and len(replace) == 2:
                    entries = [(e[0].replace(replace[0], replace[1]),) + tuple(e[1:]) for e in entries]
                proc = getattr(opt, "wav_processor", None)
                src = WavDataset(entries, proc if proc in ("fbank", "whisper") else None, getattr(opt, "num_mel_bin", 0) or 80,
                                 cache_size=getattr(opt, "data_cache_size", 64) or 64)
            else:
                src = SCPDataset(entries, getattr(opt, "concat", 1) or 1)
            out = {"src": src}
            for s in ("tgt", "src_lang", "tgt_lang"):
                prefix = "%s.%s.%s" % (opt.data, split, s)
                out[s] = MMapIndexedDataset(prefix) if MMapIndexedDataset.exists(prefix) else None
            for s in ("src", "tgt"):
                f = "%s.%s.%s_sizes.npy" % (opt.data, split, s)
                out[s + "_sizes"] = np.load(f) if os.path.exists(f) else None
            return out
        train, valid = side("train"), side("valid")
    else:
        raise NotImplementedError("data format %r" % fmt)
    return dicts, _dataset_from(train, opt, dicts, True), _dataset_from(valid, opt, dicts, False)


def run_process(rank, opt):
    from nmtgminor_b200.train.research import select_trainer
    if len(opt.gpus) > 1 and "RANK" not in os.environ:
        os.environ["RANK"] = str(rank)
        os.environ["LOCAL_RANK"] = str(opt.gpus[rank])
        os.environ["WORLD_SIZE"] = str(len(opt.gpus))
    os.environ.setdefault("MASTER_ADDR", opt.master_addr or "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", str(opt.master_port or 8888))
    dicts, train_data, valid_data = load_data(opt)
    if getattr(opt, "override_dict_from_checkpoint", False) and getattr(opt, "load_from", ""):
        # continue with the vocabularies the checkpoint was trained with, whatever the data files say
        ckpt_dicts = torch.load(opt.load_from, map_location="cpu", weights_only=False).get("dicts")
        if ckpt_dicts:
            dicts.update({k: v for k, v in ckpt_dicts.items() if k in ("src", "tgt", "langs", "atbs")})
    if getattr(opt, "patch_vocab_multiplier", 1) > 1 and "tgt" in dicts:
        dicts["tgt"].patch(opt.patch_vocab_multiplier)
    constants = Constants.from_dicts(opt, dicts)
    trainer = select_trainer(opt)(opt.gpus[rank] if opt.gpus else -1, dicts, opt, constants)
    trainer.run(train_data=train_data, valid_data=valid_data)


def cli_main(argv=None):
    opt = make_parser().parse_args(argv)
    if "WORLD_SIZE" in os.environ and int(os.environ["WORLD_SIZE"]) > 1:
        opt.gpus = list(range(int(os.environ["WORLD_SIZE"])))
        run_process(int(os.environ["RANK"]), opt)
    elif len(opt.gpus) <= 1:
        run_process(0, opt)
    else:
        torch.multiprocessing.spawn(run_process, nprocs=len(opt.gpus), args=(opt,))


if __name__ == "__main__":
    cli_main()
