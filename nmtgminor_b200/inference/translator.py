"""Translator: load one or several checkpoints, batch raw sentences, run beam search, return strings.

``Translator(opt)`` mirrors what the reference's ``FastTranslator`` offers to ``translate.py`` and the
serving shims (onmt/inference/fast_translator.py:16-338 set-up, :1123-1230 ``build_data``, :1244-1366
``translate``; base class onmt/inference/translator.py:14-186):

* ``-model a|b|c`` loads an ensemble; log-probabilities are combined per step (``-ensemble_op mean`` =
  arithmetic mean of probabilities, ``logSum`` = mean of log-probabilities, optional ``-ensemble_weight``);
* ``translate(src_sents, tgt_sents=None)`` returns ``(pred_batch, pred_ids, pred_score, pred_pos_scores,
  pred_length, gold_score, gold_words, allgold)`` with ``n_best`` hypotheses per sentence;
* inputs are token lists (already BPE-split); words are mapped with the checkpoint's dictionaries.

Weights are kept in bf16 on the GPU (flat store) and decoding runs through the same fused ops as training.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch

from .. import constants as C
from ..data.dataset import collate
from ..models.factory import build_model
from ..options import backward_compatible
from ..parallel.flat import FlatParameterStore
from ..train.checkpoint import load_checkpoint, load_model_state
from .beam_search import BeamConfig, Hypothesis, beam_search


class EnsembleModel(torch.nn.Module):
    """Presents several models as one for beam search by combining their next-token distributions."""

    def __init__(self, models, op: str = "mean", weights: Optional[Sequence[float]] = None, sub_flags: Optional[Sequence[bool]] = None):
        super().__init__()
        self.models = torch.nn.ModuleList(models)
        # members flagged here read the batch's ``sub_batch`` (``-sub_model`` / ``-sub_src``: e.g. a text model fed the
        # transcript next to a speech model fed the audio) instead of the main batch
        self.sub_flags = list(sub_flags) if sub_flags else [False] * len(models)
        self.op = op
        w = list(weights) if weights else [1.0] * len(models)
        s = sum(w)
        self.weights = [x / s for x in w]

    def create_decoder_state(self, batch, beam_size, **kw):
        pick = lambda sub: batch.sub_batch if (sub and getattr(batch, "sub_batch", None) is not None) else batch
        return _EnsembleState([m.create_decoder_state(pick(sub), beam_size, **kw) for m, sub in zip(self.models, self.sub_flags)])

    def step(self, input_t, state):
        outs = [m.step(input_t, s)["log_prob"] for m, s in zip(self.models, state.states)]
        if len(outs) == 1:
            lp = outs[0]
        elif self.op == "logSum":
            lp = sum(w * o for w, o in zip(self.weights, outs))
            lp = lp - torch.logsumexp(lp, dim=-1, keepdim=True)
        else:   # mean of probabilities
            lp = torch.logsumexp(torch.stack([o + math.log(w) for w, o in zip(self.weights, outs)], 0), dim=0)
        return {"log_prob": lp, "coverage": None}

    def decode(self, batch):
        return self.models[0].decode(batch)

    def renew_buffer(self, n):
        for m in self.models:
            m.renew_buffer(n)


class _EnsembleState:
    def __init__(self, states):
        self.states = states

    @property
    def context(self):
        return self.states[0].context

    @property
    def src_pad_mask(self):
        return self.states[0].src_pad_mask

    def reorder(self, index):
        for s in self.states:
            s.reorder(index)


class Translator:
    def __init__(self, opt):
        self.opt = opt
        self.cuda = getattr(opt, "gpu", -1) is not None and getattr(opt, "gpu", -1) >= 0 and torch.cuda.is_available()
        self.device = torch.device("cuda", opt.gpu) if self.cuda else torch.device("cpu")
        if self.cuda:
            torch.cuda.set_device(self.device)
        self.beam_size = getattr(opt, "beam_size", 4)
        self.n_best = getattr(opt, "n_best", 1)
        models = []
        self.src_dict = self.tgt_dict = None
        self.model_opts = []
        main_paths = str(opt.model).split("|")
        sub_paths = [p for p in str(getattr(opt, "sub_model", "") or "").split("|") if p]
        self.sub_src_dict = None
        for path in main_paths + sub_paths:
            ckpt = load_checkpoint(path)
            mopt = backward_compatible(ckpt["opt"])
            dicts = ckpt["dicts"]
            if self.src_dict is None and self.tgt_dict is None:
                self.src_dict = dicts.get("src")
                self.tgt_dict = dicts["tgt"]
                self.dicts = dicts
            if len(models) >= len(main_paths) and self.sub_src_dict is None:
                self.sub_src_dict = dicts.get("src")            # source vocabulary of the first sub-model
            model = build_model(mopt, dicts, remove_pretrain=True)
            load_model_state(model, ckpt["model"])
            if hasattr(model, "renew_buffer"):             # classifiers have no decoder position buffers
                model.renew_buffer(getattr(opt, "max_sent_length", 256) + 2)
            model.eval()
            if self.cuda:
                FlatParameterStore(model, self.device)        # bf16 working copies for the fused kernels
                for b in model.buffers():
                    b.data = b.data.to(self.device)
            for p in model.parameters():
                p.requires_grad_(False)
            if not self.cuda and int(getattr(opt, "dynamic_quantile", 0) or 0) == 1:
                from ..models.layers import quantize_linears_for_cpu
                quantize_linears_for_cpu(model)
            models.append(model)
            self.model_opts.append(mopt)
        weights = None
        if getattr(opt, "ensemble_weight", ""):
            weights = [float(x) for x in str(opt.ensemble_weight).split("|")]
        self.model = models[0] if len(models) == 1 else EnsembleModel(
            models, getattr(opt, "ensemble_op", "mean"), weights, [False] * len(main_paths) + [True] * len(sub_paths))
        self.bos = self.tgt_dict.lookup(getattr(opt, "bos_token", C.BOS_WORD), C.BOS) if hasattr(self.tgt_dict, "lookup") else C.BOS
        self.eos = self.tgt_dict.lookup(C.EOS_WORD, C.EOS) if hasattr(self.tgt_dict, "lookup") else C.EOS
        self.pad = C.PAD
        self.cfg = BeamConfig(beam_size=self.beam_size, n_best=self.n_best, max_len=getattr(opt, "max_sent_length", 256),
                              min_len=getattr(opt, "min_sent_length", 1), dynamic_max_len=getattr(opt, "dynamic_max_len", False),
                              len_a=getattr(opt, "dynamic_max_len_scale", 1.5), len_b=10.0, alpha=getattr(opt, "alpha", 0.0),
                              normalize=getattr(opt, "normalize", False),
                              no_repeat_ngram_size=getattr(opt, "no_repeat_ngram_size", 0), bos=self.bos, eos=self.eos,
                              pad=self.pad, sampling=getattr(opt, "sampling", False))

    # ------------------------------------------------------------------------------------------
    def _lang_ids(self, n: int):
        """Language-id tensors for multilingual models from ``-src_lang`` / ``-tgt_lang`` and the checkpoint's table."""
        langs = self.dicts.get("langs") if isinstance(self.dicts, dict) else None
        if not langs:
            return None, None
        pick = lambda name: torch.full((n,), int(langs.get(name, 0)), dtype=torch.long)
        return pick(getattr(self.opt, "src_lang", "src")), pick(getattr(self.opt, "tgt_lang", "tgt"))

    def build_data(self, src_sents, tgt_sents: Optional[List[List[str]]] = None, past_sents: Optional[List[List[str]]] = None):
        """``src_sents``: token lists (text models) or ``[frames, features]`` tensors (audio models: ``-encoder_type
        audio`` / ``-asr_format``; a leading channel of ones marks real frames, as in training batches)."""
        audio = len(src_sents) > 0 and torch.is_tensor(src_sents[0])
        if audio:
            src = [f.float().view(f.shape[0], -1) for f in src_sents]     # collate adds the real-frame marker channel
        else:
            src = [self.src_dict.convert_to_idx(s, C.UNK_WORD) for s in src_sents]
        tgt = None
        if tgt_sents:
            tgt = [self.tgt_dict.convert_to_idx(t, C.UNK_WORD, C.BOS_WORD, C.EOS_WORD) for t in tgt_sents]
        sl, tl = self._lang_ids(len(src))
        past = None
        if past_sents and not audio:
            # an empty previous sentence (document start) is represented by a single padding symbol
            past = [self.src_dict.convert_to_idx(p, C.UNK_WORD) if p else torch.tensor([C.PAD]) for p in past_sents]
        return collate(src, tgt, src_lang=sl, tgt_lang=tl, src_type="audio" if audio else "text", padded=True, packed=True, round_to=1,
                       past_src_data=past)

    def translate_batch(self, batch, prefix_tokens=None, banned_first=None) -> List[List[Hypothesis]]:
        if self.cuda:
            batch = batch.cuda(self.device)
            if getattr(batch, "sub_batch", None) is not None:
                batch.sub_batch = batch.sub_batch.cuda(self.device)
        if getattr(self.model, "ctc_only", False):
            # encoder-only CTC models (-no_decoder): best-path decoding, one hypothesis per utterance
            return [[Hypothesis(tokens, score, [])] for tokens, score in self.model.ctc_greedy(batch)]
        return beam_search(self.model, batch, self.cfg, prefix_tokens, banned_first)

    def translate(self, src_sents, tgt_sents: Optional[List[List[str]]] = None, prefix: Optional[List[List[str]]] = None,
                  anti_prefix: Optional[List[str]] = None, past_sents: Optional[List[List[str]]] = None,
                  sub_src_sents: Optional[List[List[str]]] = None):
        """``prefix``: tokens every hypothesis of sentence i must start with (``-prefix_string`` gives one prefix for
        all sentences); ``anti_prefix``: tokens that may not open a hypothesis (``-anti_prefix_string``)."""
        batch = self.build_data(src_sents, tgt_sents, past_sents)
        if sub_src_sents and self.sub_src_dict is not None:
            # ``-sub_src``: the sub-models' own source side (same sentences, same order)
            sub = [self.sub_src_dict.convert_to_idx(s, C.UNK_WORD) for s in sub_src_sents]
            batch.sub_batch = collate(sub, None, src_type="text", padded=True, packed=True, round_to=1)
        if prefix is None and getattr(self.opt, "prefix_string", None):
            prefix = [str(self.opt.prefix_string).split()] * len(src_sents)
        if anti_prefix is None and getattr(self.opt, "anti_prefix_string", None):
            anti_prefix = str(self.opt.anti_prefix_string).split()
        banned_first = None
        if anti_prefix:
            banned_first = self.tgt_dict.convert_to_idx(anti_prefix, C.UNK_WORD).to(self.device)
        prefix_tokens = None
        if prefix:
            rows = [self.tgt_dict.convert_to_idx(p, C.UNK_WORD) for p in prefix]
            L = max(len(r) for r in rows)
            prefix_tokens = torch.full((len(rows), L), self.pad, dtype=torch.long)
            for i, r in enumerate(rows):
                prefix_tokens[i, :len(r)] = r
            prefix_tokens = prefix_tokens.to(self.device)
        gold_score, gold_words, allgold = [0.0] * len(src_sents), 0, []
        if tgt_sents:
            gb = batch.cuda(self.device) if self.cuda else batch
            _, sums, per_tok = self.model.decode(gb)
            gold_score = sums.float().cpu().tolist()
            gold_words = batch.tgt_size
            allgold = per_tok.float().cpu().t().tolist()
        hyps = self.translate_batch(batch, prefix_tokens, banned_first)
        pred_batch, pred_ids, pred_score, pred_pos, pred_len = [], [], [], [], []
        for h in hyps:
            ids = [x.tokens for x in h]
            pred_ids.append(ids)
            pred_batch.append([self.tgt_dict.convert_to_labels(t, self.eos, including_stop=False) for t in ids])
            pred_score.append([x.score for x in h])
            pred_pos.append([x.positional_scores for x in h])
            pred_len.append([len(t) for t in ids])
        return pred_batch, pred_ids, pred_score, pred_pos, pred_len, gold_score, gold_words, allgold


FastTranslator = Translator
