#!/usr/bin/env python
"""Translate a text file with beam search.

    python translate.py -model ckpt.pt[|ckpt2.pt] -src input.txt -output pred.txt -beam_size 4 -batch_size 64 -gpu 0

Sentences are read in blocks of ``-batch_size``, translated by ``Translator`` and written one per line
(``-n_best > 1`` with ``-print_nbest``: ``"<hyp> ||| <score>"`` per hypothesis).  ``-tgt`` enables gold scoring;
``-verbose`` prints source / prediction / scores.  Option names follow the reference (translate.py:20-168;
main loop :238-856; output conventions :745-852).
"""
import math
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch

from nmtgminor_b200.inference.translator import Translator
from nmtgminor_b200.options import make_translate_parser


def report_score(name, score_total, words_total):
    if words_total <= 0:
        return
    print("%s AVG SCORE: %.4f, %s PPL: %.4f" % (name, score_total / words_total, name,
                                                math.exp(-score_total / words_total)), file=sys.stderr)


def get_sentence_from_tokens(tokens, input_type="word"):
    return "".join(tokens) if input_type == "char" else " ".join(tokens)


class _Null:
    def __enter__(self):
        return None

    def __exit__(self, *a):
        return False


def _audio_inputs(opt):
    """Yields ``[frames, features]`` tensors for ``-encoder_type audio``."""
    from nmtgminor_b200.data import audio
    concat = int(str(getattr(opt, "concat", "1")).split("|")[0] or 1)
    if getattr(opt, "asr_format", "scp") == "scp":
        for _key, (path, offset) in audio.read_scp(opt.src).items():
            feats = torch.from_numpy(audio.read_ark_matrix(path, offset)).float()
            yield audio.stack_frames(feats, concat) if concat > 1 else feats
    else:
        with open(opt.src, encoding="utf-8") as fh:
            for line in fh:
                parts = line.split()
                if not parts:
                    continue
                path = parts[-1] if len(parts) <= 2 else parts[1]
                start = float(parts[2]) if len(parts) > 3 else 0.0
                end = float(parts[3]) if len(parts) > 3 else 0.0
                wav, _sr = audio.read_wav(path, start, end)
                yield torch.from_numpy(wav).float().view(-1, 1)


def main(argv=None):
    opt = make_translate_parser().parse_args(argv)
    opt.cuda = opt.gpu > -1 and torch.cuda.is_available()
    if getattr(opt, "streaming", False) or getattr(opt, "global_search", False):
        from nmtgminor_b200.inference.scoring import StreamTranslator
        translator = StreamTranslator(opt, context_tokens=getattr(opt, "max_memory_size", 0) and 8)
    else:
        translator = Translator(opt)
    if getattr(opt, "diverse_beamsearch", False):
        translator.cfg.diversity_rate = 0.5
    out = open(opt.output, "w", encoding="utf-8") if opt.output and opt.output != "stdout" else sys.stdout
    tgt_f = open(opt.tgt, encoding="utf-8") if getattr(opt, "tgt", None) else None
    # -past_src: the previous source sentence of every line (document-context models); an empty line = document start
    past_f = open(opt.past_src, encoding="utf-8") if getattr(opt, "past_src", None) else None
    past_batch = []
    # -sub_src: the source side read by the -sub_model members of the ensemble, line by line parallel to -src
    sub_f = open(opt.sub_src, encoding="utf-8") if getattr(opt, "sub_src", None) else None
    sub_batch = []
    pred_score_total = pred_words_total = gold_score_total = gold_words_total = 0.0
    src_batch, tgt_batch, count = [], [], 0
    t0 = time.time()

    def flush():
        nonlocal pred_score_total, pred_words_total, gold_score_total, gold_words_total, count, src_batch, tgt_batch, past_batch, sub_batch
        if not src_batch:
            return
        extra = {"past_sents": past_batch} if past_batch else {}
        if sub_batch:
            extra["sub_src_sents"] = sub_batch
        pred_batch, pred_ids, pred_score, pred_pos, pred_len, gold_score, gold_words, allgold = translator.translate(
            src_batch, tgt_batch if tgt_batch else None, **extra)
        for b in range(len(src_batch)):
            count += 1
            best = get_sentence_from_tokens(pred_batch[b][0], getattr(opt, "input_type", "word"))
            if getattr(opt, "print_nbest", False) and opt.n_best > 1:
                for n in range(len(pred_batch[b])):
                    out.write("%s ||| %.4f\n" % (get_sentence_from_tokens(pred_batch[b][n]), pred_score[b][n]))
            else:
                out.write(best + "\n")
            pred_score_total += pred_score[b][0] if math.isfinite(pred_score[b][0]) else 0.0
            pred_words_total += len(pred_batch[b][0]) + 1
            if tgt_batch:
                gold_score_total += gold_score[b]
            if opt.verbose:
                if not torch.is_tensor(src_batch[b]):
                    print("SENT %d: %s" % (count, " ".join(src_batch[b])))
                print("PRED %d: %s" % (count, best))
                print("PRED SCORE: %.4f" % pred_score[b][0])
                if tgt_batch:
                    print("GOLD %d: %s" % (count, " ".join(tgt_batch[b])))
                    print("GOLD SCORE: %.4f" % gold_score[b])
                print("")
        if tgt_batch:
            gold_words_total += gold_words
        out.flush()
        src_batch, tgt_batch, past_batch, sub_batch = [], [], [], []

    if getattr(opt, "encoder_type", "text") == "audio":
        # audio input: a Kaldi scp of feature matrices (``-asr_format scp``) or a list of wav paths (``wav``), one
        # utterance per line, in the order of the optional reference file
        for feats in _audio_inputs(opt):
            src_batch.append(feats)
            if tgt_f is not None:
                tgt_batch.append(tgt_f.readline().split())
            if sub_f is not None:
                sub_batch.append(sub_f.readline().split())
            if len(src_batch) >= opt.batch_size:
                flush()
        flush()
        src_lines = []
    else:
        src_lines = open(opt.src, encoding="utf-8")
    with src_lines if hasattr(src_lines, "close") else _Null() as src_f:
        for line in (src_f or []):
            toks = line.split()
            if getattr(opt, "input_type", "word") == "char":
                toks = list(line.strip())
            src_batch.append(toks)
            if tgt_f is not None:
                tgt_batch.append(tgt_f.readline().split())
            if past_f is not None:
                past_batch.append(past_f.readline().split())
            if sub_f is not None:
                sub_batch.append(sub_f.readline().split())
            if len(src_batch) >= opt.batch_size:
                flush()
    flush()
    if opt.verbose:
        report_score("PRED", pred_score_total, pred_words_total)
        if tgt_f is not None:
            report_score("GOLD", gold_score_total, gold_words_total)
        print("Translated %d sentences in %.1f s" % (count, time.time() - t0), file=sys.stderr)
    if out is not sys.stdout:
        out.close()
    if tgt_f is not None:
        tgt_f.close()
    if past_f is not None:
        past_f.close()
    if sub_f is not None:
        sub_f.close()


if __name__ == "__main__":
    main()
