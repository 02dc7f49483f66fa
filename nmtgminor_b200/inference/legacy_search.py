"""The classic per-sentence beam (``Beam``), pluggable candidate-selection strategies (``BeamSearch``,
``DiverseBeamSearch``, ``Sampling``) and the two translators built on them: ``LegacyTranslator`` (one ``Beam`` object per
sentence, the algorithm of the original OpenNMT decoder) and ``GlobalStreamTranslator`` (documents decoded segment by
segment with ONE beam that lives across segments: hypothesis scores, lengths and decoder memories are carried over
instead of being reset at every segment border).

The device-resident batched search in ``beam_search.py`` is the fast path; the classes here are the reference's other
search API, kept for its users (custom rescoring loops call ``Beam.advance`` directly) and used by the tests as an
independent oracle of the fast path.

Reference: onmt/inference/Beam.py:20-139 (``Beam``), onmt/inference/search.py:15-347 (strategies),
onmt/inference/translator.py:331-480 (``translate_batch`` with Beam objects),
onmt/inference/global_translator.py:13-603 and onmt/inference/stream_translator.py:13-522 (stream translators).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import constants as C
from .beam_search import BeamConfig, Hypothesis
from .translator import Translator


class Beam:
    """Beam of one sentence.  ``advance(word_lk, attn)`` takes the ``[beam, vocab]`` log-probabilities of the next word
    for every live hypothesis, keeps the best ``size`` continuations, and records back-pointers so that
    ``get_hyp(k)`` can walk a hypothesis back to the start.  ``done`` turns true when the best hypothesis ends in EOS.
    """

    def __init__(self, size: int, bos_id: int = C.BOS, cuda: bool = False, sampling: bool = False, eos_id: int = C.EOS,
                 pad_id: int = C.PAD):
        self.size = size
        self.done = False
        self.sampling = sampling
        self.eos, self.pad = eos_id, pad_id
        dev = torch.device("cuda") if cuda else torch.device("cpu")
        self.scores = torch.zeros(size, device=dev)
        self.all_scores: List[torch.Tensor] = []
        self.prev_ks: List[torch.Tensor] = []                                   # back-pointers per step
        first = torch.full((size,), pad_id, dtype=torch.long, device=dev)
        first[0] = bos_id
        self.next_ys: List[torch.Tensor] = [first]                                # outputs per step
        self.attn: List[torch.Tensor] = []
        self.finished: List[Tuple[float, int, int]] = []                         # (score, step, beam index)

    # reference spellings
    def getCurrentState(self):
        return self.get_current_state()

    def getCurrentOrigin(self):
        return self.get_current_origin()

    def get_current_state(self) -> torch.Tensor:
        return self.next_ys[-1]

    def get_current_origin(self) -> torch.Tensor:
        return self.prev_ks[-1]

    def advance(self, word_lk: torch.Tensor, attn: Optional[torch.Tensor] = None) -> bool:
        num_words = word_lk.size(1)
        if self.prev_ks:
            beam_lk = word_lk + self.scores[:, None]
            # a hypothesis that already ended can only be continued by padding-free EOS at unchanged score
            ended = self.next_ys[-1] == self.eos
            if bool(ended.any()):
                beam_lk = beam_lk.clone()
                beam_lk[ended] = float("-inf")
                beam_lk[ended, self.eos] = self.scores[ended]
        else:
            beam_lk = word_lk[0:1]                                                # only the BOS row is alive
        flat = beam_lk.reshape(-1)
        if self.sampling and self.prev_ks:
            probs = torch.softmax(word_lk, -1)
            pick = torch.multinomial(probs, 1).squeeze(1)
            best_scores = self.scores + word_lk.gather(1, pick[:, None]).squeeze(1)
            best_ids = torch.arange(self.size, device=flat.device) * num_words + pick
        else:
            k = min(self.size, flat.numel())
            best_scores, best_ids = flat.topk(k, 0, True, True)
            if k < self.size:
                fill = self.size - k
                best_scores = torch.cat([best_scores, best_scores.new_full((fill,), float("-inf"))])
                best_ids = torch.cat([best_ids, best_ids.new_zeros(fill)])
        self.all_scores.append(self.scores)
        self.scores = best_scores
        prev_k = best_ids // num_words
        self.prev_ks.append(prev_k)
        self.next_ys.append(best_ids - prev_k * num_words)
        if attn is not None:
            self.attn.append(attn.index_select(0, prev_k))
        for i in range(self.size):
            if int(self.next_ys[-1][i]) == self.eos and math.isfinite(float(self.scores[i])):
                self.finished.append((float(self.scores[i]), len(self.next_ys) - 1, i))
        if int(self.next_ys[-1][0]) == self.eos:
            self.done = True
        return self.done

    def sort_best(self):
        return torch.sort(self.scores, 0, True)

    sortBest = sort_best

    def get_best(self):
        scores, ids = self.sort_best()
        return scores[0], ids[0]

    getBest = get_best

    def get_hyp(self, k: int):
        """Walks back from beam slot ``k`` of the last step; returns (tokens without BOS, attention rows)."""
        hyp, attn = [], []
        for j in range(len(self.prev_ks) - 1, -1, -1):
            hyp.append(int(self.next_ys[j + 1][k]))
            if self.attn:
                attn.append(self.attn[j][k])
            k = int(self.prev_ks[j][k])
        hyp.reverse()
        attn.reverse()
        # the padding-free continuation repeats EOS after the end: keep one
        if self.eos in hyp:
            cut = hyp.index(self.eos) + 1
            hyp, attn = hyp[:cut], attn[:cut]
        return hyp, (torch.stack(attn) if attn else None)

    getHyp = get_hyp


# ---------------------------------------------------------------------------------------------------------
# candidate-selection strategies (batched): step(step, lprobs [B, K, V], scores [B, K, step]) -> scores, tokens, beams [B, 2K]
# ---------------------------------------------------------------------------------------------------------
class Search:
    def __init__(self, tgt_dict=None, pad: int = C.PAD, eos: int = C.EOS, unk: int = C.UNK):
        self.pad, self.eos, self.unk = pad, eos, unk
        self.vocab_size = tgt_dict.size() if tgt_dict is not None and hasattr(tgt_dict, "size") else None
        self.src_lengths = None

    def set_src_lengths(self, src_lengths):
        self.src_lengths = src_lengths

    def step(self, step: int, lprobs: torch.Tensor, scores: Optional[torch.Tensor]):
        raise NotImplementedError


class BeamSearch(Search):
    def step(self, step, lprobs, scores):
        B, K, V = lprobs.shape
        if step == 0:
            lprobs = lprobs[:, ::K, :].contiguous()                               # all beams are equal at the first step
        else:
            lprobs = lprobs + scores[:, :, step - 1].unsqueeze(-1)
        top_scores, top_idx = lprobs.view(B, -1).topk(min(2 * K, lprobs.view(B, -1).size(1) - 1), dim=1)
        return top_scores, top_idx % V, top_idx // V


class DiverseBeamSearch(Search):
    """Beams are split into ``num_groups`` groups searched one after another; a word already chosen by an earlier group
    at this step is penalised by ``diversity_strength`` per earlier use (Vijayakumar et al., 2016)."""

    def __init__(self, tgt_dict=None, num_groups: int = 2, diversity_strength: float = 0.5, **kw):
        super().__init__(tgt_dict, **kw)
        self.num_groups = num_groups
        self.diversity_strength = -abs(diversity_strength)
        self.beam = BeamSearch(tgt_dict, **kw)

    def step(self, step, lprobs, scores):
        B, K, V = lprobs.shape
        if K % self.num_groups != 0:
            raise ValueError("beam size must be divisible by the number of groups")
        used = torch.zeros(B, V, device=lprobs.device, dtype=lprobs.dtype)
        s_g, i_g, b_g = [], [], []
        for g in range(self.num_groups):
            lp = lprobs[:, g::self.num_groups, :]
            sc = scores[:, g::self.num_groups, :] if step > 0 else None
            if g > 0:
                lp = lp + self.diversity_strength * used.unsqueeze(1)
            s, i, b = self.beam.step(step, lp.contiguous(), sc)
            b = b * self.num_groups + g
            s_g.append(s)
            i_g.append(i)
            b_g.append(b)
            used.scatter_add_(1, i, torch.ones_like(i, dtype=used.dtype))
        # interleave the groups' results so that slot j belongs to group j % num_groups
        stack = lambda xs: torch.stack(xs, dim=2).view(B, -1)
        return stack(s_g), stack(i_g), stack(b_g)


class Sampling(Search):
    """Draws the continuation of every beam from the (top-k or top-p truncated) distribution instead of ranking."""

    def __init__(self, tgt_dict=None, sampling_topk: int = -1, sampling_topp: float = -1.0, **kw):
        super().__init__(tgt_dict, **kw)
        self.sampling_topk, self.sampling_topp = sampling_topk, sampling_topp

    def _truncate(self, probs):
        if self.sampling_topk > 0:
            top, idx = probs.topk(min(self.sampling_topk, probs.size(-1)), dim=-1)
            return top, idx
        if self.sampling_topp > 0:
            sp, si = probs.sort(dim=-1, descending=True)
            cum = sp.cumsum(-1)
            keep = cum - sp < self.sampling_topp                                   # smallest prefix with mass >= p
            last = int(keep.sum(-1).max())
            sp, si, keep = sp[..., :last], si[..., :last], keep[..., :last]
            return sp.masked_fill(~keep, 0.0), si
        return probs, None

    def step(self, step, lprobs, scores):
        B, K, V = lprobs.shape
        if step == 0:
            lprobs = lprobs[:, ::K, :].contiguous()
        probs, idx = self._truncate(lprobs.exp())
        rows = probs.view(-1, probs.size(-1))
        n_draw = K if step == 0 else 1
        draw = torch.multinomial(rows, n_draw, replacement=True).view(B, -1)
        if step == 0:
            beams = torch.zeros(B, K, dtype=torch.long, device=lprobs.device)
            pick_p = probs[:, 0, :].gather(1, draw)
            tok = idx[:, 0, :].gather(1, draw) if idx is not None else draw
            sc = pick_p.log()
        else:
            beams = torch.arange(K, device=lprobs.device).repeat(B, 1)
            pick_p = probs.gather(2, draw.unsqueeze(-1)).squeeze(-1)
            tok = idx.gather(2, draw.unsqueeze(-1)).squeeze(-1) if idx is not None else draw
            sc = pick_p.log() + scores[:, :, step - 1]
        return sc, tok, beams


# ---------------------------------------------------------------------------------------------------------
# translators
# ---------------------------------------------------------------------------------------------------------
class LegacyTranslator(Translator):
    """``translate_batch`` with one ``Beam`` object per sentence: every step scores all ``batch * beam`` rows, hands
    each sentence's ``[beam, vocab]`` slice to its ``Beam``, and re-orders the decoder state by the beams' back-pointers.
    Slower than the device-resident search (the host touches every beam every step) but it is the reference's other
    public search API and an independent check of the fast one."""

    def translate_batch(self, batch, prefix_tokens=None, banned_first=None) -> List[List[Hypothesis]]:
        if prefix_tokens is not None or banned_first is not None:
            return super().translate_batch(batch, prefix_tokens, banned_first)
        cfg: BeamConfig = self.cfg
        if self.cuda:
            batch = batch.cuda(self.device)
        K = cfg.beam_size
        with torch.no_grad():
            state = self.model.create_decoder_state(batch, K)
            B = state.context.shape[0] // K
            dev = state.context.device
            beams = [Beam(K, cfg.bos, cuda=dev.type == "cuda", sampling=cfg.sampling, eos_id=cfg.eos, pad_id=cfg.pad)
                     for _ in range(B)]
            tokens = torch.full((B * K, 1), cfg.bos, dtype=torch.long, device=dev)
            base = torch.arange(B, device=dev) * K
            for step in range(cfg.max_len + 1):
                lp = self.model.step(tokens, state)["log_prob"].float().view(B, K, -1)
                if step < cfg.min_len:
                    lp[:, :, cfg.eos] = float("-inf")
                if step >= cfg.max_len:
                    forced = torch.full_like(lp, float("-inf"))
                    forced[:, :, cfg.eos] = 0.0
                    lp = forced
                lp[:, :, cfg.pad] = float("-inf")
                origin, nxt = [], []
                for b, beam in enumerate(beams):
                    if not beam.done:
                        beam.advance(lp[b])
                    else:                                   # a finished sentence idles: same rows, EOS again
                        beam.prev_ks.append(torch.arange(K, device=dev))
                        beam.next_ys.append(torch.full((K,), cfg.eos, dtype=torch.long, device=dev))
                    origin.append(base[b] + beam.get_current_origin())
                    nxt.append(beam.get_current_state())
                if all(beam.done for beam in beams):
                    break
                reorder = torch.cat(origin)
                tokens = torch.cat([tokens.index_select(0, reorder), torch.cat(nxt)[:, None]], 1)
                state.reorder(reorder)
        out: List[List[Hypothesis]] = []
        for beam in beams:
            norm = lambda s, n: s / (float(n) ** cfg.alpha) if (cfg.normalize and cfg.alpha > 0) else s
            fin = sorted(beam.finished, key=lambda f: -norm(f[0], f[1]))
            hyps, seen = [], set()
            for score, t, k in fin:
                # walk back from (step t, slot k)
                toks, kk = [], k
                for j in range(t - 1, -1, -1):
                    toks.append(int(beam.next_ys[j + 1][kk]))
                    kk = int(beam.prev_ks[j][kk])
                toks.reverse()
                if cfg.eos in toks[:-1]:
                    continue                                # the idle continuation of an already finished hypothesis
                key = tuple(toks)
                if key in seen:
                    continue
                seen.add(key)
                hyps.append(Hypothesis(toks, norm(score, t)))
                if len(hyps) >= cfg.n_best:
                    break
            if not hyps:
                toks, _ = beam.get_hyp(0)
                hyps.append(Hypothesis(toks, float(beam.scores[0])))
            out.append(hyps)
        return out


class GlobalStreamTranslator(Translator):
    """Decodes a document segment by segment with a beam that is global to the document: the ``beam_size`` hypotheses
    that survive a segment - their cumulative scores, lengths and the last ``context_tokens`` target words - open the
    next segment, so a locally second-best choice can still win once later segments have been seen.  Models with
    segment memories (``init_stream``) keep them across segments as well.  ``reset_stream()`` starts a new document.

    ``translate_segment(src_tokens)`` returns the current best hypothesis' words for this segment;
    ``document()`` returns the best whole-document hypothesis so far as a list of segments."""

    def __init__(self, opt, context_tokens: int = 0):
        super().__init__(opt)
        self.context_tokens = int(context_tokens or getattr(opt, "stream_context_tokens", 0) or 0)
        self.max_memory_size = int(getattr(opt, "max_memory_size", 512) or 512)
        self.reset_stream()

    def reset_stream(self):
        K = self.cfg.beam_size
        self.prev_scores = torch.full((K,), float("-inf"))
        self.prev_scores[0] = 0.0
        self.prev_lengths = torch.zeros(K, dtype=torch.long)
        self.prev_hyps: List[List[List[int]]] = [[] for _ in range(K)]            # per beam: list of segments (token ids)
        self.stream = self.model.init_stream() if hasattr(self.model, "init_stream") else None

    def _norm(self, score: float, length: int) -> float:
        cfg = self.cfg
        return score / (float(max(length, 1)) ** cfg.alpha) if (cfg.normalize and cfg.alpha > 0) else score

    @torch.no_grad()
    def translate_segment(self, src_tokens: Sequence[str]) -> List[str]:
        cfg: BeamConfig = self.cfg
        K = cfg.beam_size
        batch = self.build_data([list(src_tokens)])
        if self.cuda:
            batch = batch.cuda(self.device)
        state = self.model.create_decoder_state(batch, K, streaming_state=self.stream)
        dev = state.context.device
        flat_prev = [[t for seg in h for t in seg] for h in self.prev_hyps]
        c = min([self.context_tokens] + [len(h) for h in flat_prev]) if self.context_tokens > 0 else 0
        tokens = torch.full((K, 1), cfg.bos, dtype=torch.long, device=dev)
        for j in range(c):                                                       # forced, unscored context of every beam
            self.model.step(tokens, state)
            col = torch.tensor([h[len(h) - c + j] for h in flat_prev], dtype=torch.long, device=dev)
            tokens = torch.cat([tokens, col[:, None]], 1)
        scores = self.prev_scores.to(dev).clone()
        origin_slot = torch.arange(K, device=dev)                                # which carried hypothesis a row descends from
        src_len = int((~state.src_pad_mask[0]).sum())
        max_len = int(min(cfg.max_len, cfg.len_a * src_len + cfg.len_b)) if cfg.dynamic_max_len else cfg.max_len
        finished: List[Tuple[float, List[int], int]] = []                         # (cumulative score, new tokens, origin slot)
        for step in range(max_len + 1):
            lp = self.model.step(tokens, state)["log_prob"].float()
            lp[:, cfg.pad] = float("-inf")
            if step < cfg.min_len:
                lp[:, cfg.eos] = float("-inf")
            if step >= max_len:
                forced = torch.full_like(lp, float("-inf"))
                forced[:, cfg.eos] = 0.0
                lp = forced
            V = lp.shape[1]
            cand = (scores[:, None] + lp).view(-1)
            top, idx = cand.topk(min(2 * K, cand.numel()))
            rows, toks = (idx // V).tolist(), (idx % V).tolist()
            keep_rows, keep_toks, keep_scores = [], [], []
            for rank, (s, r, t) in enumerate(zip(top.tolist(), rows, toks)):
                if not math.isfinite(s):
                    continue
                if t == cfg.eos:
                    if rank < K:
                        finished.append((s, tokens[r, 1 + c:].tolist(), int(origin_slot[r])))
                    continue
                if len(keep_rows) < K:
                    keep_rows.append(r)
                    keep_toks.append(t)
                    keep_scores.append(s)
            if len(finished) >= K or not keep_rows:
                break
            while len(keep_rows) < K:                                            # fewer live candidates than slots
                keep_rows.append(keep_rows[0])
                keep_toks.append(keep_toks[0])
                keep_scores.append(float("-inf"))
            reorder = torch.tensor(keep_rows, dtype=torch.long, device=dev)
            tokens = torch.cat([tokens.index_select(0, reorder), torch.tensor(keep_toks, device=dev)[:, None]], 1)
            scores = torch.tensor(keep_scores, device=dev)
            origin_slot = origin_slot.index_select(0, reorder)
            state.reorder(reorder)
        if not finished:
            finished.append((float(scores[0]), tokens[0, 1 + c:].tolist(), int(origin_slot[0])))
        prev_len = self.prev_lengths.tolist()
        finished.sort(key=lambda f: -self._norm(f[0], prev_len[f[2]] + len(f[1]) + 1))
        finished = finished[:K]
        new_hyps, new_scores, new_lengths = [], [], []
        for s, toks, slot in finished:
            new_hyps.append(self.prev_hyps[slot] + [toks])
            new_scores.append(s)
            new_lengths.append(prev_len[slot] + len(toks) + 1)
        while len(new_hyps) < K:
            new_hyps.append(new_hyps[0])
            new_scores.append(float("-inf"))
            new_lengths.append(new_lengths[0])
        self.prev_hyps, self.prev_scores = new_hyps, torch.tensor(new_scores)
        self.prev_lengths = torch.tensor(new_lengths, dtype=torch.long)
        if self.stream is not None and hasattr(self.stream, "trim"):
            self.stream.trim(self.max_memory_size)
        return self.tgt_dict.convert_to_labels(new_hyps[0][-1], self.eos, including_stop=False)

    def document(self) -> List[List[str]]:
        return [self.tgt_dict.convert_to_labels(seg, self.eos, including_stop=False) for seg in self.prev_hyps[0]]
