"""Batched beam search with a fixed ``[sentences, beam]`` layout that never leaves the device.

Every step: the model scores the last symbol of all ``B * beam`` hypotheses (incremental key/value
caches), the ``2 * beam`` best continuations per sentence are taken from the flattened ``beam * V`` scores,
continuations ending in EOS are moved into a per-sentence table of finished hypotheses (kept sorted, best
``beam`` only), the first ``beam`` non-EOS continuations become the new active set and the decoder caches
are re-indexed accordingly.  A sentence stops when it has ``beam`` finished hypotheses and its best active
score can no longer enter the table; the loop ends when all sentences stopped or ``max_len`` is reached.
The batch is not shrunk when sentences finish (static shapes keep the step graph-capturable); finished
sentences simply stop contributing.  One ``any()`` read per step is the only host synchronisation.

Constraints supported: minimum length, maximum length (absolute or ``a * src_len + b``), length-normalised
scores (``score / len^alpha``), n-gram blocking, forced target prefixes, banned first tokens, vocabulary
masks, sampling instead of top-k.

Functional counterpart of the reference's ``FastTranslator._translate_batch``
(onmt/inference/fast_translator.py:428-1010) and ``BeamSearch.step`` (onmt/inference/search.py:62-106).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch


@dataclass
class BeamConfig:
    beam_size: int = 4
    n_best: int = 1
    max_len: int = 256
    min_len: int = 1
    dynamic_max_len: bool = False
    len_a: float = 1.5          # max_len = len_a * src_len + len_b when dynamic
    len_b: float = 10.0
    alpha: float = 0.0          # length-penalty exponent (0 = raw sum of log-probabilities)
    normalize: bool = False
    no_repeat_ngram_size: int = 0
    bos: int = 2
    eos: int = 3
    pad: int = 0
    sampling: bool = False
    sampling_temperature: float = 1.0
    vocab_mask: Optional[torch.Tensor] = None   # bool [V], True = allowed
    fused_step: bool = True     # CUDA: fused log-softmax + top-k kernel when no constraint needs full log-probabilities


@dataclass
class Hypothesis:
    tokens: List[int]
    score: float
    positional_scores: List[float] = field(default_factory=list)


def _block_ngrams(tokens, step, lprobs, n, pad):
    """Set to -inf every symbol that would complete an n-gram already present in its hypothesis."""
    if n <= 0 or step + 1 < n:
        return lprobs
    hist = tokens[:, :step + 1]
    R = hist.shape[0]
    if n == 1:
        lprobs.scatter_(1, hist, float("-inf"))
        return lprobs
    prefix = hist[:, -(n - 1):]                                   # last n-1 symbols
    windows = hist.unfold(1, n, 1)                                # [R, W, n]
    match = (windows[:, :, :n - 1] == prefix[:, None, :]).all(-1)  # [R, W]
    banned = windows[:, :, n - 1]
    rows = torch.arange(R, device=tokens.device)[:, None].expand_as(banned)
    lprobs[rows[match], banned[match]] = float("-inf")
    return lprobs


def _masked_topk(lprobs, cfg, step, max_rows, prefix_tokens, banned_first, tokens, scores, B, K):
    """Reference step: apply the length / prefix / n-gram constraints to ``lprobs`` [R, V] and pick 2K candidates."""
    device = lprobs.device
    R = B * K
    V = lprobs.shape[1]
    lprobs[:, cfg.pad] = float("-inf")
    if cfg.vocab_mask is not None:
        lprobs.masked_fill_(~cfg.vocab_mask[None, :].to(device), float("-inf"))
    if step < cfg.min_len:
        lprobs[:, cfg.eos] = float("-inf")
    force_eos = (step >= max_rows)                             # at the length limit only EOS may follow
    if force_eos.any():
        keep = lprobs[:, cfg.eos].clone()
        lprobs[force_eos] = float("-inf")
        lprobs[force_eos, cfg.eos] = keep[force_eos]
    if prefix_tokens is not None and step < prefix_tokens.shape[1]:
        want = prefix_tokens[:, step].repeat_interleave(K)
        forced = want != cfg.pad
        if forced.any():
            keep = lprobs.gather(1, want[:, None]).squeeze(1)
            lprobs[forced] = float("-inf")
            lprobs[forced, want[forced]] = keep[forced]
    if banned_first is not None and step == 0:
        lprobs[:, banned_first] = float("-inf")
    lprobs = _block_ngrams(tokens, step, lprobs, cfg.no_repeat_ngram_size, cfg.pad)

    cand = scores[:, :, None] + lprobs.view(B, K, V)            # [B, K, V]
    flat = cand.view(B, K * V)
    if cfg.sampling and step > 0:
        probs = torch.softmax(lprobs.view(B, K, V) / cfg.sampling_temperature, -1)
        samp = torch.multinomial(probs.view(R, V), 2).view(B, K * 2)
        beam_of = torch.arange(K, device=device).repeat_interleave(2)[None, :].expand(B, -1)
        top_idx = beam_of * V + samp
        top_scores = flat.gather(1, top_idx)
    else:
        top_scores, top_idx = flat.topk(min(2 * K, K * V), dim=1)
    return top_scores, top_idx, V


@torch.no_grad()
def beam_search(model, batch, cfg: BeamConfig, prefix_tokens: Optional[torch.Tensor] = None,
                banned_first: Optional[torch.Tensor] = None) -> List[List[Hypothesis]]:
    """Decode every sentence of ``batch``; returns ``n_best`` hypotheses per sentence (best first)."""
    K = cfg.beam_size
    state = model.create_decoder_state(batch, K)
    # batch size / source lengths come from the encoder output, so audio batches (no packed source) work too
    device = state.context.device
    B = state.context.shape[0] // K
    src_len = (~state.src_pad_mask).sum(1)[::K].to(torch.float32)
    if cfg.dynamic_max_len:
        max_len_per = (cfg.len_a * src_len + cfg.len_b).clamp(max=cfg.max_len).long()
    else:
        max_len_per = torch.full((B,), cfg.max_len, device=device, dtype=torch.long)
    T = int(max_len_per.max().item())
    R = B * K
    tokens = torch.full((R, T + 2), cfg.pad, dtype=torch.long, device=device)
    tokens[:, 0] = cfg.bos
    pos_scores = torch.zeros((R, T + 2), dtype=torch.float32, device=device)
    scores = torch.zeros((B, K), dtype=torch.float32, device=device)
    scores[:, 1:] = float("-inf")                                  # only beam 0 is alive at step 0
    fin_scores = torch.full((B, K), float("-inf"), device=device)
    fin_tokens = torch.full((B, K, T + 2), cfg.pad, dtype=torch.long, device=device)
    fin_pos = torch.zeros((B, K, T + 2), dtype=torch.float32, device=device)
    fin_len = torch.zeros((B, K), dtype=torch.long, device=device)
    fin_count = torch.zeros(B, dtype=torch.long, device=device)
    done = torch.zeros(B, dtype=torch.bool, device=device)
    base = (torch.arange(B, device=device) * K)[:, None]
    max_rows = max_len_per.repeat_interleave(K)

    if hasattr(state, "set_cache_capacity") and device.type == "cuda":
        state.set_cache_capacity(T + 2)
    # fused step: log-softmax, masks and the per-sentence top-2K in two kernels, no [R, V] log-probabilities
    fused = (device.type == "cuda" and cfg.fused_step and getattr(model, "supports_logits_step", False)
             and not cfg.sampling and cfg.no_repeat_ngram_size <= 0 and cfg.vocab_mask is None and 2 * K <= 64)

    for step in range(T + 1):
        use_fused = (fused and not (prefix_tokens is not None and step < prefix_tokens.shape[1])
                     and not (banned_first is not None and step == 0))
        if use_fused:
            from .. import ops
            logits = model.step(tokens[:, :step + 1], state, logits_only=True)["logits"]
            V = logits.shape[1]
            if logits.dtype not in (torch.float32, torch.bfloat16):
                logits = logits.float()
            top_scores, top_idx, _ = ops.ext().beam_topk(logits, scores.reshape(-1).contiguous(),
                                                         (step >= max_rows).to(torch.uint8), K, cfg.pad, cfg.eos,
                                                         step < cfg.min_len)
            lprobs = None
        else:
            top_scores = None
            out = model.step(tokens[:, :step + 1], state)
            lprobs = out["log_prob"].float()                       # [R, V]
        if lprobs is not None:
            top_scores, top_idx, V = _masked_topk(lprobs, cfg, step, max_rows, prefix_tokens, banned_first, tokens, scores, B, K)
        cand_beam = top_idx // V
        cand_tok = top_idx % V
        C = top_scores.shape[1]
        is_eos = (cand_tok == cfg.eos) & torch.isfinite(top_scores)
        # an EOS candidate only counts when it is within the top `beam` of the step (fairseq convention)
        is_eos &= torch.arange(C, device=device)[None, :] < K
        is_eos &= ~done[:, None]

        # ---- finalize: merge EOS candidates into the sorted table of finished hypotheses ---------
        if is_eos.any():
            length = step + 1                                      # symbols after BOS, including EOS
            norm = (float(length) ** cfg.alpha) if (cfg.normalize and cfg.alpha > 0) else 1.0
            new_scores = torch.where(is_eos, top_scores / norm, torch.full_like(top_scores, float("-inf")))
            src_rows = (base + cand_beam).view(-1)
            new_tok = tokens[src_rows].view(B, C, T + 2).clone()
            new_tok[:, :, step + 1] = cfg.eos
            new_pos = pos_scores[src_rows].view(B, C, T + 2).clone()
            new_pos[:, :, step + 1] = top_scores - scores.gather(1, cand_beam)
            all_scores = torch.cat([fin_scores, new_scores], 1)
            order = all_scores.argsort(dim=1, descending=True, stable=True)[:, :K]
            gather3 = order[:, :, None].expand(-1, -1, T + 2)
            fin_tokens = torch.cat([fin_tokens, new_tok], 1).gather(1, gather3)
            fin_pos = torch.cat([fin_pos, new_pos], 1).gather(1, gather3)
            fin_len = torch.cat([fin_len, torch.full((B, C), length, device=device, dtype=torch.long)], 1).gather(1, order)
            fin_scores = all_scores.gather(1, order)
            fin_count = (fin_count + is_eos.sum(1)).clamp(max=K)

        # ---- next active set: first K non-EOS candidates -----------------------------------------
        alive_key = torch.where(cand_tok == cfg.eos, torch.full_like(top_scores, float("-inf")), top_scores)
        act_scores, act_pos = alive_key.topk(K, dim=1)
        act_beam = cand_beam.gather(1, act_pos)
        act_tok = cand_tok.gather(1, act_pos)
        reorder = (base + act_beam).view(-1)
        tokens = tokens.index_select(0, reorder)
        pos_scores = pos_scores.index_select(0, reorder)
        tokens[:, step + 1] = act_tok.view(-1)
        pos_scores[:, step + 1] = (act_scores - scores.gather(1, act_beam)).view(-1)
        scores = act_scores
        state.reorder(reorder)

        # ---- stopping ------------------------------------------------------------------------------
        best_possible = scores[:, 0] / ((float(T + 1) ** cfg.alpha) if (cfg.normalize and cfg.alpha > 0) else 1.0)
        worst_fin = fin_scores[:, K - 1]
        stop_early = (best_possible <= worst_fin) if cfg.normalize else torch.ones_like(done)
        done = done | ((fin_count >= K) & stop_early) | ~torch.isfinite(scores[:, 0])
        scores = torch.where(done[:, None], torch.full_like(scores, float("-inf")), scores)
        if bool(done.all()):
            break

    fin_scores_c, fin_tokens_c, fin_len_c, fin_pos_c = fin_scores.cpu(), fin_tokens.cpu(), fin_len.cpu(), fin_pos.cpu()
    results: List[List[Hypothesis]] = []
    for b in range(B):
        hyps = []
        for k in range(min(cfg.n_best, K)):
            if not torch.isfinite(fin_scores_c[b, k]):
                continue
            n = int(fin_len_c[b, k])
            hyps.append(Hypothesis(fin_tokens_c[b, k, 1:n + 1].tolist(), float(fin_scores_c[b, k]),
                                   fin_pos_c[b, k, 1:n + 1].tolist()))
        if not hyps:
            hyps.append(Hypothesis([cfg.eos], float("-inf")))
        results.append(hyps)
    return results


@torch.no_grad()
def greedy_search(model, batch, max_len: int = 256, bos: int = 2, eos: int = 3, pad: int = 0) -> List[List[int]]:
    state = model.create_decoder_state(batch, 1)
    B = state.context.shape[0]
    device = state.context.device
    tokens = torch.full((B, max_len + 2), pad, dtype=torch.long, device=device)
    tokens[:, 0] = bos
    finished = torch.zeros(B, dtype=torch.bool, device=device)
    for step in range(max_len + 1):
        lp = model.step(tokens[:, :step + 1], state)["log_prob"]
        lp[:, pad] = float("-inf")
        nxt = lp.argmax(-1)
        nxt = torch.where(finished, torch.full_like(nxt, pad), nxt)
        tokens[:, step + 1] = nxt
        finished |= nxt == eos
        if bool(finished.all()):
            break
    out = []
    for row in tokens[:, 1:].tolist():
        seq = []
        for t in row:
            if t == pad:
                break
            seq.append(t)
            if t == eos:
                break
        out.append(seq)
    return out
