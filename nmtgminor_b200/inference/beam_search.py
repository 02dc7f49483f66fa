"""Batched beam search with a fixed ``[sentences, beam]`` layout that never leaves the device.

Every step: the model scores the last symbol of all ``B * beam`` hypotheses (incremental key/value
caches), the ``2 * beam`` best continuations per sentence are taken from the flattened ``beam * V`` scores,
continuations ending in EOS are moved into a per-sentence table of finished hypotheses (kept sorted, best
``beam`` only), the first ``beam`` non-EOS continuations become the new active set and the decoder caches
are re-indexed accordingly.  A sentence stops when it has ``beam`` finished hypotheses and its best active
score can no longer enter the table; the loop ends when all sentences stopped or ``max_len`` is reached.
The batch is not shrunk when sentences finish (static shapes keep the step graph-capturable); finished
sentences simply stop contributing.  On a GPU the loop reads from the device only every fourth step (the "all sentences done" flag), finished sentences
are masked in between, and the decoder step is replayed as a CUDA graph (``BeamConfig.cuda_graph``); on the CPU one
``any()`` per step skips the merge of finished hypotheses when no EOS was produced.

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
    diversity_rate: float = 0.0  # > 0: sibling-rank penalty (the k-th best continuation of a hypothesis loses k * rate)
    vocab_mask: Optional[torch.Tensor] = None   # bool [V], True = allowed
    fused_step: bool = True     # CUDA: fused log-softmax + top-k kernel when no constraint needs full log-probabilities
    cuda_graph: bool = True     # CUDA + fused_step: replay the decoder step (embedding ... top-k) as a captured graph


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
    if cfg.diversity_rate > 0 and step > 0:
        # diverse beam search: only the best 2K continuations of a hypothesis can be selected, so ranking those suffices
        top_v, top_i = lprobs.topk(min(2 * K, V), dim=1)
        penalty = torch.arange(top_v.shape[1], device=device, dtype=lprobs.dtype) * cfg.diversity_rate
        lprobs = lprobs.scatter(1, top_i, top_v - penalty[None, :])

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


class _GraphedStep:
    """One decoding step (embedding, decoder layers over the preallocated caches, output projection, fused
    log-softmax + top-k) as CUDA graphs.  The cache write position and the token positions live on the device and are
    advanced inside the graph; hypothesis reordering swaps every layer's cache with its spare buffer, so there is one
    graph per swap parity.  The first steps (cache allocation, warm-up, steps that must not emit EOS) run eagerly
    through the same code."""

    def __init__(self, model, state, cfg, K: int, R: int):
        dev = state.context.device
        self.model, self.state, self.cfg, self.K = model, state, cfg, K
        cap = state.buffers[0].get("cap", 0)
        emb = getattr(model.decoder, "embed", None)
        if emb is not None and hasattr(emb, "renew"):
            before = id(getattr(emb, "pos", None))
            emb.renew(cap + 2)
            if id(getattr(emb, "pos", None)) != before:
                model.__dict__.pop("_decode_pools", None)      # graphs captured against the old position table are stale
        # Buffers and captured graphs are pooled on the model and reused by later batches of the same geometry
        # (rows, cache capacity, padded source length): the projected encoder states of a new batch are copied into
        # the pooled encoder-decoder caches, so the pointers recorded in the graphs stay valid.
        cross = [b for b in state.buffers if "c_k" in b and "c_len" in b]
        src_cap = (max(b["c_k"].shape[1] for b in cross) + 15) // 16 * 16 if cross else 0
        n_sent = cross[0]["c_k"].shape[0] if cross else 0
        key = (R, cap, n_sent, src_cap, len(state.buffers), str(dev), cfg.pad, cfg.eos)
        pools = model.__dict__.setdefault("_decode_pools", {})
        pool = pools.get(key)
        if pool is None:
            if len(pools) >= 4:
                pools.pop(next(iter(pools)))
            pool = pools[key] = {"graphs": {}, "layers": [dict() for _ in state.buffers], "eager_steps": 0,
                                 "tok": torch.zeros(R, dtype=torch.long, device=dev), "pos_t": torch.zeros(R, dtype=torch.long, device=dev),
                                 "scores": torch.zeros(R, dtype=torch.float32, device=dev),
                                 "force": torch.zeros(R, dtype=torch.uint8, device=dev),
                                 "pos_dev": torch.zeros(1, dtype=torch.int32, device=dev)}
        self.pool = pool
        self.tok, self.pos_t, self.scores, self.force = pool["tok"], pool["pos_t"], pool["scores"], pool["force"]
        self.graphs = pool["graphs"]
        self.pos_t.zero_()
        pool["pos_dev"].zero_()
        state.pos_dev = pool["pos_dev"]
        for buf, keep in zip(state.buffers, pool["layers"]):
            buf["pos_dev"] = pool["pos_dev"]
            if "c_k" in buf and "c_len" in buf:
                if "c_k" not in keep:
                    H = buf["c_k"].shape[2]
                    keep["c_k"] = torch.zeros(n_sent, src_cap, H, dtype=buf["c_k"].dtype, device=dev)
                    keep["c_v"] = torch.zeros_like(keep["c_k"])
                    keep["c_len"] = torch.zeros(n_sent, dtype=torch.int32, device=dev)
                ts = buf["c_k"].shape[1]
                keep["c_k"][:, :ts].copy_(buf["c_k"])
                keep["c_v"][:, :ts].copy_(buf["c_v"])
                keep["c_len"].copy_(buf["c_len"])
                buf["c_k"], buf["c_v"], buf["c_len"] = keep["c_k"], keep["c_v"], keep["c_len"]
            if "k" in keep:       # self-attention caches of an earlier batch: same pointers, contents are overwritten
                buf["k"], buf["v"], buf["k_spare"], buf["v_spare"] = keep["k"], keep["v"], keep["k_spare"], keep["v_spare"]

    def _body(self, ban_eos: bool):
        from .. import ops
        hidden = self.model.decoder.step_static(self.tok, self.pos_t, self.state)
        logits = self.model.generator(hidden)
        if logits.dtype not in (torch.float32, torch.bfloat16):
            logits = logits.float()
        ts, ti, _ = ops.ext().beam_topk(logits, self.scores, self.force, self.K, self.cfg.pad, self.cfg.eos, ban_eos)
        self.state.pos_dev.add_(1)
        self.pos_t.add_(1)
        return ts, ti, logits.shape[1]

    def run(self, last_tokens, scores, force_eos, ban_eos: bool, step: int):
        self.tok.copy_(last_tokens)
        self.scores.copy_(scores)
        # control byte per row: 1 = only EOS may follow (length limit), 2 = EOS banned (minimum length), 0 = free
        self.force.copy_(force_eos)
        if ban_eos:
            self.force.add_(2).clamp_(max=2).sub_(force_eos.to(torch.uint8))      # 0 -> 2, 1 -> 1
        key = self.state.buffers[0]["k"].data_ptr() if "k" in self.state.buffers[0] else None
        if key is None or self.pool["eager_steps"] < 2:
            self.pool["eager_steps"] += 1
            out = self._body(False)
            for buf, keep in zip(self.state.buffers, self.pool["layers"]):
                if "k" in buf and "k" not in keep:        # caches allocated by the first step: keep them for later batches
                    keep.update(k=buf["k"], v=buf["v"], k_spare=buf["k_spare"], v_spare=buf["v_spare"])
            return out
        entry = self.graphs.get(key)
        if entry is None:
            g = torch.cuda.CUDAGraph()
            torch.cuda.synchronize()
            with torch.cuda.graph(g):
                out = self._body(False)
            # capture records the launches without running them: replay once for this step's result
            self.graphs[key] = entry = (g, out)
        entry[0].replay()
        return entry[1]


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
             and not cfg.sampling and cfg.no_repeat_ngram_size <= 0 and cfg.vocab_mask is None and 2 * K <= 64
             and cfg.diversity_rate <= 0)

    graphed = None
    if (fused and cfg.cuda_graph and prefix_tokens is None and banned_first is None and hasattr(state, "enable_device_positions")
            and hasattr(getattr(model, "decoder", None), "step_static")):
        graphed = _GraphedStep(model, state, cfg, K, R)

    for step in range(T + 1):
        use_fused = (fused and not (prefix_tokens is not None and step < prefix_tokens.shape[1])
                     and not (banned_first is not None and step == 0))
        if graphed is not None:
            top_scores, top_idx, V = graphed.run(tokens[:, step], scores.reshape(-1), step >= max_rows, step < cfg.min_len, step)
            lprobs = None
        elif use_fused:
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
        # on a GPU the merge runs whenever EOS is possible instead of asking the device (`any()` would stall the host)
        if step >= cfg.min_len and (device.type == "cuda" or bool(is_eos.any())):
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
        if (device.type != "cuda" or step % 4 == 3 or step == T) and bool(done.all()):
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
