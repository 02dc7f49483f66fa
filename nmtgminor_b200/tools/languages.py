"""Checkpoint surgery for multilingual models: more languages for the per-language parameters, and language tables
re-ordered to another checkpoint's language dictionary.

``extend_languages`` covers the reference's ``extend_weight.py:21-161``: every parameter with one slice per language gets
``n_languages`` slices; the old slices are kept, the new ones start like fresh parameters of their kind (additive factors
and embeddings N(0, 0.02), multiplicative factors and norm scales 1, biases 0, adapters as a copy of language 0).
``rematch_language_table`` covers ``rematch_language_embedding.py:26-81``: rows of a language table move to the indices
that another checkpoint's ``dicts['langs']`` gives the same languages."""
from __future__ import annotations

import re
from typing import Dict, List

import torch

# parameter name endings of this framework's per-language tensors, with the value new slices start from
_ADDITIVE = re.compile(r"(^|\.)(r|s)$")                      # FactorizedLinear additive factors [n_lang, rank, dim]
_MULTIPLICATIVE = re.compile(r"(^|\.)(rm|sm)$")              # multiplicative factors [n_lang, 1, dim]
_TABLES = re.compile(r"(lang_embed|language_embedding|factor_embeddings)(\.\w+)*\.weight$")
_ML_NORM = re.compile(r"norm\.(weight|bias)$")               # MultilingualLayerNorm [n_lang, dim]
_ADAPTER = re.compile(r"^(.*adapters\.\d+\.adapters)\.(\d+)\.(.*)$")


def extend_languages(state: Dict[str, torch.Tensor], n_old: int, n_new: int, seed: int = 0) -> List[str]:
    """Grow the language dimension of ``state`` (a model state dict, modified in place) from ``n_old`` to ``n_new``.
    Returns the names that were extended or added."""
    if n_new <= n_old:
        return []
    gen = torch.Generator().manual_seed(seed)
    touched = []
    for name in list(state.keys()):
        p = state[name]
        if not torch.is_tensor(p) or p.dim() == 0 or p.shape[0] != n_old:
            continue
        if _ADDITIVE.search(name) or _TABLES.search(name):
            fresh = torch.randn((n_new - n_old,) + tuple(p.shape[1:]), generator=gen).to(p.dtype) * 0.02
        elif _MULTIPLICATIVE.search(name) or (_ML_NORM.search(name) and name.endswith("weight") and p.dim() == 2):
            fresh = torch.ones((n_new - n_old,) + tuple(p.shape[1:]), dtype=p.dtype)
        elif _ML_NORM.search(name) and name.endswith("bias") and p.dim() == 2:
            fresh = torch.zeros((n_new - n_old,) + tuple(p.shape[1:]), dtype=p.dtype)
        else:
            continue
        state[name] = torch.cat([p, fresh.to(p.device)], 0)
        touched.append(name)
    # adapters are sub-modules, one per language: new languages get a copy of language 0's adapter
    groups: Dict[str, Dict[int, List[str]]] = {}
    for name in state:
        m = _ADAPTER.match(name)
        if m:
            groups.setdefault(m.group(1), {}).setdefault(int(m.group(2)), []).append(m.group(3))
    for prefix, langs in groups.items():
        if len(langs) != n_old:
            continue
        for new in range(n_old, n_new):
            for tail in langs[0]:
                state["%s.%d.%s" % (prefix, new, tail)] = state["%s.0.%s" % (prefix, tail)].clone()
                touched.append("%s.%d.%s" % (prefix, new, tail))
    return touched


def rematch_language_table(weight: torch.Tensor, langs_old: Dict[str, int], langs_new: Dict[str, int]) -> torch.Tensor:
    """Rows of a ``[n_languages, ...]`` table re-ordered (and the table grown if needed) so that every language known to
    both dictionaries sits at its index in ``langs_new``; other rows keep what the old table had at that index, or small
    random values where the old table had nothing."""
    n = max(max(langs_new.values()) + 1, weight.shape[0]) if langs_new else weight.shape[0]
    out = torch.randn((n,) + tuple(weight.shape[1:]), generator=torch.Generator().manual_seed(0)).to(weight.dtype) * 0.02
    out[:weight.shape[0]] = weight
    for lang, old in langs_old.items():
        if lang in langs_new and old < weight.shape[0]:
            out[langs_new[lang]] = weight[old]
    return out
