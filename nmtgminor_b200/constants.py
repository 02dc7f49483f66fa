"""Special-token ids and run-wide switches.

The reference keeps these as mutable module globals (onmt/constants.py:3-18) that ``add_tokenidx``
(:50-93) rebinds from the dictionaries; here they are fields of a ``Constants`` object created per
run (``Constants.from_dicts``) and passed explicitly, with a module-level default instance for callers
that do not care.
"""
from __future__ import annotations

from dataclasses import dataclass

PAD, UNK, BOS, EOS = 0, 1, 2, 3
PAD_WORD, UNK_WORD, BOS_WORD, EOS_WORD = "<blank>", "<unk>", "<s>", "</s>"


# the options that name the special tokens of each dictionary (mBART / DeltaLM vocabularies use <pad>, </s>, ...)
_SPECIAL_WORD_OPTIONS = {
    "src": {"pad": "src_pad_word", "unk": "src_unk_word", "bos": "src_bos_word", "eos": "src_eos_word"},
    "tgt": {"pad": "tgt_pad_word", "unk": "tgt_unk_word", "bos": "tgt_bos_word", "eos": "tgt_eos_word"},
}


@dataclass
class Constants:
    PAD: int = PAD
    UNK: int = UNK
    BOS: int = BOS
    EOS: int = EOS
    SRC_PAD: int = PAD
    SRC_UNK: int = UNK
    SRC_BOS: int = BOS
    SRC_EOS: int = EOS
    TGT_PAD: int = PAD
    TGT_UNK: int = UNK
    TGT_BOS: int = BOS
    TGT_EOS: int = EOS
    PAD_WORD: str = PAD_WORD
    UNK_WORD: str = UNK_WORD
    BOS_WORD: str = BOS_WORD
    EOS_WORD: str = EOS_WORD
    checkpointing: int = 0
    max_position_length: int = 8192
    static: bool = False
    recompute: bool = False
    double_precision: bool = False
    weight_norm: bool = False

    @staticmethod
    def from_dicts(opt, dicts) -> "Constants":
        """Bind the special ids to the words named by ``-src_pad_word`` ... ``-tgt_eos_word``."""
        c = Constants()
        for side, key in (("src", "SRC"), ("tgt", "TGT")):
            d = dicts.get(side) if isinstance(dicts, dict) else None
            if d is None or not hasattr(d, "lookup"):
                continue
            words = _SPECIAL_WORD_OPTIONS[side]
            for tok, default_word in (("pad", PAD_WORD), ("unk", UNK_WORD), ("bos", BOS_WORD), ("eos", EOS_WORD)):
                word = getattr(opt, words[tok], default_word)
                idx = d.lookup(word)
                if idx is not None:
                    setattr(c, "%s_%s" % (key, tok.upper()), idx)
        c.PAD, c.UNK, c.BOS, c.EOS = c.TGT_PAD, c.TGT_UNK, c.TGT_BOS, c.TGT_EOS
        c.checkpointing = getattr(opt, "checkpointing", 0)
        c.max_position_length = getattr(opt, "max_position_length", 8192)
        return c


default = Constants()
