"""Every training flag either has a consumer in the code, is accepted with a stated reason, or is refused.

A flag that parses and does nothing lets a command line of the reference "work" while training a different model, so the
option table is checked against the sources: for every flag of the training parser, some file other than the option
tables must read it (``opt.<name>`` or the quoted name), or it must be listed in ``ALWAYS_ON_FLAGS`` (the fused path it
would switch on is the only path), ``NO_EFFECT_IN_REFERENCE`` (the reference never reads it either) or
``UNSUPPORTED_FLAGS`` (``build_model`` raises when it is set)."""
import os
import re

import pytest

from nmtgminor_b200.options import (ALWAYS_ON_FLAGS, EXTRA_TRAIN_FLAGS, NO_EFFECT_IN_REFERENCE, UNSUPPORTED_FLAGS, default_options,
                                    unsupported_flags_in, validate_model_options)
from nmtgminor_b200.options_spec import TRAIN_FLAGS

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _sources():
    out = []
    with open(os.path.join(ROOT, ".gitignore")) as fh:       # scratch and build folders are not sources
        ignored = {line.strip().strip("/") for line in fh if line.strip() and not line.startswith("#")}
    skip = ignored | {"baseline", ".git", "tests", "__pycache__", "profiles"}
    for base, dirs, files in os.walk(ROOT):
        dirs[:] = [d for d in dirs if d not in skip]
        for f in files:
            if f.endswith(".py") and f not in ("options_spec.py", "options.py"):
                with open(os.path.join(base, f)) as fh:
                    out.append(fh.read())
    # options.py minus its status tables (backward_compatible and the parsers do consume flags)
    with open(os.path.join(ROOT, "nmtgminor_b200", "options.py")) as fh:
        text = fh.read()
    out.append(text.split("# what every training flag does here")[0])
    return "\n".join(out)


def test_every_training_flag_is_consumed_accepted_or_refused():
    blob = _sources()
    orphans = []
    for row in list(TRAIN_FLAGS) + list(EXTRA_TRAIN_FLAGS):
        name = row[0]
        if name in ALWAYS_ON_FLAGS or name in NO_EFFECT_IN_REFERENCE or name in UNSUPPORTED_FLAGS:
            continue
        if not re.search(r"(\.%s\b|[\"']%s[\"'])" % (re.escape(name), re.escape(name)), blob):
            orphans.append(name)
    assert not orphans, "flags without a consumer, a reason or a refusal: %s" % orphans


def test_status_tables_name_real_flags_and_do_not_overlap():
    names = {row[0] for row in list(TRAIN_FLAGS) + list(EXTRA_TRAIN_FLAGS)}
    for table in (ALWAYS_ON_FLAGS, NO_EFFECT_IN_REFERENCE, UNSUPPORTED_FLAGS):
        assert set(table) <= names, sorted(set(table) - names)
    assert not (set(ALWAYS_ON_FLAGS) & set(UNSUPPORTED_FLAGS))
    assert not (set(NO_EFFECT_IN_REFERENCE) & set(UNSUPPORTED_FLAGS))


def test_an_unsupported_flag_stops_the_run_and_defaults_do_not():
    opt = default_options([])
    assert unsupported_flags_in(opt) == []
    validate_model_options(opt)
    opt = default_options(["-weight_norm"])
    assert [b[0] for b in unsupported_flags_in(opt)] == ["weight_norm"]
    with pytest.raises(NotImplementedError, match="weight_norm"):
        validate_model_options(opt)
    opt = default_options(["-transducer_loss", "0.5"])
    with pytest.raises(NotImplementedError, match="transducer_loss"):
        from nmtgminor_b200.data.synthetic import synthetic_dict
        from nmtgminor_b200.models.factory import build_model
        d = synthetic_dict(50)
        build_model(opt, {"src": d, "tgt": d})
