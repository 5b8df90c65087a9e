"""The options reference is generated from the parser; the committed file must be current and complete."""
import argparse
import os

from cuteafd_b200.cli import build_parser
from cuteafd_b200.utils.options_doc import render


def test_every_flag_has_help():
    ap = build_parser()
    subs = next(a for a in ap._actions if isinstance(a, argparse._SubParsersAction))
    bare = [(name, a.dest) for name, sp in [("", ap)] + list(subs.choices.items()) for a in sp._actions
            if not a.help and not isinstance(a, argparse._SubParsersAction)]
    assert bare == []


def test_committed_options_doc_is_current():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "docs", "options.md")
    with open(path) as f:
        assert f.read() == render(build_parser()), "run: python -m cuteafd_b200.utils.options_doc > docs/options.md"
