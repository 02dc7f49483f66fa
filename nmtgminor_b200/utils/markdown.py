"""``-md`` on any of the command-line tools prints its options as Markdown (for the documentation pages).

Reference: onmt/markdown.py:7-58 (``MarkdownHelpFormatter`` / ``MarkdownHelpAction``).
"""
from __future__ import annotations

import argparse


class MarkdownHelpFormatter(argparse.HelpFormatter):
    """Sections become ``###`` headings, every option a bold bullet with its default and help text."""

    def _format_usage(self, usage, actions, groups, prefix):
        return "# %s\n\n%s\n\n" % (self._prog, self._root_section.heading or "")

    def format_help(self):
        return self._root_section.format_help()

    def start_section(self, heading):
        super().start_section("### **%s**" % heading)

    def _format_action(self, action):
        if not action.option_strings or action.dest in ("help", "md"):
            return ""
        lines = ["* **%s" % ", ".join(action.option_strings)]
        if action.metavar or action.nargs != 0:
            lines[-1] += " %s" % (action.metavar or action.dest.upper())
        lines[-1] += "**"
        if action.default not in (None, argparse.SUPPRESS):
            lines[-1] += " [%s]" % (action.default,)
        if action.choices:
            lines[-1] += " (one of: %s)" % ", ".join(str(c) for c in action.choices)
        if action.help:
            lines.append("  " + self._expand_help(action))
        return "\n".join(lines) + "\n\n"


class MarkdownHelpAction(argparse.Action):
    def __init__(self, option_strings, dest=argparse.SUPPRESS, default=argparse.SUPPRESS, **kwargs):
        super().__init__(option_strings=option_strings, dest=dest, default=default, nargs=0, **kwargs)

    def __call__(self, parser, namespace, values, option_string=None):
        parser.formatter_class = MarkdownHelpFormatter
        parser.print_help()
        parser.exit()


def add_md_help_argument(parser: argparse.ArgumentParser) -> None:
    parser.add_argument("-md", action=MarkdownHelpAction, help="print the options as Markdown and exit")
