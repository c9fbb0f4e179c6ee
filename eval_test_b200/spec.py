"""Parser for the harness's shape-list files (``tests.txt`` / ``benchmarks.txt``).

Same grammar as the reference's ``get_test_cases`` (eval/common/eval_base.py:62-109): one case per line,
``key: value`` pairs separated by ``;``, values are ints, bare identifiers, or ``[...]`` / ``(...)`` literals;
an optional global seed is mixed into every ``seed`` with the pairing of ``_combine`` (eval_base.py:58-59).
Malformed input raises ``ValueError`` where the reference exits with status 113.
"""
from __future__ import annotations

import ast
import re
from dataclasses import dataclass

_IDENT = re.compile(r"[a-zA-Z_]+")


@dataclass
class TestCase:
    args: dict
    spec: str
    __test__ = False  # not a pytest class


def combine(a: int, b: int) -> int:
    return int(a + (a + b) * (a + b + 1) // 2)


def parse_line(line: str) -> dict:
    case = {}
    for part in line.split(";"):
        if not part.strip():
            continue
        key, sep, raw = part.partition(":")
        key, raw = key.strip(), raw.strip()
        if not sep or not key or not raw or not _IDENT.fullmatch(key):
            raise ValueError(f"invalid test case: '{line}': '{part}'")
        if raw[0] in "[(" and raw[-1] in "])":
            try:
                val = ast.literal_eval(raw)
            except (SyntaxError, ValueError):
                raise ValueError(f"invalid test case: '{line}': '{part}'") from None
        else:
            try:
                val = int(raw)
            except ValueError:
                if not _IDENT.fullmatch(raw):
                    raise ValueError(f"invalid test case: '{line}': '{part}'") from None
                val = raw
        case[key] = val
    return case


def parse_cases(text: str, seed: int | None = None) -> list[TestCase]:
    cases = [TestCase(args=parse_line(line), spec=line) for line in text.splitlines()]
    if seed is not None:
        for c in cases:
            if "seed" in c.args:
                c.args["seed"] = combine(c.args["seed"], seed)
    return cases
