"""Test-case specifications: the ``key: value; key: value`` tests-file grammar
and ``task.yml`` loading.

The grammar is the reference's (``eval.py:60-93``) with one fix: ``True`` /
``False`` become booleans instead of staying (truthy) strings, so
``has_bias: False`` really disables the bias.  Seeds are mixed with the secret
seed by the same Cantor pairing (``eval.py:49-57``).
"""
from __future__ import annotations

import dataclasses
import re
from pathlib import Path
from typing import Any, Dict, List, Optional

import yaml


@dataclasses.dataclass
class TestCase:
    __test__ = False  # not a pytest class, whatever its name

    args: Dict[str, Any]
    spec: str


class SpecError(ValueError):
    pass


_PART = re.compile(r"\s*([a-zA-Z_]+)\s*:\s*([a-zA-Z_][a-zA-Z_0-9]*|[+-]?[0-9]+)\s*")


def combine_seeds(a: int, b: int) -> int:
    """Cantor pairing: a public per-case seed and a secret seed give a seed that
    is large whenever the secret one is."""
    return int(a + (a + b) * (a + b + 1) // 2)


def parse_value(text: str) -> Any:
    if re.fullmatch(r"[+-]?[0-9]+", text):
        return int(text)
    if text == "True":
        return True
    if text == "False":
        return False
    return text


def parse_line(line: str) -> TestCase:
    args: Dict[str, Any] = {}
    for part in line.split(";"):
        m = _PART.fullmatch(part)
        if m is None:
            raise SpecError(f"invalid test case: '{line}': '{part}'")
        args[m.group(1)] = parse_value(m.group(2))
    return TestCase(args=args, spec=line)


def mix_seed(cases: List[TestCase], seed: Optional[int]) -> List[TestCase]:
    if seed is not None:
        for case in cases:
            if "seed" in case.args:
                case.args["seed"] = combine_seeds(case.args["seed"], seed)
    return cases


def parse_tests(text: str, seed: Optional[int] = None) -> List[TestCase]:
    cases = [parse_line(line) for line in text.splitlines() if line.strip()]
    return mix_seed(cases, seed)


def format_spec(args: Dict[str, Any]) -> str:
    return "; ".join(f"{k}: {v}" for k, v in args.items())


def load_task_yaml(path) -> Dict[str, Any]:
    doc = yaml.safe_load(Path(path).read_text())
    if not isinstance(doc, dict):
        raise SpecError(f"{path}: not a mapping")
    return doc


def cases_from_yaml(path, section: str = "tests", seed: Optional[int] = None) -> List[TestCase]:
    doc = load_task_yaml(path)
    if section not in doc:
        raise SpecError(f"{path}: no '{section}' list")
    cases = [TestCase(args=dict(item), spec=format_spec(item)) for item in doc[section]]
    return mix_seed(cases, seed)


def write_tests_file(path, cases: List[Dict[str, Any]]) -> None:
    Path(path).write_text("\n".join(format_spec(c) for c in cases) + "\n")
