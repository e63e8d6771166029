"""Reads kernel signatures out of MLIR text: ``func.func`` arguments and results that carry a
``vernon.semantic`` attribute, as in the reference's only Vernon input file
(source/tests/integration/color.mlir:4-9,43-45), and maps each to the runtime's argument class.

The reference pass walks the same attributes and only prints them
(source/lib/Dialect/Vernon/Transforms/VernonToSpirv.cpp:36-58; `varying` falls through its
if-chain unhandled).  Here every name of the vocabulary, `varying` included, resolves through
``vrhi_arg_class_from_semantic``; an unknown name is an error, not a silent default.
Pure text processing: no MLIR installation is involved.
"""
from __future__ import annotations

import ctypes as C
import re
from dataclasses import dataclass
from typing import List, Optional, Tuple

from . import _lib as L


@dataclass(frozen=True)
class Param:
    name: Optional[str]      # "%pos" for arguments, None for results
    type: str                # e.g. "tensor<4x4xf32>"
    semantic: Optional[str]  # the vernon.semantic string, or None if the attribute is absent
    arg_class: Optional[int]  # vrhi_arg_class, None without a semantic

    @property
    def shape(self) -> Tuple[int, ...]:
        m = re.fullmatch(r"tensor<((?:\d+x)*)(\w+)>", self.type.replace(" ", ""))
        if not m:
            return ()
        return tuple(int(d) for d in m.group(1).split("x") if d)

    @property
    def n_elements(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n


@dataclass(frozen=True)
class Signature:
    name: str
    args: Tuple[Param, ...]
    results: Tuple[Param, ...]


def semantic_to_class(semantic: str) -> int:
    v = C.c_int()
    L.check(L.lib().vrhi_arg_class_from_semantic(semantic.encode(), C.byref(v)))
    return v.value


def _split_top_level(text: str) -> List[str]:
    parts, depth, cur = [], 0, []
    for ch in text:
        if ch in "<({[":
            depth += 1
        elif ch in ">)}]":
            depth -= 1
        if ch == "," and depth == 0:
            parts.append("".join(cur))
            cur = []
        else:
            cur.append(ch)
    if "".join(cur).strip():
        parts.append("".join(cur))
    return [p.strip() for p in parts]


_SEM = re.compile(r"vernon\.semantic\s*=\s*\"([^\"]*)\"")


def _param(text: str, is_arg: bool) -> Param:
    name = None
    if is_arg:
        m = re.match(r"(%[\w.$-]+)\s*:\s*", text)
        if not m:
            raise ValueError(f"cannot read argument {text!r}")
        name, text = m.group(1), text[m.end():]
    attr = ""
    brace = text.find("{")
    if brace >= 0:
        attr, text = text[brace:], text[:brace]
    sem = _SEM.search(attr)
    semantic = sem.group(1) if sem else None
    return Param(name, text.strip(), semantic, semantic_to_class(semantic) if semantic is not None else None)


def _matching(text: str, start: int) -> int:
    """Index just past the parenthesis that closes the one at text[start]."""
    depth = 0
    for k in range(start, len(text)):
        if text[k] == "(":
            depth += 1
        elif text[k] == ")":
            depth -= 1
            if depth == 0:
                return k + 1
    raise ValueError("unbalanced parentheses in a func.func signature")


def parse_signatures(mlir_text: str) -> List[Signature]:
    """All ``func.func @name(args) -> (results)`` signatures of a module, in order."""
    text = re.sub(r"//[^\n]*", "", mlir_text)
    out = []
    for m in re.finditer(r"func\.func\s+(?:private\s+|public\s+)?@([\w.$-]+)\s*\(", text):
        a0 = m.end() - 1
        a1 = _matching(text, a0)
        args = tuple(_param(p, True) for p in _split_top_level(text[a0 + 1:a1 - 1]))
        rest = text[a1:]
        results: Tuple[Param, ...] = ()
        r = re.match(r"\s*->\s*", rest)
        if r:
            rest = rest[r.end():]
            if rest.startswith("("):
                r1 = _matching(rest, 0)
                results = tuple(_param(p, False) for p in _split_top_level(rest[1:r1 - 1]))
            else:
                single = re.match(r"[^{\n]+", rest)  # result attributes require the parenthesised form
                results = (_param(single.group(0), False),)
        out.append(Signature(m.group(1), args, results))
    return out
