"""JSON-with-comments reader. String aware: `//` and `/* */` inside string literals
(URLs, shell commands) are kept. Accepts everything the reference's regex stripper
accepts (scripts/build_script.sh:48-54: line comments, block comments, trailing
commas), without its flaw of eating `//` inside strings."""
from __future__ import annotations

import json


def strip(text: str) -> str:
    out = []
    i, n = 0, len(text)
    in_str = False
    while i < n:
        c = text[i]
        if in_str:
            out.append(c)
            if c == "\\" and i + 1 < n:
                out.append(text[i + 1])
                i += 2
                continue
            if c == '"':
                in_str = False
            i += 1
            continue
        if c == '"':
            in_str = True
            out.append(c)
            i += 1
        elif c == "/" and i + 1 < n and text[i + 1] == "/":
            while i < n and text[i] != "\n":
                i += 1
        elif c == "/" and i + 1 < n and text[i + 1] == "*":
            j = text.find("*/", i + 2)
            if j < 0:
                raise ValueError("unterminated block comment")
            out.append(" " * 0 + "\n" * text.count("\n", i, j + 2))  # keep line numbers for error messages
            i = j + 2
        else:
            out.append(c)
            i += 1
    s = "".join(out)
    # trailing commas: a comma followed only by whitespace and then } or ], outside strings
    res = []
    i, n = 0, len(s)
    in_str = False
    while i < n:
        c = s[i]
        if in_str:
            res.append(c)
            if c == "\\" and i + 1 < n:
                res.append(s[i + 1])
                i += 2
                continue
            if c == '"':
                in_str = False
        elif c == '"':
            in_str = True
            res.append(c)
        elif c == ",":
            j = i + 1
            while j < n and s[j] in " \t\r\n":
                j += 1
            if j < n and s[j] in "}]":
                i += 1
                continue
            res.append(c)
        else:
            res.append(c)
        i += 1
    return "".join(res)


def loads(text: str):
    return json.loads(strip(text))


def load(path):
    with open(path) as f:
        return loads(f.read())
