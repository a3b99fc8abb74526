"""A small YAML reader with the scalar rules of the reference's hand-written parser
(src/util/yaml.zig:200-551): indentation-nested maps, ``-`` lists, quoted strings,
``#`` comments, ``null``/``~``, booleans ``true/True/yes`` and ``false/False/no``,
decimal and hex integers, floats only when the token has a ``.`` or an exponent, and a
tab counting as two spaces (yaml.zig:541-543).  Anything else is a string.
"""
from __future__ import annotations

import re
from typing import Any

_INT = re.compile(r"^[+-]?\d+$")
_HEX = re.compile(r"^[+-]?0[xX][0-9a-fA-F]+$")
_FLOAT = re.compile(r"^[+-]?(\d+\.\d*|\.\d+|\d+)([eE][+-]?\d+)?$")


class YamlError(ValueError):
    pass


def parse_scalar(tok: str) -> Any:
    t = tok.strip()
    if len(t) >= 2 and t[0] == t[-1] and t[0] in "\"'":
        body = t[1:-1]
        if t[0] == '"':
            body = body.replace("\\n", "\n").replace("\\t", "\t").replace('\\"', '"') \
                       .replace("\\\\", "\\")
        return body
    if t in ("", "null", "~", "Null", "NULL"):
        return None
    if t in ("true", "True", "yes", "TRUE"):
        return True
    if t in ("false", "False", "no", "FALSE"):
        return False
    if _INT.match(t):
        return int(t)
    if _HEX.match(t):
        return int(t, 16)
    if ("." in t or "e" in t or "E" in t) and _FLOAT.match(t):
        return float(t)
    return t


def _strip_comment(line: str) -> str:
    out, quote = [], None
    for i, ch in enumerate(line):
        if quote:
            if ch == quote and line[i - 1] != "\\":
                quote = None
        elif ch in "\"'":
            quote = ch
        elif ch == "#" and (i == 0 or line[i - 1] in " \t"):
            break
        out.append(ch)
    return "".join(out).rstrip()


def _lines(text: str):
    for raw in text.splitlines():
        raw = raw.replace("\t", "  ")
        s = _strip_comment(raw)
        if not s.strip() or s.strip() in ("---", "..."):
            continue
        yield len(s) - len(s.lstrip(" ")), s.strip()


def _split_key(s: str):
    quote = None
    for i, ch in enumerate(s):
        if quote:
            if ch == quote:
                quote = None
        elif ch in "\"'":
            quote = ch
        elif ch == ":" and (i + 1 == len(s) or s[i + 1] == " "):
            key = s[:i].strip()
            if len(key) >= 2 and key[0] == key[-1] and key[0] in "\"'":
                key = key[1:-1]
            return key, s[i + 1:].strip()
    return None, s


def _parse_inline(s: str) -> Any:
    s = s.strip()
    if s.startswith("[") and s.endswith("]"):
        inner = s[1:-1].strip()
        return [parse_scalar(x) for x in _split_commas(inner)] if inner else []
    if s.startswith("{") and s.endswith("}"):
        out = {}
        inner = s[1:-1].strip()
        for part in _split_commas(inner) if inner else []:
            k, v = _split_key(part.strip())
            if k is None:
                raise YamlError(f"bad inline map entry: {part!r}")
            out[k] = parse_scalar(v)
        return out
    return parse_scalar(s)


def _split_commas(s: str):
    parts, cur, quote, depth = [], [], None, 0
    for ch in s:
        if quote:
            if ch == quote:
                quote = None
        elif ch in "\"'":
            quote = ch
        elif ch in "[{":
            depth += 1
        elif ch in "]}":
            depth -= 1
        elif ch == "," and depth == 0:
            parts.append("".join(cur).strip())
            cur = []
            continue
        cur.append(ch)
    if cur:
        parts.append("".join(cur).strip())
    return parts


def _parse_block(items, pos: int, indent: int):
    """Parse the block starting at items[pos] whose lines all have indentation >= indent."""
    if pos >= len(items):
        return None, pos
    first_indent, first = items[pos]
    if first.startswith("- ") or first == "-":
        out = []
        while pos < len(items) and items[pos][0] == first_indent and \
                (items[pos][1].startswith("- ") or items[pos][1] == "-"):
            body = items[pos][1][1:].strip()
            if not body:
                val, pos = _parse_block(items, pos + 1, first_indent + 1)
                out.append(val)
                continue
            k, v = _split_key(body)
            if k is not None and not body.startswith(("[", "{", '"', "'")):
                # a map that starts on the dash line; its other keys sit two columns in
                sub = [(first_indent + 2, body)]
                pos += 1
                while pos < len(items) and items[pos][0] > first_indent:
                    sub.append(items[pos])
                    pos += 1
                val, _ = _parse_block(sub, 0, first_indent + 2)
                out.append(val)
            else:
                out.append(_parse_inline(body))
                pos += 1
        return out, pos
    out = {}
    while pos < len(items) and items[pos][0] == first_indent:
        k, v = _split_key(items[pos][1])
        if k is None:
            raise YamlError(f"expected 'key: value', got {items[pos][1]!r}")
        if v == "":
            if pos + 1 < len(items) and items[pos + 1][0] > first_indent:
                val, pos = _parse_block(items, pos + 1, items[pos + 1][0])
            elif pos + 1 < len(items) and items[pos + 1][0] == first_indent and \
                    items[pos + 1][1].startswith("-"):
                val, pos = _parse_block(items, pos + 1, first_indent)
            else:
                val, pos = None, pos + 1
            out[k] = val
        else:
            out[k] = _parse_inline(v)
            pos += 1
    if pos < len(items) and items[pos][0] > first_indent:
        raise YamlError(f"unexpected indentation at {items[pos][1]!r}")
    return out, pos


def loads(text: str) -> Any:
    items = list(_lines(text))
    if not items:
        return {}
    val, pos = _parse_block(items, 0, items[0][0])
    if pos != len(items):
        raise YamlError(f"could not parse line {items[pos][1]!r}")
    return val


def load(path) -> Any:
    with open(path, "r", encoding="utf-8") as f:
        return loads(f.read())


def dumps(obj: Any, indent: int = 0) -> str:
    """Writes maps / lists / scalars back in the subset ``loads`` reads."""
    pad = " " * indent
    if isinstance(obj, dict):
        lines = []
        for k, v in obj.items():
            if isinstance(v, (dict, list)) and v:
                lines.append(f"{pad}{k}:")
                lines.append(dumps(v, indent + 2))
            else:
                lines.append(f"{pad}{k}: {_scalar_str(v)}")
        return "\n".join(lines)
    if isinstance(obj, list):
        lines = []
        for v in obj:
            if isinstance(v, dict) and v:
                body = dumps(v, indent + 2).split("\n")
                lines.append(f"{pad}- {body[0].lstrip()}")
                lines.extend(body[1:])
            else:
                lines.append(f"{pad}- {_scalar_str(v)}")
        return "\n".join(lines)
    return pad + _scalar_str(obj)


def _scalar_str(v: Any) -> str:
    if v is None:
        return "null"
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, float):
        r = repr(v)
        return r if ("." in r or "e" in r) else r + ".0"
    if isinstance(v, (dict, list)):
        return "{}" if isinstance(v, dict) else "[]"
    s = str(v)
    if isinstance(v, str) and (s == "" or parse_scalar(s) != s or ":" in s or "#" in s):
        return '"' + s.replace("\\", "\\\\").replace('"', '\\"') + '"'
    return s
