"""Argument cursor used by the CLI (reference: src/util/cli.zig:4-87): ``next``, ``peek``,
``expect_string / expect_int / expect_float``, ``parse_flag``, ``parse_option`` and
``parse_key_value("a=b,c=d")``."""
from __future__ import annotations


class CliError(ValueError):
    pass


class ArgParser:
    def __init__(self, argv):
        self.argv = list(argv)
        self.pos = 0

    def next(self):
        if self.pos >= len(self.argv):
            return None
        a = self.argv[self.pos]
        self.pos += 1
        return a

    def peek(self):
        return self.argv[self.pos] if self.pos < len(self.argv) else None

    def expect_string(self, what: str = "value") -> str:
        a = self.next()
        if a is None:
            raise CliError(f"missing value for {what}")
        return a

    def expect_int(self, what: str = "value") -> int:
        a = self.expect_string(what)
        try:
            return int(a, 0)
        except ValueError:
            raise CliError(f"{what}: expected an integer, got {a!r}") from None

    def expect_float(self, what: str = "value") -> float:
        a = self.expect_string(what)
        try:
            return float(a)
        except ValueError:
            raise CliError(f"{what}: expected a number, got {a!r}") from None

    def parse_flag(self, name: str) -> bool:
        """Consumes ``name`` if it is the next argument."""
        if self.peek() == name:
            self.pos += 1
            return True
        return False

    def parse_option(self, name: str):
        """Consumes ``name VALUE`` or ``name=VALUE`` if next; returns the value or None."""
        a = self.peek()
        if a is None:
            return None
        if a == name:
            self.pos += 1
            return self.expect_string(name)
        if a.startswith(name + "="):
            self.pos += 1
            return a[len(name) + 1:]
        return None


def parse_key_value(text: str) -> dict:
    out = {}
    for part in text.split(","):
        part = part.strip()
        if not part:
            continue
        if "=" not in part:
            raise CliError(f"expected key=value, got {part!r}")
        k, v = part.split("=", 1)
        out[k.strip()] = v.strip()
    return out
