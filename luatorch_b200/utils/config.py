"""Key/value configuration (lua/luatorch/utils/config.lua): defaults table, `load(path)`
overrides, `get(key, default)`, `set`, sorted `print`.

The reference executes the config file as Lua code.  Here `load` accepts JSON, or a
restricted Lua-table file of the form `return { key = value, ... }` (numbers, strings,
booleans, nil, `--` comments) parsed WITHOUT executing anything."""
from __future__ import annotations

import json
import os
import re


def parse_lua_table(text: str) -> dict:
    text = re.sub(r"--\[\[.*?\]\]", "", text, flags=re.S)
    text = re.sub(r"--[^\n]*", "", text)
    m = re.search(r"return\s*\{(.*)\}\s*$", text.strip(), flags=re.S)
    if not m:
        raise ValueError("config: file must return a table")
    body = m.group(1)
    out = {}
    token = re.compile(
        r"""\s*(?:\[\s*["']([^"']+)["']\s*\]|([A-Za-z_][A-Za-z0-9_]*))\s*=\s*
            (?:"((?:[^"\\]|\\.)*)"|'((?:[^'\\]|\\.)*)'|([-+]?(?:0x[0-9a-fA-F]+|\d+\.?\d*(?:[eE][-+]?\d+)?|\.\d+(?:[eE][-+]?\d+)?))|(true|false|nil))
            \s*[,;]?""", re.X)
    pos = 0
    while pos < len(body):
        if body[pos:].strip() == "":
            break
        mm = token.match(body, pos)
        if not mm:
            raise ValueError("config: cannot parse near %r" % body[pos:pos + 40].strip())
        key = mm.group(1) or mm.group(2)
        if mm.group(3) is not None or mm.group(4) is not None:
            val = mm.group(3) if mm.group(3) is not None else mm.group(4)
        elif mm.group(5) is not None:
            s = mm.group(5)
            val = int(s, 16) if s.lower().startswith("0x") else (int(s) if re.fullmatch(r"[-+]?\d+", s) else float(s))
        else:
            val = {"true": True, "false": False, "nil": None}[mm.group(6)]
        if val is not None:
            out[key] = val
        pos = mm.end()
    return out


class Config:
    def __init__(self, defaults=None):
        self.values = dict(defaults or {})

    @classmethod
    def new(cls, defaults=None):
        return cls(defaults)

    def load(self, path: str):
        if not os.path.exists(path):
            print("config: using defaults, no config file at " + path)
            return self
        with open(path) as f:
            text = f.read()
        try:
            overrides = json.loads(text)
        except json.JSONDecodeError:
            overrides = parse_lua_table(text)
        if not isinstance(overrides, dict):
            raise ValueError("config: file must return a table")
        self.values.update(overrides)
        return self

    def update(self, overrides: dict):
        self.values.update(overrides)
        return self

    def get(self, key, default=None):
        v = self.values.get(key)
        return default if v is None else v

    def set(self, key, value):
        self.values[key] = value

    def print(self):
        print("config:")
        for k in sorted(self.values):
            print("  %-20s = %s" % (k, self.values[k]))

    def __repr__(self):
        return "Config(%d values)" % len(self.values)
