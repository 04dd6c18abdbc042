"""Recipe files: a deliberately small YAML subset flattened to dotted keys.

Accepts exactly what the reference's recipe parser accepts (core/config.cpp:40-161 in the
reference tree): space-indented nested maps, ``key: value`` scalars (optionally quoted), inline
``[a, b]`` lists and ``- item`` lists (stored joined by newlines), ``#`` comments outside quotes
(only when at line start or preceded by white space).  Tabs for indentation, anchors, aliases, tags,
block scalars, merge keys and duplicate keys are errors.  Getters come in a lenient flavour (warn and
fall back to the default on a malformed value) and a strict one (raise) (core/config.cpp:210-327).
"""
from __future__ import annotations

import math
import re
from typing import Dict, Iterable, List, Optional

from .log import log_warn


class ConfigError(ValueError):
    pass


_BLOCK_MARKERS = {"|", ">", "|-", ">-"}
_BLOCK_VALUES = {"|", ">", "|-", ">-", "|+", ">+"}
_TRUE = {"true", "yes", "on", "1"}
_FALSE = {"false", "no", "off", "0"}
_WS = " \t\r\n"
_INT_RE = re.compile(r"^[ \t\n\v\f\r]*[+-]?\d+$")


def _unquote(s: str) -> str:
    if len(s) >= 2 and s[0] == s[-1] and s[0] in "\"'":
        return s[1:-1]
    return s


def _scan_outside_quotes(text: str, want: str, comment_rule: bool = False) -> int:
    """Index of the first ``want`` char outside quotes (-1 if none)."""
    single = double = False
    for i, ch in enumerate(text):
        if ch == "'" and not double:
            single = not single
        elif ch == '"' and not single:
            double = not double
        elif ch == want and not single and not double:
            if not comment_rule or i == 0 or text[i - 1] in " \t":
                return i
    return -1


def _parse_int(text: str) -> Optional[int]:
    t = text.strip(_WS)
    if not _INT_RE.match(t):
        return None
    v = int(t)
    if not (-(2 ** 63) <= v < 2 ** 63):
        return None
    return v


def _parse_float(text: str) -> Optional[float]:
    t = text.strip(_WS)
    if not t or "_" in t:
        return None
    try:
        v = float.fromhex(t) if re.match(r"^[+-]?0[xX]", t) else float(t)
    except ValueError:
        return None
    if not math.isfinite(v):
        return None
    return v


class Config:
    """Flat ``dotted.key -> string`` view of a recipe."""

    def __init__(self, kv: Optional[Dict[str, str]] = None):
        self.kv: Dict[str, str] = dict(kv or {})

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_string(cls, text: str) -> "Config":
        kv: Dict[str, str] = {}
        parents: List[tuple] = []          # (indent, key)
        open_list: Optional[str] = None    # key that "- item" lines append to
        open_list_indent = -1
        for lineno, line in enumerate(text.split("\n"), 1):
            cut = _scan_outside_quotes(line, "#", comment_rule=True)
            raw = line if cut < 0 else line[:cut]
            body = raw.strip(_WS)
            if not body:
                continue
            indent = len(raw) - len(raw.lstrip(" "))
            if indent < len(raw) and raw[indent] == "\t":
                raise ConfigError(f"config:{lineno}: tab indentation is not allowed (use spaces): {body}")
            if body[0] in "&*!" or body in _BLOCK_MARKERS:
                raise ConfigError(f"config:{lineno}: unsupported YAML construct (anchors/aliases/tags/blocks): {body}")
            if body.startswith("<<:"):
                raise ConfigError(f"config:{lineno}: unsupported YAML merge key '<<:': {body}")
            if body.startswith("- ") or body == "-":
                if not open_list:
                    raise ConfigError(f"config:{lineno}: orphan list item with no parent key: {body}")
                if indent < open_list_indent:
                    raise ConfigError(f"config:{lineno}: list item dedented outside '{open_list}': {body}")
                item = _unquote(body[1:].strip(_WS))
                prev = kv.get(open_list, "")
                kv[open_list] = item if not prev else prev + "\n" + item
                continue
            while parents and parents[-1][0] >= indent:
                parents.pop()
            colon = _scan_outside_quotes(body, ":")
            if colon < 0:
                raise ConfigError(f"config:{lineno}: missing ':' (want 'key: value'): {body}")
            key = body[:colon].strip(_WS)
            val = body[colon + 1:].strip(_WS)
            if not key:
                raise ConfigError(f"config:{lineno}: empty key (want 'key: value')")
            if val in _BLOCK_VALUES:
                raise ConfigError(f"config:{lineno}: unsupported block scalar '{val}' for key '{key}'")
            if val and val[0] in "&*!":
                raise ConfigError(f"config:{lineno}: unsupported YAML construct in value for key '{key}': {val}")
            full = ".".join([p[1] for p in parents] + [key])
            if full in kv:
                raise ConfigError(f"config:{lineno}: duplicate key '{full}'")
            if not val:
                parents.append((indent, key))
                open_list, open_list_indent = full, indent
                kv[full] = ""
            elif val[0] == "[" and val[-1] == "]":
                items = [_unquote(it.strip(_WS)) for it in val[1:-1].split(",")]
                kv[full] = "\n".join(it for it in items if it)
                open_list = None
            else:
                kv[full] = _unquote(val)
                open_list = None
        return cls(kv)

    @classmethod
    def from_file(cls, path: str) -> "Config":
        try:
            with open(path, "rb") as f:
                data = f.read()
        except OSError as e:
            raise ConfigError(f"cannot open config file: {path}") from e
        return cls.from_string(data.decode("utf-8", errors="surrogateescape"))

    # ------------------------------------------------------------------ lenient getters
    def has(self, key: str) -> bool:
        return key in self.kv

    def _raw(self, key: str) -> Optional[str]:
        v = self.kv.get(key)
        return v if v else None

    def get_str(self, key: str, default: str = "") -> str:
        v = self._raw(key)
        return default if v is None else v

    def get_int(self, key: str, default: int = 0) -> int:
        v = self._raw(key)
        if v is None:
            return default
        out = _parse_int(v)
        if out is None:
            log_warn(f"config: ignoring malformed int for '{key}': '{v}'")
            return default
        return out

    def get_float(self, key: str, default: float = 0.0) -> float:
        v = self._raw(key)
        if v is None:
            return default
        out = _parse_float(v)
        if out is None:
            log_warn(f"config: ignoring malformed number for '{key}': '{v}'")
            return default
        return out

    def get_bool(self, key: str, default: bool = False) -> bool:
        v = self._raw(key)
        if v is None:
            return default
        low = v.lower()
        if low in _TRUE:
            return True
        if low in _FALSE:
            return False
        log_warn(f"config: ignoring malformed bool for '{key}': '{v}'")
        return default

    def get_list(self, key: str) -> List[str]:
        v = self._raw(key)
        return [] if v is None else [it for it in v.split("\n") if it]

    # ------------------------------------------------------------------ strict getters
    def get_int_strict(self, key: str) -> int:
        v = self._raw(key)
        if v is None:
            raise ConfigError(f"config: missing required int '{key}'")
        out = _parse_int(v)
        if out is None:
            raise ConfigError(f"config: malformed int for '{key}': '{v}' (refusing silent default)")
        return out

    def get_float_strict(self, key: str) -> float:
        v = self._raw(key)
        if v is None:
            raise ConfigError(f"config: missing required number '{key}'")
        out = _parse_float(v)
        if out is None:
            raise ConfigError(f"config: malformed number for '{key}': '{v}' (refusing silent default)")
        return out

    def get_bool_strict(self, key: str) -> bool:
        v = self._raw(key)
        if v is None:
            raise ConfigError(f"config: missing required bool '{key}'")
        low = v.lower()
        if low in _TRUE:
            return True
        if low in _FALSE:
            return False
        raise ConfigError(f"config: malformed bool for '{key}': '{v}' (refusing silent default)")

    def set(self, key: str, value) -> None:
        self.kv[key] = str(value)

    # ------------------------------------------------------------------ typo gate
    def check_known(self, exact: Iterable[str], prefixes: Iterable[str] = (), strict: bool = False) -> int:
        """Count (warn about, or with ``strict`` raise on) keys outside the allow-list.

        A valueless key that only opens a nested map is fine; a valueless leaf is reported as a typo.
        """
        exact = set(exact)
        prefixes = tuple(prefixes)
        unknown = 0
        for k, v in sorted(self.kv.items()):
            if k in exact or any(k.startswith(p) for p in prefixes):
                continue
            if not v:
                pre = k + "."
                if any(k2.startswith(pre) and len(k2) > len(pre) for k2 in self.kv):
                    continue
                if strict:
                    raise ConfigError(f"config: '{k}' has no value (typo?)")
                log_warn(f"[cfg ] '{k}' has no value and does nothing (typo?)")
            else:
                if strict:
                    raise ConfigError(f"config: unknown key '{k}' (typo?)")
                log_warn(f"[cfg ] unknown key '{k}' is ignored (typo? use --strict-config to fail)")
            unknown += 1
        return unknown

    def dump(self) -> str:
        return "".join(f"{k} = {v.replace(chr(10), '|')}\n" for k, v in sorted(self.kv.items()))
