"""Constrained decoding: JSON grammar as an incremental byte-level state machine plus per-vocabulary
allow masks (core-llm/src/constraint.rs:19-186).

`JsonState` accepts exactly the prefixes of a single JSON value (RFC 8259, with surrounding whitespace).
`JsonConstraint` lifts it to token pieces: `allowed()` marks every vocabulary piece that keeps the text a
valid JSON prefix, `accept()` advances, `can_stop()` says the value is complete."""
from __future__ import annotations

import enum
from dataclasses import dataclass, field


class Constraint(enum.Enum):
    JSON = "json"


@dataclass
class ConstraintDecodeTable:
    """Decoded text piece of every token id; `special` ids are never allowed inside the constraint."""
    pieces: list[str]
    special: set[int] = field(default_factory=set)


_WS = " \t\n\r"
_HEX = "0123456789abcdefABCDEF"


class JsonState:
    """Pushdown recogniser over characters. `stack` holds containers ('{' or '['), `mode` the lexical state."""

    __slots__ = ("stack", "mode", "lit", "lit_pos", "hex_left", "done", "obj_state", "num")

    def __init__(self):
        self.stack: list[list] = []   # each entry: [kind, state] ; object states: key_or_end, key, colon, value, comma_or_end
        self.mode = "value"           # value | string | escape | hex | literal | number | after
        self.lit = ""
        self.lit_pos = 0
        self.hex_left = 0
        self.done = False
        self.num = ""                 # number sub-state: sign, zero, int, frac0, frac, exp0, expsign, exp
        self.obj_state = None

    @staticmethod
    def start() -> "JsonState":
        return JsonState()

    def clone(self) -> "JsonState":
        c = JsonState()
        c.stack = [list(e) for e in self.stack]
        c.mode, c.lit, c.lit_pos, c.hex_left, c.done, c.num = self.mode, self.lit, self.lit_pos, self.hex_left, \
            self.done, self.num
        return c

    # ---- helpers -------------------------------------------------------------------------------
    def _value_done(self) -> None:
        if not self.stack:
            self.done = True
            self.mode = "after"
            return
        top = self.stack[-1]
        if top[0] == "{":
            if top[1] == "key":
                top[1] = "colon"
            else:
                top[1] = "comma_or_end"
        else:
            top[1] = "comma_or_end"
        self.mode = "after"

    def _number_can_end(self) -> bool:
        return self.num in ("zero", "int", "frac", "exp")

    def _begin_value(self, ch: str) -> bool:
        if ch == "{":
            self.stack.append(["{", "key_or_end"])
            self.mode = "after"
            return True
        if ch == "[":
            self.stack.append(["[", "value_or_end"])
            self.mode = "after"
            return True
        if ch == '"':
            self.mode = "string"
            return True
        if ch in "tfn":
            self.lit = {"t": "true", "f": "false", "n": "null"}[ch]
            self.lit_pos = 1
            self.mode = "literal"
            return True
        if ch == "-":
            self.mode, self.num = "number", "sign"
            return True
        if ch == "0":
            self.mode, self.num = "number", "zero"
            return True
        if ch in "123456789":
            self.mode, self.num = "number", "int"
            return True
        return False

    def advance(self, ch: str) -> bool:
        """Consume one character; returns False (state unspecified afterwards) if it is not a valid continuation."""
        m = self.mode
        if m == "string":
            if ch == '"':
                top = self.stack[-1] if self.stack else None
                if top is not None and top[0] == "{" and top[1] in ("key_or_end", "key"):
                    top[1] = "key"
                self._value_done()
                return True
            if ch == "\\":
                self.mode = "escape"
                return True
            return ord(ch) >= 0x20
        if m == "escape":
            if ch in '"\\/bfnrt':
                self.mode = "string"
                return True
            if ch == "u":
                self.mode, self.hex_left = "hex", 4
                return True
            return False
        if m == "hex":
            if ch in _HEX:
                self.hex_left -= 1
                if self.hex_left == 0:
                    self.mode = "string"
                return True
            return False
        if m == "literal":
            if self.lit_pos < len(self.lit) and ch == self.lit[self.lit_pos]:
                self.lit_pos += 1
                if self.lit_pos == len(self.lit):
                    self._value_done()
                return True
            return False
        if m == "number":
            n = self.num
            if ch in "0123456789":
                if n == "sign":
                    self.num = "zero" if ch == "0" else "int"
                elif n == "zero":
                    return False
                elif n in ("frac0", "frac"):
                    self.num = "frac"
                elif n in ("exp0", "expsign", "exp"):
                    self.num = "exp"
                return True
            if ch == "." and n in ("zero", "int"):
                self.num = "frac0"
                return True
            if ch in "eE" and n in ("zero", "int", "frac"):
                self.num = "exp0"
                return True
            if ch in "+-" and n == "exp0":
                self.num = "expsign"
                return True
            if not self._number_can_end():
                return False
            self._value_done()
            return self.advance(ch)   # the terminator belongs to the enclosing context
        if m == "value":
            if ch in _WS:
                return True
            return self._begin_value(ch)
        # m == "after": between tokens inside a container, or after the top-level value
        if ch in _WS:
            return True
        if not self.stack:
            return False
        top = self.stack[-1]
        kind, st = top
        if kind == "{":
            if st == "key_or_end":
                if ch == "}":
                    self.stack.pop()
                    self._value_done()
                    return True
                if ch == '"':
                    top[1] = "key"
                    self.mode = "string"
                    return True
                return False
            if st == "expect_key":
                if ch == '"':
                    top[1] = "key"
                    self.mode = "string"
                    return True
                return False
            if st == "colon":
                if ch == ":":
                    top[1] = "value"
                    self.mode = "value"
                    return True
                return False
            if st == "comma_or_end":
                if ch == ",":
                    top[1] = "expect_key"
                    return True
                if ch == "}":
                    self.stack.pop()
                    self._value_done()
                    return True
                return False
            return False
        # array
        if st == "value_or_end":
            if ch == "]":
                self.stack.pop()
                self._value_done()
                return True
            top[1] = "value"
            return self._begin_value(ch)
        if st == "comma_or_end":
            if ch == ",":
                top[1] = "value"
                self.mode = "value"
                return True
            if ch == "]":
                self.stack.pop()
                self._value_done()
                return True
            return False
        return False

    def advance_str(self, s: str) -> bool:
        for ch in s:
            if not self.advance(ch):
                return False
        return True

    def can_stop(self) -> bool:
        """True when the text so far is one complete JSON value (a top-level number may end here too)."""
        if self.done and not self.stack:
            return True
        return not self.stack and self.mode == "number" and self._number_can_end()


class JsonConstraint:
    def __init__(self, table: ConstraintDecodeTable):
        self.table = table
        self.state = JsonState.start()

    def allowed(self) -> list[bool]:
        out = [False] * len(self.table.pieces)
        for i, piece in enumerate(self.table.pieces):
            if i in self.table.special or not piece:
                continue
            out[i] = self.state.clone().advance_str(piece)
        return out

    def accept(self, token_id: int) -> bool:
        return self.state.advance_str(self.table.pieces[token_id])

    def can_stop(self) -> bool:
        return self.state.can_stop()
