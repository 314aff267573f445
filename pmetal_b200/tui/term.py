"""Raw-mode key input for the terminal front end (POSIX ttys; no curses dependency)."""
from __future__ import annotations

import os
import select
import sys
from typing import List, Optional

_ESCAPES = {"[A": "up", "[B": "down", "[C": "right", "[D": "left", "[Z": "backtab", "[H": "home", "[F": "end",
            "[5~": "pageup", "[6~": "pagedown", "[3~": "delete", "OA": "up", "OB": "down", "OC": "right", "OD": "left"}


def decode_keys(data: str) -> List[str]:
    """Split a chunk of terminal input into key names: printable characters stay themselves, control bytes and escape
    sequences become ``enter``, ``tab``, ``backspace``, ``esc``, ``up`` ... and ``ctrl-c``."""
    keys: List[str] = []
    i = 0
    while i < len(data):
        ch = data[i]
        if ch == "\x1b":
            hit = next((name for seq, name in _ESCAPES.items() if data.startswith(seq, i + 1)), None)
            if hit is not None:
                seq = next(s for s, n in _ESCAPES.items() if data.startswith(s, i + 1))
                keys.append(hit)
                i += 1 + len(seq)
                continue
            keys.append("esc")
        elif ch in "\r\n":
            keys.append("enter")
        elif ch == "\t":
            keys.append("tab")
        elif ch in "\x7f\x08":
            keys.append("backspace")
        elif ch == "\x03":
            keys.append("ctrl-c")
        elif ch >= " ":
            keys.append(ch)
        i += 1
    return keys


class RawTerminal:
    """Context manager: stdin in cbreak mode without echo; ``read_keys(timeout)`` returns the keys typed since the last call."""

    def __init__(self, stream=None):
        self.stream = stream or sys.stdin
        self.fd = self.stream.fileno()
        self._saved = None

    def __enter__(self) -> "RawTerminal":
        import termios
        import tty
        self._saved = termios.tcgetattr(self.fd)
        tty.setcbreak(self.fd)
        return self

    def __exit__(self, *exc) -> None:
        import termios
        if self._saved is not None:
            termios.tcsetattr(self.fd, termios.TCSADRAIN, self._saved)

    def read_keys(self, timeout: float) -> List[str]:
        r, _, _ = select.select([self.fd], [], [], timeout)
        if not r:
            return []
        data = os.read(self.fd, 1024).decode("utf-8", "replace")
        return decode_keys(data)


def is_interactive(stream: Optional[object] = None) -> bool:
    s = stream or sys.stdin
    try:
        return bool(s.isatty()) and sys.stdout.isatty()
    except (AttributeError, ValueError):
        return False
