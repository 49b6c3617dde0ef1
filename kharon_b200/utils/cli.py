"""``--flag value`` command lines shared by every entry point.

Same conventions as the reference binaries (src/train.c:29-41): flags are scanned linearly,
unknown flags are ignored, a bare flag is a boolean.  ``--help`` prints the known flags.
"""
from __future__ import annotations

import sys


class Flags:
    def __init__(self, argv=None, prog=""):
        self.argv = list(sys.argv[1:] if argv is None else argv)
        self.prog = prog
        self.known = []

    def _find(self, name):
        key = "--" + name
        for i, a in enumerate(self.argv):
            if a == key:
                return i
        return -1

    def has(self, name, help=""):
        self.known.append((name, "flag", False, help))
        return self._find(name) >= 0

    def _val(self, name, default, conv, help):
        self.known.append((name, conv.__name__, default, help))
        i = self._find(name)
        if i >= 0 and i + 1 < len(self.argv):
            return conv(self.argv[i + 1])
        return default

    def int(self, name, default, help=""):
        return self._val(name, default, int, help)

    def float(self, name, default, help=""):
        return self._val(name, default, float, help)

    def str(self, name, default, help=""):
        return self._val(name, default, str, help)

    def maybe_help(self):
        if "--help" in self.argv or "-h" in self.argv:
            print("usage: python -m kharon_b200.%s [flags]" % self.prog)
            for name, kind, default, help in self.known:
                print("  --%-12s %-6s default %-12r %s" % (name, kind, default, help))
            raise SystemExit(0)
