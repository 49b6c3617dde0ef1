"""``--flag value`` command lines shared by every entry point.

Same conventions as the reference binaries (src/train.c:29-41): flags are scanned linearly,
unknown flags are ignored, a bare flag is a boolean.  ``--help`` prints the known flags.

Every flag can also be written ``--kh-<name>``.  That spelling is for launches under
``python -m torch.distributed.run``, whose argument parser rejects the whole command line when a
script flag is an abbreviation of one of its own options (``--d`` of ``--duplicate-...``, ``--log``
of ``--log-dir``): ``... -m kharon_b200.pp_train --kh-d 2048 --kh-log 10``.
"""
from __future__ import annotations

import sys


class Flags:
    def __init__(self, argv=None, prog=""):
        self.argv = list(sys.argv[1:] if argv is None else argv)
        self.prog = prog
        self.known = []

    def _find(self, name):
        keys = ("--" + name, "--kh-" + name)
        for i, a in enumerate(self.argv):
            if a in keys:
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
