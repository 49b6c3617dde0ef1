"""Writes a byte-level training corpus: ``python -m kharon_b200.utils.prep_data [data/input.bin]``.
A text file given with ``--from`` is copied as bytes; otherwise a repeatable synthetic corpus is
generated (the reference's scripts/prep_data.py falls back to the same kind of corpus when it cannot
download tinyshakespeare; there is no network access here)."""
import os
import sys


def synthetic(n_lines=20000) -> bytes:
    return "".join("to be or not to be that is the question %d\n" % (i % 97) for i in range(n_lines)).encode()


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    src = None
    if "--from" in argv:
        i = argv.index("--from")
        src = argv[i + 1]
        argv = argv[:i] + argv[i + 2:]
    out = argv[0] if argv else "data/input.bin"
    os.makedirs(os.path.dirname(out) or ".", exist_ok=True)
    data = open(src, "rb").read() if src else synthetic()
    with open(out, "wb") as f:
        f.write(data)
    print("wrote %s (%d bytes)" % (out, len(data)))
    return out


if __name__ == "__main__":
    main()
