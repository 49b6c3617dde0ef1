"""`bench.py --impl reference`: runs the unmodified reference build under baseline/_ref through
its own entry point (pp_train) for the same metric, or reports why it cannot."""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def main(argv):
    exe = os.path.join(HERE, "_ref", "build", "pp_train.exe")
    if not os.path.exists(exe):
        print(json.dumps({"impl": "reference", "unavailable": "reference build not present under baseline/_ref (run baseline/build_reference.sh)"}))
        return 0
    from . import reference_run
    return reference_run.run(argv)
