"""Format interoperability with the reference's own binaries (built unchanged under baseline/_ref by
``baseline/build_reference.sh``): its test programs must accept the CHRN fixtures this project writes,
and CKP1 checkpoints must travel in both directions between ``python -m kharon_b200.train`` and the
reference's ``train.exe --resume`` (src/core/ckpt.c:25-68, src/train.c:65-70)."""
import os
import re
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BUILD = os.path.join(ROOT, "baseline", "_ref", "build")


def _exe(name):
    path = os.path.join(BUILD, name)
    if not os.path.exists(path):
        pytest.skip("reference binary %s not built (baseline/build_reference.sh)" % name)
    return path


def _env():
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = "/usr/local/cuda/lib64:" + env.get("LD_LIBRARY_PATH", "")
    env["PYTHONPATH"] = ROOT + ":" + env.get("PYTHONPATH", "")
    return env


def _run(cmd, cwd=None):
    p = subprocess.run(cmd, env=_env(), cwd=cwd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    return p.returncode, p.stdout


@pytest.mark.parametrize("kind,tests", [("m1", ["test_loadref", "test_forward", "test_backward", "test_step", "test_grpo"]),
                                        ("attn", ["test_flash"]), ("gen", ["test_infer"])])
def test_reference_tests_accept_our_fixtures(tmp_path, kind, tests):
    from kharon_b200.utils import gen_fixtures
    path = str(tmp_path / (kind + "_ref.bin"))
    gen_fixtures.main([kind, path])
    for t in tests:
        rc, out = _run([_exe(t + ".exe"), path])
        assert rc == 0, "%s on our %s fixture:\n%s" % (t, kind, out[-2000:])
        if t != "test_loadref":
            assert "PASS" in out, out[-2000:]


def _corpus(tmp_path):
    import random
    rnd = random.Random(5)
    words = [bytes(rnd.choice(b"abcdefghijklmnopqrstuvwxyz") for _ in range(rnd.randint(2, 9))) for _ in range(200)]
    data = b" ".join(rnd.choice(words) for _ in range(40000))
    p = tmp_path / "corpus.bin"
    p.write_bytes(data)
    return str(p)


SHAPE = ["--layers", "2", "--d", "128", "--heads", "4", "--seq", "64", "--batch", "8", "--log", "1", "--ckptevery", "0"]


def _losses(out):
    return {int(m.group(1)): float(m.group(2)) for m in re.finditer(r"step\s+(\d+)\s+loss ([\d.]+)", out)}


def test_reference_resumes_from_our_checkpoint(tmp_path):
    data, ck = _corpus(tmp_path), str(tmp_path / "ours.ckpt")
    rc, out = _run([sys.executable, "-m", "kharon_b200.train"] + SHAPE + ["--steps", "6", "--data", data, "--ckpt", ck])
    assert rc == 0, out[-2000:]
    ours = _losses(out)
    rc, out = _run([_exe("train.exe")] + SHAPE + ["--steps", "12", "--data", data, "--ckpt", ck, "--resume"])
    assert rc == 0, out[-2000:]
    assert "resumed from" in out and "at step 6" in out, out[-2000:]
    ref = _losses(out)
    assert sorted(ref) == list(range(7, 13)), out[-2000:]
    # training continues from where ours stopped: the next loss is in line with our curve and it keeps falling
    assert abs(ref[7] - ours[6]) < 0.15 and ref[12] < ours[1], (ours, ref)


def test_we_resume_from_the_reference_checkpoint(tmp_path):
    data, ck = _corpus(tmp_path), str(tmp_path / "ref.ckpt")
    rc, out = _run([_exe("train.exe")] + SHAPE + ["--steps", "6", "--data", data, "--ckpt", ck])
    assert rc == 0, out[-2000:]
    ck12 = str(tmp_path / "ref12.ckpt")
    import shutil
    shutil.copy(ck, ck12)
    rc, out_ref = _run([_exe("train.exe")] + SHAPE + ["--steps", "12", "--data", data, "--ckpt", ck12, "--resume"])
    assert rc == 0, out_ref[-2000:]
    rc, out = _run([sys.executable, "-m", "kharon_b200.train"] + SHAPE + ["--steps", "12", "--data", data, "--ckpt", ck, "--resume"])
    assert rc == 0, out[-2000:]
    assert "resumed from" in out and "at step 6" in out, out[-2000:]
    ours, ref = _losses(out), _losses(out_ref)
    # same weights, moments, step count and data stream: the two bf16 implementations stay together
    for s in range(7, 13):
        assert abs(ours[s] - ref[s]) < 3e-2 * max(1.0, ref[s]), (s, ours, ref)
