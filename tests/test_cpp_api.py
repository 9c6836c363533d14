"""Runs the C++ API tests (tests/cpp) built by topoanns_b200/host/Makefile."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "tests", "cpp", "build")


def _build():
    subprocess.check_call(["make", "-C", os.path.join(ROOT, "topoanns_b200", "csrc"), "-j8"], stdout=subprocess.DEVNULL)
    subprocess.check_call(["make", "-C", os.path.join(ROOT, "topoanns_b200", "host"), "-j8"], stdout=subprocess.DEVNULL)


def _run(name, tmp_path):
    _build()
    env = dict(os.environ, TANN_TEST_TMP=str(tmp_path))
    r = subprocess.run([os.path.join(BIN, name)], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert f"{name} passed" in r.stdout


def test_cpp_host_only_api(tmp_path):
    _run("test_api_host", tmp_path)


@pytest.mark.gpu
def test_cpp_search_api(tmp_path):
    _run("test_api_search", tmp_path)
