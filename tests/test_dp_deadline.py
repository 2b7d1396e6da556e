"""Host-side failure path of the data-parallel layer, without a GPU: the deadline loop behind
prad_dp_wait_host (csrc/dp_deadline.h) driven by CPU threads that stand for ranks and a stub
communicator (tests/cpp/dp_deadline_test.cpp).  A rank that never arrives must end the others' wait
with "timed out" after the deadline and exactly one abort per waiting rank; a late rank inside the
deadline is simply waited for; an asynchronous error ends the wait at once."""
import os
import shutil
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def lines(tmp_path_factory):
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else shutil.which("g++")
    if not cxx:
        pytest.skip("no C++ compiler")
    exe = tmp_path_factory.mktemp("dp") / "dp_deadline_test"
    subprocess.run([cxx, "-O1", "-std=c++17", "-pthread", os.path.join(HERE, "cpp", "dp_deadline_test.cpp"), "-o", str(exe)],
                   check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True, timeout=60).stdout
    rows = []
    for ln in out.splitlines():
        name, *kv = ln.split()
        rows.append((name, {k: float(v) for k, v in (x.split("=") for x in kv)}))
    return rows


def _of(lines, name):
    return [d for n, d in lines if n == name]


def test_everybody_arrives(lines):
    rows = _of(lines, "all_arrive")
    assert len(rows) == 4 and all(r["outcome"] == 0 and r["aborts"] == 0 for r in rows)


def test_a_late_rank_inside_the_deadline_is_waited_for(lines):
    rows = _of(lines, "one_late")
    assert len(rows) == 4 and all(r["outcome"] == 0 and r["aborts"] == 0 for r in rows)
    assert max(r["waited_ms"] for r in rows) >= 40


def test_a_rank_that_never_arrives_times_the_others_out(lines):
    rows = _of(lines, "one_absent")
    assert len(rows) == 3 and all(r["outcome"] == 2 for r in rows)
    assert all(150 <= r["waited_ms"] < 1500 for r in rows)
    assert rows[-1]["aborts"] <= 3 and max(r["aborts"] for r in rows) == 3     # one abort per waiting rank


def test_an_asynchronous_error_ends_the_wait_at_once(lines):
    rows = _of(lines, "async_error")
    assert len(rows) == 1 and rows[0]["outcome"] == 1 and rows[0]["aborts"] == 1 and rows[0]["waited_ms"] < 500
