"""Builds the stand-alone network simulator with sanitizers, runs its C++ unit tests and a few
command-line scenarios."""
import json
import os
import shutil
import subprocess

import pytest

SRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "meshslice_b200", "csrc", "netsim")

pytestmark = pytest.mark.skipif(shutil.which("g++") is None, reason="no C++ compiler")


@pytest.fixture(scope="module")
def build(tmp_path_factory):
    out = tmp_path_factory.mktemp("netsim")
    srcs = [os.path.join(SRC, f) for f in ("netsim.cc", "scenarios.cc")]
    subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-Wall", "-Werror", "-o",
                    str(out / "netsim_test"), *srcs, os.path.join(SRC, "test.cc")], check=True)
    subprocess.run(["g++", "-std=c++17", "-O2", "-o", str(out / "netsim"), *srcs, os.path.join(SRC, "main.cc")], check=True)
    return out


def test_cpp_unit_tests_pass_under_sanitizers(build):
    r = subprocess.run([str(build / "netsim_test")], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "netsim tests passed" in r.stdout


def _run(build, *args):
    r = subprocess.run([str(build / "netsim"), *args, "--json"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    return json.loads(r.stdout)


def test_msg_scenario_reference_size(build):
    """The reference's msg test: 100 words from node 0 to node 1 on a 2-node torus."""
    out = _run(build, "--scenario", "msg", "--nodes", "2", "--bytes", "400")
    assert out["ok"] and out["packets"] == 1 and out["data_ok"] == 1
    assert 0.1 < out["sim_time_us"] < 100


def test_crossbar_vs_torus_latency_and_bandwidth_curves(build):
    small_t = _run(build, "--scenario", "sendrecv", "--nodes", "8", "--topology", "torus:2x2x2", "--bytes", "64")
    small_x = _run(build, "--scenario", "sendrecv", "--nodes", "8", "--topology", "crossbar", "--bytes", "64")
    assert small_t["ok"] and small_x["ok"]
    big = _run(build, "--scenario", "sendrecv", "--nodes", "8", "--topology", "crossbar", "--bytes", str(8 << 20),
               "--link-gbs", "900", "--nic-gbs", "900", "--mem-gbs", "3000", "--max-mem-reqs", "1024")
    assert big["ok"] and big["gb_per_s_per_node"] > small_x["gb_per_s_per_node"]
    b8 = _run(build, "--scenario", "barrier", "--nodes", "8", "--topology", "crossbar", "--repeat", "4")
    assert b8["barrier_msgs"] == 2 * 7 * 4


def test_bad_arguments_are_rejected(build):
    r = subprocess.run([str(build / "netsim"), "--scenario", "nope"], capture_output=True, text=True)
    assert r.returncode == 2
    r = subprocess.run([str(build / "netsim"), "--topology", "torus:3x3", "--nodes", "8"], capture_output=True, text=True)
    assert r.returncode == 2
