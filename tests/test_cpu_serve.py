"""The engine process's host half without a GPU: request lines (fields, ranges, errors as the reference's parse_gen words
them), the STOP rule, and the command line."""
import pathlib
import subprocess

import pytest

ROOT = pathlib.Path(__file__).resolve().parents[1]
PKG = ROOT / "qwen3.8-flash-next-2x-p100_b200"


@pytest.fixture(scope="module")
def check_exe():
    exe = ROOT / "tests" / "csrc" / "serve_input_check"
    subprocess.run(["g++", "-std=c++17", "-O1", "-Wall", str(ROOT / "tests" / "csrc" / "serve_input_check.cpp"), "-o", str(exe), "-lpthread"], check=True)
    return exe


def _parse(exe, lines):
    r = subprocess.run([str(exe)], input="\n".join(lines) + "\n", capture_output=True, text=True, check=True)
    return r.stdout.strip().split("\n")


def test_request_lines(check_exe):
    out = _parse(check_exe, [
        "GEN 16 1,2,3",
        "GEN 8 temperature=0.7 top_p=0.9 top_k=40 min_p=0.05 seed=18446744073709551615 penalty_repeat=1.1 penalty_last_n=32 5,6",
        "GEN 4 temperature=0.5 logit_bias=7:1.5,3:-2 keep=10 ckpt=0 pin=abc 9",
        "BGEN 2 5 temperature=0 top_p=7 11,12",
    ])
    assert out[0] == "OK slot=-1 max_new=16 t=0 top_p=1 top_k=0 min_p=0 rep=1 freq=0 pres=0 last_n=64 seed=none pen=0 bias= ids=1;2;3;"
    assert out[1] == "OK slot=-1 max_new=8 t=0.7 top_p=0.9 top_k=40 min_p=0.05 rep=1.1 freq=0 pres=0 last_n=32 seed=18446744073709551615 pen=1 bias= ids=5;6;"
    assert out[2] == "OK slot=-1 max_new=4 t=0.5 top_p=1 top_k=0 min_p=0 rep=1 freq=0 pres=0 last_n=64 seed=none pen=0 bias=3:-2;7:1.5; ids=9;"
    assert out[3].startswith("OK slot=2 max_new=5 t=0 top_p=7 ")      # a greedy request's other values are not checked


@pytest.mark.parametrize("line, msg", [
    ("GEN", "GEN: no max_new"),
    ("GEN x 1", "GEN: max_new=x is not a whole number"),
    ("GEN 0 1", "GEN: max_new must be a number >= 1"),
    ("GEN 4", "GEN: no token ids"),
    ("GEN 4 temperature=0.5", "GEN: no token ids"),
    ("GEN 4 1,2 3", "GEN: text after the token ids"),
    ("GEN 4 1,,2", "GEN: token id '' is not a whole number"),
    ("GEN 4 1,1000", "GEN: token id 1000 outside the vocabulary"),
    ("GEN 4 -1", "GEN: token id -1 outside the vocabulary"),
    ("GEN 4 colour=red 1", "GEN: unknown key colour"),
    ("GEN 4 temperature=warm 1", "GEN: temperature=warm is not a number"),
    ("GEN 4 temperature=-1 1", "GEN: sampling: temperature must be a finite number >= 0"),
    ("GEN 4 temperature=1 top_p=0 1", "GEN: sampling: top_p must be in (0, 1]"),
    ("GEN 4 temperature=1 min_p=2 1", "GEN: sampling: min_p must be in [0, 1]"),
    ("GEN 4 temperature=1 top_k=-3 1", "GEN: sampling: top_k must be >= 0"),
    ("GEN 4 temperature=1 penalty_repeat=0 1", "GEN: sampling: penalty_repeat must be a finite number > 0"),
    ("GEN 4 temperature=1 penalty_last_n=-1 1", "GEN: sampling: penalty_last_n must be >= 0"),
    ("GEN 4 temperature=1 penalty_freq=0.5 penalty_last_n=5000 1", "GEN: sampling: penalty_last_n above 4096"),
    ("GEN 4 seed=18446744073709551616 1", "GEN: seed=18446744073709551616 is not a whole number from 0 to 2^64-1"),
    ("GEN 4 seed=-4 1", "GEN: seed=-4 is not a whole number from 0 to 2^64-1"),
    ("GEN 4 logit_bias=5 1", "GEN: logit_bias entry '5' is not <token id>:<bias> within the vocabulary"),
    ("GEN 4 logit_bias=5000:1 1", "GEN: logit_bias entry '5000:1' is not <token id>:<bias> within the vocabulary"),
    ("GEN 4 logit_bias=5:101 1", "GEN: logit_bias 5:101: a bias is from -100 to 100"),
    ("GEN 4 logit_bias=5:1,5:2 1", "GEN: logit_bias names token 5 twice"),
    ("BGEN 4", "BGEN: no max_new"),
    ("BGEN", "BGEN: no slot"),
])
def test_request_errors(check_exe, line, msg):
    assert _parse(check_exe, [line]) == ["ERR " + msg]


def test_stop_is_for_the_latest_request_line(check_exe):
    r = subprocess.run([str(check_exe), "--stop"], capture_output=True, text=True, check=True)
    a, b = r.stdout.strip().split("\n")[:2]
    assert a.strip() == "GEN:1:stopped PING:0:runs GEN:2:runs GEN:3:stopped"
    assert b == "0 1"
    # BSTOP <slot> is for that slot's latest BGEN: slot 1's first request is stopped, its second is not, slot 2's never was
    assert r.stdout.strip().split("\n")[2] == "1 0 0 1"


@pytest.mark.parametrize("args, msg", [
    ([], "fnx_serve runs as --serve"),
    (["--serve"], "--native is required"),
    (["--serve", "--native"], "--native needs a value"),
    (["--serve", "--native", "m.gguf", "--spec", "99"], "--spec must be 0..31"),
    (["--serve", "--native", "m.gguf", "--batch", "9"], "--batch must be 1..8"),
    (["--serve", "--native", "m.gguf", "--colour", "red"], "unknown argument --colour"),
])
def test_command_line(args, msg):
    exe = PKG / "fnx_serve"
    assert exe.exists(), "build the package first (python <package>/build.py)"
    r = subprocess.run([str(exe), *args], capture_output=True, text=True, stdin=subprocess.DEVNULL)
    assert r.returncode == 2 and msg in r.stderr
