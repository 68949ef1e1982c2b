"""The C++ mirror of the reference interface (include/qpack_b200/sampler.hpp): a port of the reference's own
micro-benchmark is compiled against it, run on the GPU and compared with the fixtures generated from the
reference, including draw() / accept() on host-side pairs (checked against the CPU checker's stream)."""
import os
import re
import subprocess

import numpy as np
import pytest

from oracle import Oracle
from qpack_b200 import build, synth

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_sampler_bench_port(golden, tmp_path):
    lib = build.build()
    exe = str(tmp_path / "sampler_bench_port")
    subprocess.run(["g++", "-std=c++17", "-O2", "-I", os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "cpp", "sampler_bench_port.cpp"), "-o", exe, lib,
                    "-Wl,-rpath," + os.path.dirname(lib)], check=True)
    out = subprocess.run([exe], check=True, capture_output=True, text=True).stdout.strip().splitlines()
    assert len(out) == 4
    x, h = synth.sampler_bench_row()
    for k, line in enumerate(out):
        m = re.search(r"dist (\d+) first (\d+) p0 (\S+) draws((?: \d+){8}) accept (\d) repl (-?\d+) draw (\d+)", line)
        assert m, line
        want_ids = golden[f"sb{k}_dist_ids"]
        assert int(m.group(1)) == len(want_ids) and int(m.group(2)) == int(want_ids[0])
        assert np.float32(float(m.group(3))) == golden[f"sb{k}_dist_p"][0]
        assert [int(v) for v in m.group(4).split()] == golden[f"sb{k}_draws"].tolist()
        # the same call sequence on the CPU checker: dist, 8 samples, accept(first id), draw
        o = Oracle(golden[f"sb{k}_params"])
        ids, pr = o.dist(x[0], h[0])
        for _ in range(8):
            o.sample(x[0], h[0])
        acc, repl = o.accept(ids, pr, int(ids[0]))
        drawn = o.draw(ids, pr)
        assert int(m.group(5)) == int(acc) and int(m.group(7)) == drawn
        if not acc:
            assert int(m.group(6)) == repl
