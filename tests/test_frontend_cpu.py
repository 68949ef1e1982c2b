"""Front-end parameter plumbing (no GPU): the request and command-line mappings of the reference's front ends
(tools/qpack-server.cpp:72-82, tools/qpack-cli.cpp:43-49), restated as expectations."""
import numpy as np
import pytest

from qpack_b200.frontend import params_from_cli, params_from_request
from qpack_b200.sampler import SamplerParams


def test_request_defaults_are_the_structs():
    assert params_from_request({}) == SamplerParams()  # engine.h:18-24


def test_request_fields_override():
    p = params_from_request({"temperature": 0.3, "top_p": 0.8, "top_k": 12, "min_p": 0.0, "repeat_penalty": 1.3, "seed": 77})
    assert p.top_k == 12 and p.seed == 77
    assert np.float32(p.temperature) == np.float32(0.3) and np.float32(p.top_p) == np.float32(0.8)
    assert p.min_p == 0.0 and np.float32(p.repeat_penalty) == np.float32(1.3)
    assert p.repeat_last_n == 64  # not a request field: stays at its default


def test_frequency_penalty_maps_to_repeat_penalty():
    # qpack-server.cpp:79: 1.f + (float)x * 0.5f, only when repeat_penalty is absent
    assert np.float32(params_from_request({"frequency_penalty": 0.4}).repeat_penalty) == np.float32(1.0) + np.float32(0.4) * np.float32(0.5)
    assert np.float32(params_from_request({"frequency_penalty": -2.0}).repeat_penalty) == np.float32(0.0)
    both = params_from_request({"frequency_penalty": 1.0, "repeat_penalty": 1.05})
    assert np.float32(both.repeat_penalty) == np.float32(1.05)


def test_params_block_layout_from_request():
    arr = params_from_request({"temperature": 0.0, "seed": 2 ** 63 + 5}).to_array()
    assert arr.dtype.itemsize == 32 and int(arr["seed"][0]) == 2 ** 63 + 5 and float(arr["temperature"][0]) == 0.0


def test_cli_flags():
    p = params_from_cli(["-m", "model.qpack", "--temp", "0.2", "--top-k", "5", "--top-p", "0.5", "--min-p", "0.1",
                         "--repeat-penalty", "1.2", "--repeat-last-n", "128", "--seed", "9", "--think"])
    assert (p.top_k, p.repeat_last_n, p.seed) == (5, 128, 9)
    assert (p.temperature, p.top_p, p.min_p, p.repeat_penalty) == (0.2, 0.5, 0.1, 1.2)
    assert params_from_cli(["--ctx", "4096"]) == SamplerParams()
    with pytest.raises(ValueError):
        params_from_cli(["--top-k"])
