"""Front-end plumbing around the sampler, mirroring the reference's front ends:

* `params_from_request` — the OpenAI-style request fields of the HTTP server (tools/qpack-server.cpp:72-82,
  `sampling(const Json&)`), incl. `frequency_penalty -> 1 + 0.5 * x` when no `repeat_penalty` is given;
* `params_from_cli` — the command-line flags of the CLI (tools/qpack-cli.cpp:43-49);
* `RequestBatcher` — many requests sharing one handle.  The reference creates one `qp::Sampler` per request
  (tools/qpack-server.cpp:127) and serialises generations behind a mutex (qpack-server.cpp:159); here every request
  owns a row of a `BatchSampler` (its own parameters and random stream), rows are taken and released while other
  requests keep decoding, and one sampling call serves all of them.

Host logic only: no CUDA code in this file.
"""
from __future__ import annotations

from typing import Dict, Hashable, List, Mapping, Optional, Sequence

import numpy as np
import torch

from .sampler import BatchSampler, SamplerParams


def params_from_request(body: Mapping) -> SamplerParams:
    """qpack-server.cpp:72-82: fields that are present override the defaults of qp::SamplerParams; `repeat_penalty`
    wins over `frequency_penalty`, which maps to 1 + 0.5 * frequency_penalty."""
    p = SamplerParams()
    if "temperature" in body:
        p.temperature = float(np.float32(body["temperature"]))
    if "top_p" in body:
        p.top_p = float(np.float32(body["top_p"]))
    if "top_k" in body:
        p.top_k = int(body["top_k"])
    if "min_p" in body:
        p.min_p = float(np.float32(body["min_p"]))
    if "repeat_penalty" in body:
        p.repeat_penalty = float(np.float32(body["repeat_penalty"]))
    elif "frequency_penalty" in body:
        p.repeat_penalty = float(np.float32(1.0) + np.float32(body["frequency_penalty"]) * np.float32(0.5))
    if "seed" in body:
        p.seed = int(body["seed"]) & 0xFFFFFFFFFFFFFFFF
    return p


_CLI_FLAGS = {  # tools/qpack-cli.cpp:43-49
    "--temp": ("temperature", float),
    "--top-k": ("top_k", int),
    "--top-p": ("top_p", float),
    "--min-p": ("min_p", float),
    "--repeat-penalty": ("repeat_penalty", float),
    "--repeat-last-n": ("repeat_last_n", int),
    "--seed": ("seed", int),
}


def params_from_cli(argv: Sequence[str]) -> SamplerParams:
    """The sampler flags of the CLI; other arguments are skipped.  A flag without a value raises ValueError (the
    reference's `next()` fails the same way)."""
    p = SamplerParams()
    i = 0
    while i < len(argv):
        a = argv[i]
        if a in _CLI_FLAGS:
            if i + 1 >= len(argv):
                raise ValueError(f"{a} needs a value")
            name, conv = _CLI_FLAGS[a]
            setattr(p, name, conv(argv[i + 1]))
            i += 2
        else:
            i += 1
    return p


class RequestBatcher:
    """Requests that come and go, sampled together.

    Every admitted request owns the lowest free row of the handle; `step` samples the rows [0, span) in one call
    (row r of the logits belongs to the request on row r; rows without a request are sampled too and ignored).
    Admission and release are ordered on the sampler's stream, so they may be interleaved with steps freely.
    """

    def __init__(self, max_requests: int, device: int = 0, defaults: Optional[SamplerParams] = None):
        self.sampler = BatchSampler(max_requests, device)
        self.sampler.set_params(defaults or SamplerParams(seed=1))
        self._row_of: Dict[Hashable, int] = {}
        self._free: List[int] = list(range(max_requests))

    def admit(self, request_id: Hashable, params: SamplerParams) -> int:
        if request_id in self._row_of:
            raise KeyError(f"request {request_id!r} is already admitted")
        if not self._free:
            raise RuntimeError("no free row: release a request first")
        row = min(self._free)
        self._free.remove(row)
        self.sampler.set_row_params(row, params)
        self._row_of[request_id] = row
        return row

    def release(self, request_id: Hashable) -> None:
        self._free.append(self._row_of.pop(request_id))

    def row(self, request_id: Hashable) -> int:
        return self._row_of[request_id]

    @property
    def span(self) -> int:
        """Rows a step has to cover: one past the highest row in use."""
        return 1 + max(self._row_of.values()) if self._row_of else 0

    def step(self, logits: torch.Tensor, history: Optional[torch.Tensor] = None, hist_len=None,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Samples rows [0, span) of `logits` ([>= span, V] on the sampler's GPU); returns the ids [span] (device)."""
        n = self.span
        if n == 0:
            return torch.empty(0, dtype=torch.int32, device=logits.device)
        hl = hist_len[:n] if isinstance(hist_len, torch.Tensor) else hist_len
        return self.sampler.sample(logits[:n], None if history is None else history[:n], hl, out=out)

    def tokens(self, ids: torch.Tensor) -> Dict[Hashable, int]:
        """The sampled token of every admitted request, from the ids of a step (one device-to-host copy)."""
        host = ids.cpu().numpy()
        return {rid: int(host[row]) for rid, row in self._row_of.items()}

    def close(self) -> None:
        self.sampler.close()
