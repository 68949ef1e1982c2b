"""CPU tests of the checker itself: the C restatement against the fixtures generated from the reference
(tests/golden/make_golden.py) and, when the compiled reference is present, against it directly."""
import numpy as np
import pytest

from oracle import Oracle, Ref, make_params
from qpack_b200 import synth

from helpers import small_case


def test_mt19937_64_known_answers():
    # ISO C++ [rand.predef]: the 10000th output of a default-constructed mt19937_64 (seed 5489)
    o = Oracle(make_params(1, seed=5489))
    for _ in range(9999):
        o.next_word()
    assert o.next_word() == 9981545732273789042
    # uniform = word * 2^-64 (libstdc++ generate_canonical on a 64-bit engine)
    a, b = Oracle(make_params(1, seed=42)), Oracle(make_params(1, seed=42))
    for _ in range(1000):
        assert a.next_uniform() == b.next_word() * 2.0 ** -64


def test_small_cases_match_reference_fixtures(golden):
    for i in range(int(golden["n_small"])):
        x, hist, hl, p, ids, cnt, dids, dp = small_case(golden, i)
        r = Oracle.sample_rows(p, x, hist, hl, max_out=dids.shape[1])
        assert np.array_equal(r["ids"], ids), i
        assert np.array_equal(r["count"], cnt), i
        assert np.array_equal(r["dist_ids"], dids), i
        assert np.array_equal(r["dist_p"].view(np.uint32), dp.view(np.uint32)), i


def test_sampler_bench_row_known_answers(golden):
    x, h = synth.sampler_bench_row()
    for k in range(4):
        s = Oracle(golden[f"sb{k}_params"])
        ids, pr = s.dist(x[0], h[0])
        assert np.array_equal(ids, golden[f"sb{k}_dist_ids"])
        assert np.array_equal(pr.view(np.uint32), golden[f"sb{k}_dist_p"].view(np.uint32))
        draws = np.array([s.sample(x[0], h[0]) for _ in range(8)], np.int32)
        assert np.array_equal(draws, golden[f"sb{k}_draws"])
    # greedy picks the lowest index of the ~152 copies of the maximum
    assert golden["sb0_dist_ids"].tolist() == [321] and golden["sb1_dist_ids"].tolist() == [321]
    assert len(golden["sb2_dist_ids"]) == 36


def test_single_row_loop_matches_reference_fixture(golden):
    params, hist0 = synth.single_row_loop()
    s = Oracle(params)
    hist = list(hist0)
    for step in range(len(golden["loop_ids"])):
        lg = synth.single_row_step(step)
        assert float(lg.astype(np.float64).sum()) == golden["loop_logit_sums"][step], "input generator drifted"
        ids, pr = s.dist(lg[0], np.array(hist, np.int32))
        t = s.draw(ids, pr)
        assert t == golden["loop_ids"][step] and len(ids) == golden["loop_counts"][step], step
        hist.append(t)


@pytest.mark.parametrize("name,maker", [("serving", lambda: synth.serving_batch(rows=8)),
                                        ("mixed", lambda: synth.mixed_batch(rows=16)),
                                        ("sharded", lambda: synth.sharded_batch(rows=8)),
                                        ("llama3", lambda: synth.llama3_batch(rows=4))])
def test_config_rows_match_reference_fixtures(golden, name, maker):
    wl = maker()
    assert np.array_equal(wl.logits.astype(np.float64).sum(axis=1), golden[f"{name}_logit_sums"])
    r = Oracle.sample_rows(wl.params, wl.logits, wl.history, wl.hist_len, max_out=golden[f"{name}_dist_ids"].shape[1])
    assert np.array_equal(r["ids"], golden[f"{name}_ids"])
    assert np.array_equal(r["count"], golden[f"{name}_count"])
    assert np.array_equal(r["dist_ids"], golden[f"{name}_dist_ids"])
    assert np.array_equal(r["dist_p"].view(np.uint32), golden[f"{name}_dist_p"].view(np.uint32))


def test_accept_rule_against_compiled_reference():
    if not Ref.available():
        pytest.skip("compiled reference not present")
    rng = np.random.default_rng(7)
    for case in range(200):
        V = 500
        x = (rng.standard_normal(V) * 3).astype(np.float32)
        p = make_params(1, temperature=0.9, top_k=8, top_p=0.95, min_p=0.0, repeat_penalty=1.0, seed=int(case + 1))
        o, r = Oracle(p), Ref(p)
        ids, pr = o.dist(x)
        ids2, pr2 = r.dist(x)
        assert np.array_equal(ids, ids2) and np.array_equal(pr, pr2)
        tok = int(rng.choice(np.concatenate([ids, [int(rng.integers(0, V))]])))
        for _ in range(3):
            assert o.accept(ids, pr, tok) == r.accept(ids2, pr2, tok)


def test_random_rows_against_compiled_reference():
    if not Ref.available():
        pytest.skip("compiled reference not present")
    rng = np.random.default_rng(11)
    for case in range(120):
        V = int(rng.choice([1, 2, 7, 64, 1000, 5000, 20000]))
        B = 3
        x = (rng.standard_normal((B, V)) * 2).astype(np.float32)
        if case % 2:
            x = np.round(x * 2) / 2
        H = int(rng.choice([1, 5, 100]))
        hist = rng.integers(-1, V + 1, size=(B, H)).astype(np.int32)
        hl = rng.integers(0, H + 1, size=B).astype(np.int32)
        p = make_params(B, temperature=rng.choice([0, 0.7, 1.2], B), top_k=rng.choice([0, 3, 40], B),
                        top_p=rng.choice([0.8, 0.95, 1.0], B), min_p=rng.choice([0, 0.1], B),
                        repeat_penalty=rng.choice([1.0, 1.2, 0.85], B), repeat_last_n=rng.choice([0, 3, 64], B),
                        seed=rng.integers(1, 1 << 62, B).astype(np.uint64))
        a = Oracle.sample_rows(p, x, hist, hl, max_out=32)
        b = Ref.sample_rows(p, x, hist, hl, max_out=32, threads=2)
        for k in ("ids", "count", "dist_ids"):
            assert np.array_equal(a[k], b[k]), (case, k)
        assert np.array_equal(a["dist_p"].view(np.uint32), b["dist_p"].view(np.uint32)), case


def test_adversarial_rows_against_compiled_reference():
    """The rows the GPU tests use to force the fallback paths (orderings, plateaus, ties, outliers, -inf): the
    checker agrees with the compiled reference on them, so they are valid expectations."""
    if not Ref.available():
        pytest.skip("compiled reference not present")
    from helpers import adversarial_rows
    V = 151936
    rng = np.random.default_rng(7)
    rows = adversarial_rows(V, rng)
    x = np.stack([rows[n] for n in rows]).astype(np.float32)
    B = x.shape[0]
    hist = rng.integers(0, V, (B, 96)).astype(np.int32)
    hist[:, :8] = np.argsort(-x, axis=1, kind="stable")[:, :8]
    for top_k, rp in ((50, 1.15), (200, 1.0), (40, 0.9), (1, 1.3)):
        p = make_params(B, temperature=0.8, top_k=top_k, top_p=0.95, min_p=0.01, repeat_penalty=rp, repeat_last_n=96,
                        seed=np.arange(B) + 11)
        a = Oracle.sample_rows(p, x, hist, None, max_out=256)
        b = Ref.sample_rows(p, x, hist, None, max_out=256, threads=2)
        for k in ("ids", "count", "dist_ids"):
            assert np.array_equal(a[k], b[k]), (top_k, rp, k)
        assert np.array_equal(a["dist_p"].view(np.uint32), b["dist_p"].view(np.uint32)), (top_k, rp)
