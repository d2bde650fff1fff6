"""Search: quasi-random points, GP and TPE find a quadratic's minimum, ASHA promotes the
best third, and the driver resumes from trials.jsonl."""
import json
import math

import numpy as np
import pytest

from bux_b200.lang import compile_spaces
from bux_b200.search import Search, gp, halving, methods, tpe
from bux_b200.config import training as T


def _f(u):
    return float(((u - np.array([0.3, 0.7])) ** 2).sum())


def test_points_are_in_the_cube_and_repeatable():
    for name, fn in methods.POINTS.items():
        pts = np.array([fn(i, 3, 5) for i in range(16)])
        assert pts.shape == (16, 3) and (pts >= 0).all() and (pts < 1).all(), name
        assert np.allclose(fn(7, 3, 5), pts[7])
    h = np.array([methods.halton_point(i, 2, 0) for i in range(64)])
    assert abs(h.mean() - 0.5) < 0.05  # low discrepancy


@pytest.mark.parametrize("which", ["gp", "tpe"])
def test_model_based_methods_beat_random(which):
    rng = np.random.default_rng(0)
    x = np.array([methods.halton_point(i, 2, 0) for i in range(8)])
    y = np.array([_f(p) for p in x])
    for _ in range(20):
        p = gp.suggest(x, y, 2, rng) if which == "gp" else tpe.suggest(x, y, 2, rng, gamma=0.25, candidates=48)
        x, y = np.vstack([x, p]), np.append(y, _f(p))
    start = y[:8].min()
    assert y.min() < (0.01 if which == "gp" else 0.05) and y.min() < start
    assert np.median(y[-8:]) < np.median(y[:8])  # later trials concentrate near the minimum


def test_gp_interpolates_and_log_ei_is_finite_in_the_tail():
    x = np.linspace(0, 1, 8)[:, None]
    y = np.sin(4 * x[:, 0])
    g = gp.GP(x, y)
    mu, sd = g.predict(x)
    assert np.allclose(mu, y, atol=0.05) and (sd < 0.2).all()
    out = gp.log_ei(np.array([0.0, 50.0]), np.array([1.0, 1.0]), best=0.0)
    assert np.isfinite(out).all() and out[0] > out[1]


def test_asha_promotes_the_best_third():
    h = halving.Halving(T.HalvingConfig(eta=3, rungs=3), steps=900)
    assert [h.rung_steps(r) for r in range(3)] == [100, 300, 900]
    for t in range(3):
        assert h.next_job(t) == (t, 0, 100)
        h.report(t, 0, float(t))
    assert h.next_job(3) == (0, 1, 300)      # asynchronous: the best of three goes up at once
    assert h.next_job(3) == (3, 0, 100)      # 3 // 3 = 1 promotion, then new trials again
    h.report(3, 0, -1.0)
    assert h.next_job(4) == (3, 1, 300)      # a new best of its rung that was not sent up yet
    assert h.next_job(4) == (4, 0, 100)
    h.report(0, 1, 0.5)
    h.report(3, 1, 0.4)
    assert h.next_job(5) == (5, 0, 100)      # two results at rung 1: 2 // 3 = 0 promotions


SRC = """
d_model=16
vocab_size=32
block = [rmsnorm gqa(num_heads=2, num_kv_heads=1, rope=rope())] [rmsnorm gated_mlp(intermediate_size=32, activation=swish)]
model = embed block n head
n = rmsnorm
data = synthetic
optimizer = adamw(lr=log_uniform(1e-4, 1e-1), weight_decay=uniform(0.0, 0.2))
seq_len = 8
batch = 2
steps = 9
search = search(method=gp(startup=4), trials=10)
"""


def test_driver_records_resumes_and_writes_best(tmp_path):
    (space,) = compile_spaces(SRC, filename="s.bux")
    s = Search(space, out=tmp_path)
    assert sorted(s.cube.names) == ["optimizer.lr", "optimizer.weight_decay"]

    def train(run):  # a stand-in for training: the loss is a function of the settings
        lr, wd = run.train.optimizer.lr, run.train.optimizer.weight_decay
        return {"loss": (math.log10(lr) + 2.5) ** 2 + (wd - 0.05) ** 2}

    seen = []
    for _ in range(4):
        job = s.next_job()
        seen.append(job["values"])
        s.report(job, train(job["run"]))
    again = Search(space, out=tmp_path)          # resumes: four trials on file
    assert len(again.trials) == 4 and again.folder == s.folder
    best = again.run(train, echo=lambda *_: None)
    assert len(again.trials) == 10 and again.next_job() is None
    assert best["objective"] < 0.5
    text = (again.folder / "best.bux").read_text()
    assert "objective" in text and "adamw" in text
    lines = [json.loads(x) for x in (again.folder / "trials.jsonl").read_text().splitlines()]
    assert [r["trial"] for r in lines] == list(range(10))
