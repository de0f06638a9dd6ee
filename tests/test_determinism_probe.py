"""Determinism probe and drift diff on the CPU null engine."""
import json

import numpy as np

from layerstorm_b200 import build as _build

_build.build_all(only="runtime")

from layerstorm_b200.utils import determinism_probe as dp


def test_first_divergence():
    assert dp.first_divergence([1, 2, 3], [1, 2, 3]) == -1
    assert dp.first_divergence([1, 2, 3], [1, 9, 3]) == 1
    assert dp.first_divergence([1, 2], [1, 2, 3]) == 2


def test_probe_is_identical_on_the_null_engine_with_and_without_prefix_cache(capsys):
    for extra in ([], ["--prefix-cache"]):
        assert dp.main(["probe", "--test-engine", "--prompt-len", "200", "--gen", "8", "--reps", "3"] + extra) == 0
        rep = json.loads(capsys.readouterr().out.strip())
        assert rep["identical"] and len(rep["runs"]) == 3 and len(rep["runs"][0]) == 8
        assert set(rep["first_divergence"].values()) == {-1}


def test_probe_reports_divergence():
    class Flaky:
        """Orchestrator stand-in whose third run differs at token 2."""
        n = 0

        def submit_request(self, req):
            self.req = req

        def step(self):
            self.n += 1
            self.req.output_ids = [5, 6, 7 if self.n != 3 else 8, 9]
            self.req.done.set()
            return True
    rep = dp.probe(Flaky(), [1, 2, 3], gen=4, reps=3)
    assert not rep["identical"] and rep["first_divergence"] == {"0-1": -1, "0-2": 2, "1-2": 2}


def test_drift_names_the_first_layer_over_tolerance(tmp_path, capsys):
    a = {"l0": np.ones((4, 8)), "l1": np.arange(8.0), "l2": np.ones(3)}
    b = {"l0": np.ones((4, 8)), "l1": np.arange(8.0) + 1e-6, "l2": np.ones(3) * 1.1, "extra": np.zeros(1)}
    rep = dp.drift(a, b, rtol=1e-3)
    assert rep["first_over_tolerance"] == "l2" and rep["only_in_b"] == ["extra"] and rep["rows"][1]["rel"] < 1e-6
    np.savez(tmp_path / "a.npz", **a)
    np.savez(tmp_path / "b.npz", **a)
    assert dp.main(["drift", str(tmp_path / "a.npz"), str(tmp_path / "b.npz")]) == 0
    np.savez(tmp_path / "c.npz", **b)
    assert dp.main(["drift", str(tmp_path / "a.npz"), str(tmp_path / "c.npz")]) == 1
