"""Advisory expert-reuse predictor on synthetic sticky routing: better pool coverage than a frequency ranking."""
import numpy as np

from layerstorm_b200.speculation.expert_ridge import ExpertRidge


def _routing(rng, J, E, K, T):
    """Sticky routing: a position keeps most of the previous position's experts; layer j+1 copies half of layer j's set."""
    out = np.zeros((T, J, K), np.int64)
    cur = [rng.choice(E, K, replace=False) for _ in range(J)]
    for t in range(T):
        for j in range(J):
            keep = cur[j][rng.random(K) < 0.7]
            if j > 0:
                keep = np.union1d(keep, rng.choice(out[t, j - 1], K // 2, replace=False))[:K]
            fill = rng.choice(np.setdiff1d(np.arange(E), keep), K - len(keep), replace=False)
            cur[j] = np.concatenate([keep, fill])[:K]
            out[t, j] = cur[j]
    return out


def test_ridge_pool_beats_frequency_ranking():
    rng = np.random.default_rng(0)
    J, E, K, T, M = 3, 64, 6, 400, 16
    routed = _routing(rng, J, E, K, T)
    er = ExpertRidge(J, E, K, lag=1, refresh=8)
    freq = np.zeros((J, E))
    hit_f = seen = 0
    for t in range(T):
        pool = er.pool(M)
        assert pool.shape == (J, M) and len(set(pool[0].tolist())) == M
        if t >= 100:
            fpool = np.argsort(-freq, axis=1)[:, :M]
            for j in range(J):
                hit_f += int(np.isin(routed[t, j], fpool[j]).sum())
                seen += K
        if t == 100:
            er.hits[:] = 0; er.seen[:] = 0
        er.step(routed[t])
        for j in range(J):
            freq[j, routed[t, j]] += 1
    cov_ridge, cov_freq = float(er.coverage().mean()), hit_f / seen
    assert cov_ridge > cov_freq + 0.15 and cov_ridge > 0.6, (cov_ridge, cov_freq)
    ev = er.evict_scores()
    assert ev.shape == (J, E) and np.all(ev == -er.score())
    assert er.w[:, 1].mean() > 0                                   # "routed at the previous position" carries weight


def test_score_then_update_is_causal():
    er = ExpertRidge(2, 8, 2, refresh=1)
    s0 = er.score().copy()
    er.step(np.array([[1, 2], [3, -1]]))
    assert np.all(s0 == 0) and er.prev[0, 1] == 1 and er.prev[1, 3] == 1 and er.prev.sum() == 3
    assert er.score()[0, 1] >= er.score()[0, 5]
