"""The multi-block top-k selection (csrc/kernels/indexer.cu: three histogram passes over 11 + 11 + 10 key bits, a count pass, an emit
pass) restated block by block in NumPy and checked against a stable sort: same entries, ascending, ties to the lower index.  This
checks the algorithm and its bookkeeping (bucket walk from the top, quota of threshold-equal entries, per-block output offsets), not
the CUDA code; the GPU test compares the kernels with the single-block kernel."""
import numpy as np
import pytest

CH = 2048


def sortable(x):
    b = x.view(np.uint32)
    return np.where(b & 0x80000000, ~b, b | 0x80000000).astype(np.uint32)


def split_topk(sc, ne, budget):
    key = sortable(sc[:ne].astype(np.float32))
    nb = (ne + CH - 1) // CH
    prefix, need = np.uint32(0), budget
    for shift, nbins, decided in ((21, 2048, None), (10, 2048, 21), (0, 1024, 10)):
        hist = np.zeros(nbins, np.int64)
        for b in range(nb):                                   # every block adds its own histogram
            k = key[b * CH: (b + 1) * CH]
            if decided is not None:
                k = k[(k >> decided) == (prefix >> decided)]
            np.add.at(hist, (k >> shift) & (nbins - 1), 1)
        per = nbins // 256                                    # the last block: thread t owns buckets nbins-1-t*per .. downwards
        parts = [int(sum(hist[nbins - 1 - (t * per + j)] for j in range(per))) for t in range(256)]
        before, found = 0, False
        for t in range(256):
            if before < need and before + parts[t] >= need:
                n, bin_ = need - before, nbins - 1 - t * per
                for j in range(per):
                    m = int(hist[nbins - 1 - (t * per + j)])
                    if m >= n or j == per - 1:
                        break
                    n -= m
                    bin_ -= 1
                prefix, need, found = np.uint32(prefix | np.uint32(bin_ << shift)), int(n), True
                break
            before += parts[t]
        assert found
    T, quota = prefix, need
    gt = [int((key[b * CH: (b + 1) * CH] > T).sum()) for b in range(nb)]
    eq = [int((key[b * CH: (b + 1) * CH] == T).sum()) for b in range(nb)]
    eq_before, off, e, p = [0] * nb, [0] * nb, 0, 0
    for b in range(nb):                                       # the count pass's last block
        eq_before[b], off[b] = e, p
        p += gt[b] + min(eq[b], max(0, quota - e))
        e += eq[b]
    out = []
    for b in range(nb):                                       # emit: every block writes from its own offset
        r = eq_before[b]
        assert off[b] == len(out)
        for i in range(b * CH, min(ne, (b + 1) * CH)):
            if key[i] > T:
                out.append(i)
            elif key[i] == T:
                if r < quota:
                    out.append(i)
                r += 1
    return out


@pytest.mark.parametrize("ne,budget,kind", [(10000, 512, "normal"), (262144, 512, "normal"), (50000, 512, "relu"), (9000, 2048, "normal"),
                                            (3000, 512, "const"), (70001, 512, "relu"), (2049, 2048, "normal"), (4096, 1, "normal")])
def test_split_selection_equals_a_stable_sort(ne, budget, kind):
    rng = np.random.default_rng(ne + budget)
    sc = rng.standard_normal(ne).astype(np.float32)
    if kind == "relu":
        sc = np.maximum(sc - 2.5, 0)
    elif kind == "const":
        sc[:] = 1.0
    got = split_topk(sc, ne, budget)
    want = sorted(np.lexsort((np.arange(ne), -sc.astype(np.float64)))[:budget].tolist())
    assert got == want
