"""KDA math against the reference's published golden fixture (test-data/kda-goldens, case A "synth": all inputs come from a
documented splitmix64 stream, the expected outputs are a float32 transcription of the recurrent gated-delta-rule kernel).
The inputs are regenerated here from the fixture's PRNG specification; a sample of its expected values is embedded below
(the full tensors agree with this implementation to 2e-7 relative for the recurrence and 7e-7 for the chunk-parallel form)."""
import numpy as np
import torch

from layerstorm_b200.models.kda_chunked import kda_chunk_prepare, kda_chunk_scan, kda_chunked, kda_sequential

T, TP, H, D = 152, 144, 4, 128

CORE = [((122, 2, 50), -7.314036338357255e-05), ((91, 2, 109), -0.0023092261981219053), ((73, 3, 70), -0.00044122818508185446),
        ((38, 2, 4), 7.071017171256244e-05), ((44, 2, 97), 0.0004660864360630512), ((5, 2, 93), -0.0006062852335162461),
        ((10, 2, 108), 6.569499964825809e-05), ((2, 3, 22), -0.00019305513706058264), ((25, 1, 11), -4.739457290270366e-05),
        ((117, 3, 110), -0.0006079330341890454), ((93, 2, 2), -4.827561497222632e-06), ((131, 0, 69), -0.0016611681785434484)]
STATE = [((0, 1, 58), 0.028165632858872414), ((1, 85, 127), 0.005276092793792486), ((1, 67, 103), -0.00833061896264553),
         ((1, 82, 125), -0.0012862163130193949), ((1, 32, 48), 0.00916201900690794), ((0, 78, 87), 0.001244292943738401),
         ((0, 97, 121), 0.00355361495167017), ((0, 49, 83), 0.0005374153261072934)]
ONORM = [((121, 2, 54), -0.020461153239011765), ((99, 2, 62), 0.027674272656440735), ((101, 3, 92), 0.17254222929477692),
         ((56, 2, 113), 0.0031262573320418596), ((126, 1, 9), -0.00044056170736439526), ((19, 1, 119), -0.00786260049790144)]
DECODE = [((4, 1, 64), -0.0008035469800233841), ((2, 1, 43), -0.0008629486546851695), ((5, 2, 97), -0.0005756797036156058),
          ((4, 2, 50), 0.00011680115130729973)]


def _splitmix(seed: int, n: int) -> np.ndarray:
    with np.errstate(over="ignore"):
        s = np.uint64(seed) + (np.arange(1, n + 1, dtype=np.uint64) * np.uint64(0x9E3779B97F4A7C15))
        z = (s ^ (s >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def _bf16_round(x: np.ndarray) -> np.ndarray:
    u = x.astype(np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + np.uint64(0x7FFF) + ((u >> np.uint64(16)) & np.uint64(1))) & np.uint64(0xFFFFFFFF)) & np.uint64(0xFFFF0000)
    return r.astype(np.uint32).view(np.float32)


def _stream(seed, shape, lo, hi, bf16):
    r = _splitmix(seed, int(np.prod(shape)))
    u01 = ((r >> np.uint64(40)).astype(np.float64) * (1.0 / 16777216.0)).astype(np.float32)
    x = (lo + (hi - lo) * u01.astype(np.float64)).astype(np.float32)
    return torch.from_numpy((_bf16_round(x) if bf16 else x).reshape(shape).copy())


def _case_a():
    raw = {n: _stream(s, (T, H, D), lo, hi, True) for n, s, lo, hi in (("q", 101, -1, 1), ("k", 102, -1, 1), ("v", 103, -1, 1), ("g", 104, -3, 3), ("g2", 105, -2, 2))}
    beta_raw = _stream(106, (T, H), -2, 2, True)
    a_log, dt_bias = _stream(107, (H,), -1, 1.5, False), _stream(108, (H, D), -1, 1, False)
    conv_w = [_stream(s, (H * D, 4), -0.5, 0.5, True) for s in (109, 110, 111)]
    onorm_w, S0 = _stream(112, (D,), 0.5, 1.5, True), _stream(113, (H, D, D), -1, 1, False)
    conv_state = [_stream(s, (H * D, 3), -1, 1, True) for s in (114, 115, 116)]

    def conv_silu(x, w, st):
        hist = torch.cat([st.T, x.reshape(T, H * D)], 0)                        # three rows of history, oldest first
        acc = torch.zeros(T, H * D)
        for j in range(4):
            acc = acc + hist[j: j + T] * w[:, j][None]
        return torch.nn.functional.silu(acc).view(T, H, D)

    q, k, v = (conv_silu(raw[n], conv_w[i], conv_state[i]) for i, n in enumerate(("q", "k", "v")))
    qn = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    kn = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    decay = torch.exp(-5.0 * torch.sigmoid(torch.exp(a_log)[None, :, None] * (raw["g"] + dt_bias[None])))
    return raw, qn, kn, v, torch.sigmoid(beta_raw), decay, S0, onorm_w


def _check(got, samples, rtol):
    for idx, want in samples:
        assert abs(float(got[idx]) - want) <= rtol * abs(want) + 1e-9, (idx, float(got[idx]), want)


def test_prng_matches_the_fixture_specification():
    assert [int(x) for x in _splitmix(101, 4)] == [15060681878671775511, 317125338075985571, 4955761374856264282, 10230203001953340975]
    q_raw = _stream(101, (T, H, D), -1, 1, True)
    assert [hex(int(v)) for v in q_raw.reshape(-1)[:4].numpy().view(np.uint32)] == ["0x3f220000", "0xbf770000", "0xbeed0000", "0x3de00000"]


def test_recurrence_and_chunked_forms_reproduce_the_golden_outputs():
    raw, qn, kn, v, beta, decay, S0, onorm_w = _case_a()
    core, S = kda_sequential(qn[:TP], kn[:TP], v[:TP], beta[:TP], decay[:TP], S0)
    _check(core, CORE, 2e-4)
    _check(S, STATE, 2e-4)
    onorm = core * torch.rsqrt(core.pow(2).mean(-1, keepdim=True) + 1e-5) * onorm_w[None, None] * torch.sigmoid(raw["g2"][:TP])
    _check(onorm, ONORM, 2e-4)
    dec, _ = kda_sequential(qn[TP:], kn[TP:], v[TP:], beta[TP:], decay[TP:], S)     # one continuous recurrence: decode continues the state
    _check(dec, DECODE, 2e-4)
    core_c, S_c = kda_chunked(qn[:TP], kn[:TP], v[:TP], beta[:TP], decay[:TP], S0, chunk=64, blockwise=True)
    _check(core_c, CORE, 5e-4)
    _check(S_c, STATE, 5e-4)
    core_p, S_p = kda_chunk_scan(kda_chunk_prepare(qn[:TP], kn[:TP], beta[:TP], decay[:TP], chunk=64), v[:TP], S0)
    assert (core_p - core).abs().max() < 1e-5 * core.abs().max() + 1e-9 and (S_p - S).abs().max() < 1e-5 * S.abs().max()
