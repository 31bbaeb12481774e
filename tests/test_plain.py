"""The plain implementation against the outputs of the reference's own model
code (tests/golden/, made by tests/golden/make_golden.py) and against itself."""
import os

import numpy as np
import pytest
import torch

import fixtures
import plain_llama
from golden.make_golden import CASES

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", sorted(CASES))
def test_plain_matches_reference_model(name):
    cfg, seed, std, norm_std, gain, ids_seed, n = CASES[name]
    data = np.load(os.path.join(GOLDEN, name + ".npz"))
    ids = data["ids"].tolist()
    assert ids == fixtures.random_ids(cfg, n, ids_seed)
    w = fixtures.make_weights(cfg, seed, std, norm_std, gain)
    logits = plain_llama.plain_forward(cfg, w, ids)
    ref = torch.from_numpy(data["logits"])
    assert logits.shape == ref.shape
    torch.testing.assert_close(logits, ref, atol=2e-5, rtol=1e-5)


def test_prefix_does_not_see_the_future():
    cfg = fixtures.TINY_B
    w = fixtures.make_weights(cfg, 3, 0.05, 0.1, 4.0)
    ids = fixtures.random_ids(cfg, 40, 7)
    whole = plain_llama.plain_forward(cfg, w, ids)
    part = plain_llama.plain_forward(cfg, w, ids[:13])
    torch.testing.assert_close(whole[:13], part, atol=1e-5, rtol=1e-5)


def test_llama3_scaling_bands():
    f = plain_llama.plain_inv_freq(32, 500000.0, None)
    s = plain_llama.plain_inv_freq(32, 500000.0, fixtures.TINY_B["rope_scaling"])
    wavelen = 2 * torch.pi / f
    assert torch.equal(s[wavelen < 8], f[wavelen < 8])          # orig/high = 8
    torch.testing.assert_close(s[wavelen > 32], f[wavelen > 32] / 4.0)
    mid = (wavelen >= 8) & (wavelen <= 32)
    assert mid.any() and (s[mid] <= f[mid]).all() and (s[mid] >= f[mid] / 4.0).all()


# Scaled frequencies computed once with 50-digit decimal arithmetic from the meaning of the config.json keys
# (wavelength 2 pi / f against original_max / high_freq_factor and original_max / low_freq_factor; between them a
# blend that is linear in original_max / wavelength): for every setting the last frequency that is kept, the first
# and the last that are blended, the first and the last that are divided by the factor.  The reference has no
# scaled frequencies to compare with (python/lyapunov_engine/models/llama.py:180-184 builds the plain ones), and
# model code of installed packages is no source for this suite, so these numbers are the pin.
LLAMA3_PINS = {
    # (head_dim, theta, factor, low, high, original_max): {j: scaled f_j}
    (64, 500000.0, 32.0, 1.0, 4.0, 8192): {14: 0.003211445994752591, 15: 0.0012905479282092638,
                                           17: 9.708287802627673e-05, 18: 1.9461638184831125e-05,
                                           31: 9.41830672543491e-08},
    (128, 500000.0, 8.0, 1.0, 4.0, 8192): {28: 0.003211445994752591, 29: 0.0021665707635033587,
                                           34: 0.0001785078127679964, 35: 9.556212353964683e-05,
                                           63: 3.068925988914511e-07},
    (32, 500000.0, 4.0, 1.0, 4.0, 32): {0: 1.0, 1: 0.24691010723760984, 2: 0.04848068618717144,
                                        15: 1.1354176201519674e-06},
    (64, 500000.0, 8.0, 1.0, 4.0, 256): {5: 0.12868737343265052, 6: 0.0724300351649636, 9: 0.0032415243211269965,
                                         10: 0.002070055010124306, 31: 3.767322690173964e-07},
}


@pytest.mark.parametrize("setting", sorted(LLAMA3_PINS))
def test_llama3_scaling_pinned_values(setting):
    """Llama-3.2-1B (factor 32), Llama-3.1-8B (factor 8), tiny-B and tiny-C."""
    from lyapunov_engine_b200.parts.rope import inverse_frequencies

    hd, theta, factor, low, high, original = setting
    scaling = {"rope_type": "llama3", "factor": factor, "low_freq_factor": low, "high_freq_factor": high,
               "original_max_position_embeddings": original}
    for what, got in (("plain", plain_llama.plain_inv_freq(hd, theta, scaling)),
                      ("engine", inverse_frequencies(hd, theta, scaling))):
        assert got.dtype == torch.float32 and got.shape == (hd // 2,)
        for j, expected in LLAMA3_PINS[setting].items():
            assert abs(float(got[j]) - expected) <= 1e-6 * expected, (what, setting, j, float(got[j]), expected)
    assert fixtures.TINY_B["rope_scaling"]["original_max_position_embeddings"] == 32       # the pins' settings are
    assert fixtures.TINY_C["rope_scaling"]["factor"] == 8.0                                # the fixtures'


def test_bfloat16_bounds_tell_the_models_apart():
    """The bounds the bfloat16 replay tests use (in units of measured rounding
    noise) are met by a second evaluation of the bfloat16 pipeline and failed
    by the float32 model's logits, and by a sequence whose first two tokens
    are swapped."""
    import numpy as np
    import replay_util as ru

    for cfg, seed, std, norm_std, gain in ((fixtures.TINY_A, 0, 0.05, 0.0, 4.0), (fixtures.TINY_B, 1, 0.05, 0.1, 3.0)):
        w = fixtures.make_weights(cfg, seed, std, norm_std, gain)
        requests = {f"r{i}": fixtures.random_ids(cfg, n, 100 + i) for i, n in enumerate((21, 33, 49, 70))}
        ref, noise = ru.bf16_references(cfg, w, requests, plain_llama.plain_forward)
        rounded = {k: v.to(torch.bfloat16).float() for k, v in w.items()}

        def as_replay(logits):
            return {(r, p): logits[r][p].numpy() for r in logits for p in range(logits[r].shape[0])}

        # another valid evaluation: 64-bit sums, numerators scaled by another bound
        wide = {k: v.double() for k, v in rounded.items()}
        other = {r: plain_llama.plain_forward(cfg, wide, ids, act_dtype=torch.bfloat16, prob_dtype=torch.bfloat16,
                                              prob_shift=1.7).float() for r, ids in requests.items()}
        assert ru.compare_bf16(as_replay(other), ref, noise, "another evaluation") <= 1.1
        # the float32 model is not the bfloat16 model
        full = {r: plain_llama.plain_forward(cfg, w, ids) for r, ids in requests.items()}
        with pytest.raises(AssertionError):
            ru.compare_bf16(as_replay(full), ref, noise, "float32 model")
        # one request with its first two tokens swapped
        ids = list(requests["r2"])
        ids[0], ids[1] = ids[1], ids[0] if ids[0] != ids[1] else (ids[0] + 1) % cfg["vocab_size"]
        wrong = dict(ref, r2=plain_llama.plain_forward(cfg, rounded, ids, act_dtype=torch.bfloat16, prob_dtype=torch.bfloat16))
        with pytest.raises(AssertionError):
            ru.compare_bf16({k: v for k, v in as_replay(wrong).items() if k[1] >= 2}, ref, noise, "swapped tokens")
        assert np.isfinite(noise["rms"]) and noise["rms"] > 0


def test_window_masks_far_keys():
    g = torch.Generator().manual_seed(0)
    q = torch.randn(2, 9, 16, generator=g)
    k = torch.randn(1, 9, 16, generator=g)
    v = torch.randn(1, 9, 16, generator=g)
    full = plain_llama.plain_attention(q, k, v)
    win = plain_llama.plain_attention(q, k, v, window=3)
    torch.testing.assert_close(full[:, :3], win[:, :3])
    again = plain_llama.plain_attention(q[:, 6:9], k[:, 6:9], v[:, 6:9])
    torch.testing.assert_close(win[:, 8], again[:, 2])


def test_filtered_probs():
    logits = torch.tensor([2.0, 1.0, 0.0, -1.0, 3.0])
    p = plain_llama.plain_filtered_probs(logits, 1.0, 2, 1.0)
    assert (p > 0).tolist() == [True, False, False, False, True]
    p = plain_llama.plain_filtered_probs(logits, 1.0, -1, 0.7)
    # sorted probs .636 .234 .086 ...: the first exceeds nothing, the second's
    # predecessor mass .636 <= .7 so it stays, the third's .870 > .7 goes.
    assert (p > 0).tolist() == [True, False, False, False, True]
    assert abs(p.sum().item() - 1.0) < 1e-12
    assert plain_llama.plain_greedy(torch.tensor([1.0, 5.0, 5.0])) == 1
