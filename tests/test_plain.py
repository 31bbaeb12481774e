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
