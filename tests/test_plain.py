"""The plain implementation itself (no GPU): against the reference's own GPT-2 forward and
sampler (outputs committed under tests/golden/, made by tests/golden/make_golden.py), against
float64, and part by part against torch's functions."""

from __future__ import annotations

import json
import math
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from tests.helpers import TINY_A, TINY_B, plain_logits
from tests.plain import gpt2_plain as plain

GOLDEN = json.loads((Path(__file__).parent / "golden" / "gpt2_tiny_a.json").read_text())


def test_forward_matches_the_references_own_forward(tiny_a_dir):
    ids = GOLDEN["ids"]
    ours = plain_logits(tiny_a_dir, ids, "float32")
    for row in GOLDEN["rows"]:
        want = np.asarray(row["logits"], dtype=np.float32)
        got = ours[row["n"] - 1]
        assert np.abs(got - want).max() < 2e-6, (row["n"], np.abs(got - want).max())


def test_philox_uniforms_are_the_references_bits():
    key = tuple(GOLDEN["philox_key"])
    want = GOLDEN["philox_uniform_rows0to2_tokens0to7"]
    for row in range(3):
        for token in range(8):
            assert plain.uniform_for(row, token, key) == want[row][token]


def test_draws_match_the_references_sampler():
    key = tuple(GOLDEN["philox_key"])
    logits = torch.tensor(GOLDEN["rows"][-1]["logits"])
    for draw in GOLDEN["draws_at_row0"]:
        got = plain.sample_token(logits, draw["temperature"], draw["top_k"], key, position=0)
        assert got == draw["token"], draw


def test_float32_agrees_with_float64(tiny_a_dir, tiny_b_dir):
    for folder, tiny in ((tiny_a_dir, TINY_A), (tiny_b_dir, TINY_B)):
        gen = torch.Generator().manual_seed(9)
        ids = torch.randint(0, tiny["config"]["vocab_size"], (50,), generator=gen).tolist()
        a, b = plain_logits(folder, ids, "float32"), plain_logits(folder, ids, "float64")
        assert np.abs(a - b).max() < 1e-4 * max(1.0, np.abs(b).max())


def test_layer_norm_and_activations_against_torch():
    x = torch.randn(5, 96, dtype=torch.float64)
    g, b = torch.randn(96, dtype=torch.float64), torch.randn(96, dtype=torch.float64)
    assert torch.allclose(plain.layer_norm(x, g, b, 1e-6), F.layer_norm(x, (96,), g, b, 1e-6), atol=1e-12)
    assert torch.allclose(plain.gelu_new(x), F.gelu(x, approximate="tanh"), atol=1e-12)
    assert torch.allclose(plain.gelu_erf(x), F.gelu(x), atol=1e-12)


def test_attention_is_causal_windowed_and_grouped():
    torch.manual_seed(0)
    t, h, hkv, hd = 9, 4, 2, 16
    q, k, v = torch.randn(t, h, hd), torch.randn(t, hkv, hd), torch.randn(t, hkv, hd)
    out = plain.causal_attention(q, k, v, hd**-0.5).reshape(t, h, hd)
    # row 0 sees only key 0: its output is v[0] of its kv head
    assert torch.allclose(out[0, 3], v[0, 1], atol=1e-6) and torch.allclose(out[0, 0], v[0, 0], atol=1e-6)
    # changing a future key or value changes nothing before it
    k2, v2 = k.clone(), v.clone()
    k2[5:], v2[5:] = 7.0, -3.0
    out2 = plain.causal_attention(q, k2, v2, hd**-0.5).reshape(t, h, hd)
    assert torch.equal(out[:5], out2[:5]) and not torch.allclose(out[5:], out2[5:])
    # a window of 3: row 8 equals full attention over rows 6..8 alone
    win = plain.causal_attention(q, k, v, hd**-0.5, window=3).reshape(t, h, hd)
    tail = plain.causal_attention(q[6:], k[6:], v[6:], hd**-0.5).reshape(3, h, hd)
    assert torch.allclose(win[8], tail[2], atol=1e-6)
    # against torch's own attention
    ref = F.scaled_dot_product_attention(q.transpose(0, 1), k.repeat_interleave(2, 1).transpose(0, 1),
                                         v.repeat_interleave(2, 1).transpose(0, 1), is_causal=True).transpose(0, 1)
    assert torch.allclose(out, ref, atol=1e-5)


def test_attention_scale_options():
    assert plain.attention_scale(64, 0, True, False) == pytest.approx(0.125)
    assert plain.attention_scale(64, 2, True, True) == pytest.approx(0.125 / 3)
    assert plain.attention_scale(64, 2, False, True) == pytest.approx(1 / 3)


def test_sampling_rules():
    logits = torch.tensor([0.1, 2.0, 2.0, -1.0, 1.9])
    assert plain.sample_token(logits, 0.0, 0, (1, 2), 5) == 1  # greedy, first index on ties
    assert plain.sample_token(logits, 0.9, 1, (1, 2), 5) == 1  # top_k 1 is greedy
    seen = {plain.sample_token(logits, 1.0, 3, (7, s), s) for s in range(200)}
    assert seen <= {1, 2, 4} and len(seen) == 3  # the three largest, ties kept in
    seen = {plain.sample_token(logits, 5.0, 0, (7, s), s) for s in range(300)}
    assert seen == {0, 1, 2, 3, 4}
    u = plain.uniform_for(3, 4, (5, 6))
    assert 0.0 < u < 1.0 and u == plain.uniform_for(3, 4, (5, 6)) and u != plain.uniform_for(4, 4, (5, 6))


def test_generate_stops(tiny_a_dir):
    w, cfg = plain.read_model(tiny_a_dir)
    out = plain.generate(w, cfg, [1, 2, 3], 5)
    assert len(out) == 5
    assert plain.generate(w, cfg, [1, 2, 3], 0) == out[:1]
    assert plain.generate(w, cfg, [1, 2, 3], 5, stop_token_ids=(out[2],))[-1] == out[2]
    assert math.isfinite(float(plain.forward(w, cfg, torch.tensor([1, 2, 3])).sum()))
