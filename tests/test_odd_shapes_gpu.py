"""Configurations whose sizes are picked to be awkward: head sizes of 48 and 80 (steps of 16
that are no power of two), one head and five heads, widths and inner widths that are no
multiple of 64, an odd vocabulary, pages of 4, 12, 24 and 32 tokens. Each is replayed in portions
and mixed with other requests in a pool so small that pages are used again (asserted), in float32 and in bfloat16, against the plain
implementation: the kernels take every size that a configuration allows."""

from __future__ import annotations

import pytest

from tests import traces
from tests.helpers import make_model_dir, random_tokens
from tests.test_replay_gpu import compare, run_trace

pytestmark = pytest.mark.gpu


def config(n_layer, n_embd, n_head, n_inner, vocab, n_positions, act, eps, by_layer):
    return {
        "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2", "n_layer": n_layer, "n_embd": n_embd, "n_head": n_head,
        "n_inner": n_inner, "vocab_size": vocab, "n_positions": n_positions, "activation_function": act,
        "layer_norm_epsilon": eps, "scale_attn_weights": True, "scale_attn_by_inverse_layer_idx": by_layer,
        "tie_word_embeddings": True, "eos_token_id": None,
    }


ODD = {
    "one_head_of_48": {"config": config(2, 48, 1, 136, 301, 160, "gelu_new", 1e-5, False), "seed": 31, "std": 0.05,
                       "store_dtype": "bfloat16", "page_size": 4, "lengths": (70, 9, 131, 2, 60, 90)},
    "five_heads_of_80": {"config": config(1, 400, 5, 1000, 1203, 192, "gelu", 2e-6, True), "seed": 32, "std": 0.03,
                         "store_dtype": "float32", "page_size": 32, "lengths": (150, 33, 64, 3, 97)},
    "three_heads_of_16_width_no_multiple_of_64": {"config": config(3, 48, 3, 200, 65, 96, "gelu_new", 1e-5, True), "seed": 33,
                                                  "std": 0.08, "store_dtype": "bfloat16", "page_size": 16, "lengths": (96, 17, 40, 60)},
    # pages of 12 and of 24 tokens: no power of two, so positions are split into page and offset by division
    "pages_of_12_tokens": {"config": config(2, 64, 2, 160, 203, 128, "gelu_new", 1e-5, False), "seed": 34, "std": 0.05,
                           "store_dtype": "bfloat16", "page_size": 12, "lengths": (100, 13, 47, 128, 30)},
    "pages_of_24_tokens_heads_of_64": {"config": config(2, 128, 2, 320, 411, 320, "gelu", 1e-5, True), "seed": 35, "std": 0.04,
                                       "store_dtype": "bfloat16", "page_size": 24, "lengths": (150, 49, 24, 300, 71)},
}


@pytest.fixture(scope="module")
def odd_dirs(tmp_path_factory):
    return {name: make_model_dir(tmp_path_factory.mktemp(name), tiny) for name, tiny in ODD.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ODD))
@pytest.mark.parametrize("mode", ["portions", "mixed"])
def test_odd_shapes_replay(odd_dirs, name, dtype, mode):
    tiny, folder = ODD[name], odd_dirs[name]
    vocab = tiny["config"]["vocab_size"]
    requests = {f"r{i}": random_tokens(300 + i, n, vocab) for i, n in enumerate(tiny["lengths"])}
    tb = traces.portions(requests) if mode == "portions" else traces.mixed(requests, max_live=2)
    outputs = run_trace(folder, tb, dtype, tiny["page_size"], expect_reuse=mode == "mixed")
    compare(folder, requests, tb, outputs, dtype, f"{name}/{dtype}/{mode}")
