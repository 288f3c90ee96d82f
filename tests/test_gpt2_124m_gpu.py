"""The benchmark's own size (GPT-2 124M: 12 layers, width 768, 12 heads of 64, vocabulary
50,257) with random weights: logits in float32 and in bfloat16 against the plain implementation
in all four cuttings (whole, the last 32 tokens one by one, portions, mixed in few pages). At
this size the products run as CTA pairs or cluster split-K, attention on tcgen05, and the
logits over a vocabulary that is no multiple of anything."""

from __future__ import annotations

import pytest

from tests import traces
from tests.helpers import make_model_dir, random_tokens
from tests.test_replay_gpu import compare, round64, run_trace

pytestmark = pytest.mark.gpu

GPT2_124M = {
    "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2", "n_layer": 12, "n_embd": 768, "n_head": 12,
    "n_inner": 3072, "vocab_size": 50257, "n_positions": 1024, "activation_function": "gelu_new",
    "layer_norm_epsilon": 1e-5, "scale_attn_weights": True, "scale_attn_by_inverse_layer_idx": False,
    "tie_word_embeddings": True, "eos_token_id": None,
}


@pytest.fixture(scope="module")
def folder_124m(tmp_path_factory):
    return make_model_dir(tmp_path_factory.mktemp("gpt2_124m"), {"config": GPT2_124M, "seed": 5, "std": 0.02, "store_dtype": "float32"})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gpt2_124m_in_all_four_cuttings(folder_124m, dtype):
    requests = {f"r{i}": random_tokens(500 + i, n, GPT2_124M["vocab_size"]) for i, n in enumerate((130, 40, 9, 200))}
    cuttings = {"whole": (traces.whole(requests), 1), "decode32": (traces.prefill_then_decode(requests, 32), 1),
                "portions": (traces.portions(requests), 1), "mixed": (traces.mixed(requests, max_live=4), 4)}
    for mode, (tb, live) in cuttings.items():
        biggest = sorted((round64(len(v)) for v in requests.values()), reverse=True)[:live]
        outputs = run_trace(folder_124m, tb, dtype, sum(biggest), 16)
        compare(folder_124m, requests, tb, outputs, dtype, f"124M/{dtype}/{mode}")
