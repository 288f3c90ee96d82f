"""The benchmark's own size (GPT-2 124M: 12 layers, width 768, 12 heads of 64, vocabulary
50,257) with random weights, and the layer sizes of the 355M and 1.5B models (two layers each:
width 1,024 with 16 heads; width 1,600 with 25 heads, which is no multiple of 128): logits in
float32 and in bfloat16 against the plain implementation in all four cuttings (whole, the last
32 tokens one by one, portions, mixed in a pool of the trace's peak demand plus one page, where pages are used again). At these sizes the products run as
cluster split-K or whole tiles, attention on tcgen05, and the logits over a vocabulary that is
no multiple of anything."""

from __future__ import annotations

import pytest

from tests import traces
from tests.helpers import make_model_dir, random_tokens
from tests.test_replay_gpu import compare, run_trace

pytestmark = pytest.mark.gpu

GPT2_124M = {
    "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2", "n_layer": 12, "n_embd": 768, "n_head": 12,
    "n_inner": 3072, "vocab_size": 50257, "n_positions": 1024, "activation_function": "gelu_new",
    "layer_norm_epsilon": 1e-5, "scale_attn_weights": True, "scale_attn_by_inverse_layer_idx": False,
    "tie_word_embeddings": True, "eos_token_id": None,
}


SIZES = {
    "124M": GPT2_124M,
    "355M_two_layers": dict(GPT2_124M, n_layer=2, n_embd=1024, n_head=16, n_inner=4096),
    "1.5B_two_layers": dict(GPT2_124M, n_layer=2, n_embd=1600, n_head=25, n_inner=6400),
}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def folder(size):
        if size not in made:
            made[size] = make_model_dir(tmp_path_factory.mktemp("gpt2_" + size.replace(".", "_")),
                                        {"config": SIZES[size], "seed": 5, "std": 0.02, "store_dtype": "float32"})
        return made[size]

    return folder


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("size", sorted(SIZES))
def test_gpt2_sizes_in_all_four_cuttings(folders, size, dtype):
    folder_124m = folders(size)
    requests = {f"r{i}": random_tokens(500 + i, n, GPT2_124M["vocab_size"]) for i, n in enumerate((130, 40, 9, 200, 70, 25))}
    cuttings = {"whole": traces.whole(requests), "decode32": traces.prefill_then_decode(requests, 32),
                "portions": traces.portions(requests), "mixed": traces.mixed(requests, max_live=3)}
    for mode, tb in cuttings.items():
        outputs = run_trace(folder_124m, tb, dtype, 16, expect_reuse=mode == "mixed")
        compare(folder_124m, requests, tb, outputs, dtype, f"{size}/{dtype}/{mode}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gpt2_124m_through_cuda_graphs(folders, dtype):
    """The benchmark's own size with every step run as the CUDA graph of its shape bucket (what
    bench.py and every bfloat16 user run): portions and mixed batches in recycled pages, the last
    token of every entry against the plain implementation."""
    folder = folders("124M")
    requests = {f"r{i}": random_tokens(500 + i, n, GPT2_124M["vocab_size"]) for i, n in enumerate((130, 40, 9, 200, 70, 25))}
    for mode, tb in (("portions", traces.portions(requests)), ("mixed", traces.mixed(requests, max_live=3)),
                     ("decode32", traces.prefill_then_decode(requests, 32))):
        tb = traces.with_last_only(tb)
        outputs = run_trace(folder, tb, dtype, 16, capture=True, expect_reuse=mode == "mixed")
        compare(folder, requests, tb, outputs, dtype, f"124M/{dtype}/{mode}/graphs", partial=True)
