"""Makes tests/golden/gpt2_tiny_a.json: the reference's own GPT-2 forward and sampler on a tiny
random model, for comparison with the plain implementation (tests/plain/gpt2_plain.py).

Run once, on the CPU, where the reference tree is mounted:

    python tests/golden/make_golden.py PATH_OF_THE_REFERENCE_TREE

It imports `kelpie_models.models.torch.gpt2` and `kelpie_models.kernels.ops.sample` from the
reference's source tree (no native library is needed: the ops run their torch bodies), builds
the tiny-A model of tests/helpers.py with this repository's random-weights writer, and runs
`gpt2.forward` on growing prefixes of one sequence with hand-made plan views. The reference's
forward returns the last row only (models/torch/gpt2.py:98-101), so position p comes from the
prefix of length p + 1. The reference model has no exact-erf GELU and no inverse-layer scaling,
so tiny B's options rest on the formulas alone.
"""

from __future__ import annotations

import json
import sys
import tempfile
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))


def main(reference_root: str) -> None:
    sys.path[:0] = [f"{reference_root}/kelpie/kelpie-models", f"{reference_root}/kelpie/kelpie-engine"]
    from kelpie_models.kernels.ops.sample import philox_uniform, sample
    from kelpie_models.models.torch import gpt2
    from kelpie_models.sdk.device import Host, Requests, Tokens
    from kelpie_models.sdk.groups import FullAttn
    from kelpie_models.sdk.taps import taps_for

    from tests.helpers import TINY_A, make_model_dir, random_tokens
    from tests.plain import gpt2_plain

    with tempfile.TemporaryDirectory() as tmp:
        folder = make_model_dir(Path(tmp) / "a", TINY_A)
        w, cfg = gpt2_plain.read_model(folder, torch.float32)
    c = TINY_A["config"]
    hd = c["n_embd"] // c["n_head"]
    rcfg = gpt2.GPT2Config(c["n_layer"], c["n_head"], c["n_embd"], c["vocab_size"], c["n_positions"],
                           c["layer_norm_epsilon"], c["eos_token_id"])
    layers = tuple(
        gpt2.Layer(FullAttn(c["n_head"], hd),
                   gpt2.Norm(w[f"h.{i}.ln_1.weight"], w[f"h.{i}.ln_1.bias"]),
                   gpt2.Linear(w[f"h.{i}.attn.c_attn.weight"], w[f"h.{i}.attn.c_attn.bias"]),
                   gpt2.Linear(w[f"h.{i}.attn.c_proj.weight"], w[f"h.{i}.attn.c_proj.bias"]),
                   gpt2.Norm(w[f"h.{i}.ln_2.weight"], w[f"h.{i}.ln_2.bias"]),
                   gpt2.Linear(w[f"h.{i}.mlp.c_fc.weight"], w[f"h.{i}.mlp.c_fc.bias"]),
                   gpt2.Linear(w[f"h.{i}.mlp.c_proj.weight"], w[f"h.{i}.mlp.c_proj.bias"]))
        for i in range(c["n_layer"]))
    rw = gpt2.GPT2(w["wte.weight"], w["wpe.weight"], layers, gpt2.Norm(w["ln_f.weight"], w["ln_f.bias"]))
    ids = random_tokens(42, 24, c["vocab_size"])
    block, pages = 16, 4
    rows = []
    for n in (1, 2, 7, 16, 17, 24):
        kv = [tuple(torch.zeros(pages, block, 2, c["n_head"], hd).permute(0, 2, 1, 3, 4) for _ in range(c["n_layer"]))]
        pos = torch.arange(n, dtype=torch.int32)
        table = torch.tensor([[1, 2, 3, 0]], dtype=torch.int32)
        slots = (table[0, (pos // block).long()] * block + pos % block).to(torch.int32)
        tok = Tokens(input_ids=torch.tensor(ids[:n], dtype=torch.int32), positions=pos,
                     row_request=torch.zeros(n, dtype=torch.int32), last_rows=torch.tensor([n - 1], dtype=torch.int32),
                     tail_rows=torch.tensor([[n - 1]]))
        req = Requests(query_start_loc=torch.tensor([0, n], dtype=torch.int32), seq_lens=torch.tensor([n], dtype=torch.int32),
                       slot_mapping=(slots,), block_tables=(table,), kind=torch.zeros(1, dtype=torch.int32),
                       n_extra=torch.zeros(1, dtype=torch.int32), host=Host(1, n, (0, n), (n,), (0,)))
        logits = gpt2.forward(rw, rcfg, tok, req, kv, taps_for(()))[0, 0]
        rows.append({"n": n, "logits": [float(v) for v in logits]})
    key = torch.tensor([123, 456], dtype=torch.uint32)
    uniforms = philox_uniform(key, 3, 8)
    lg = torch.tensor(rows[-1]["logits"])[None, None, :]
    draws = []
    for top_k, temp in ((0, 0.8), (5, 1.3), (1, 1.0)):
        tok = sample(lg, torch.tensor([temp]), torch.tensor([top_k], dtype=torch.int32), key,
                     torch.full((1, 0), -1, dtype=torch.int32), False, top_k if top_k > 1 else 0)
        draws.append({"top_k": top_k, "temperature": temp, "token": int(tok[0, 0])})
    out = {
        "made_by": "tests/golden/make_golden.py", "ids": ids, "rows": rows, "philox_key": [123, 456],
        "philox_uniform_rows0to2_tokens0to7": [[float(v) for v in r] for r in uniforms],
        "draws_at_row0": draws,
    }
    (Path(__file__).parent / "gpt2_tiny_a.json").write_text(json.dumps(out))
    print("wrote", Path(__file__).parent / "gpt2_tiny_a.json")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py PATH_OF_THE_REFERENCE_TREE")
    main(sys.argv[1])
