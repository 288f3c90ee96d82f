"""Two more toy parts, defined HERE and registered without a change to the framework's files:
a feed-forward that routes every row to one of two small experts, and a position encoding
that rotates queries and keys instead of adding a table row. They are toys and no model of
anyone's; they show that the registries, the layer list and the step function serve a
feed-forward with routing and another kind of position encoding, beside the stock attention,
LayerNorm and dense feed-forward, cut into steps like any other model."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from tests.plain import gpt2_plain as plain

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
D, V, F, HEADS, HD, THETA = 32, 97, 40, 2, 16, 100.0


def rotate_pairs(x, positions):
    """x [T, heads * HD] -> pairs (2i, 2i + 1) of every head turned by positions * THETA^(-2i / HD)."""
    t = x.shape[0]
    pairs = x.float().reshape(t, -1, HD // 2, 2)
    freq = THETA ** (-torch.arange(HD // 2, device=x.device, dtype=torch.float32) * 2 / HD)
    angle = positions.to(x.device, torch.float32)[:, None, None] * freq[None, None, :]
    cos, sin = torch.cos(angle), torch.sin(angle)
    a, b = pairs[..., 0], pairs[..., 1]
    return torch.stack((a * cos - b * sin, a * sin + b * cos), dim=-1).reshape(t, -1)


def register_toys():
    from research_2_b200.parts import register_feed_forward, register_positions

    @register_positions("toy_rotation")
    class Rotation:
        """No table: the position turns queries and keys inside every mixer that has a `rotary` slot."""

        rotates = True

        def __init__(self, params, weights, rt):
            pass

        def additive_table(self):
            return None

        def rotate(self, q, k, ctx):
            pos = ctx.positions[: q.shape[0]]
            q.copy_(rotate_pairs(q, pos).to(q.dtype))
            k.copy_(rotate_pairs(k, pos).to(k.dtype))

    @register_feed_forward("toy_two_experts")
    class TwoExperts:
        """Router logits in float32; every row goes to the expert with the larger logit, and its
        output is weighted by that expert's softmax probability. Experts: gelu_new(h w1) w2."""

        def __init__(self, params, weights, rt):
            self.gate = weights["gate"].to(rt.device, torch.float32)
            self.w1 = [weights[f"e{i}.w1"].to(rt.device, rt.dtype) for i in range(2)]
            self.w2 = [weights[f"e{i}.w2"].to(rt.device, rt.dtype) for i in range(2)]

        def forward(self, h, residual, ctx):
            from research_2_b200.kernels import ops

            h = h.materialize() if hasattr(h, "materialize") else h
            logits = h.float() @ self.gate
            prob = torch.softmax(logits, dim=-1)
            pick = logits.argmax(dim=-1)
            out = residual.clone()
            for e in range(2):
                rows = (pick == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                inner = ops.linear(h[rows].contiguous(), self.w1[e], None, act="gelu_new")
                y = ops.linear(inner, self.w2[e], None, out_dtype=torch.float32)
                out[rows] += y * prob[rows, e: e + 1]
            return out

    return Rotation, TwoExperts


def toy_model(dtype):
    from research_2_b200.models.decoder import DecoderModel, ModelSpec
    from research_2_b200.parts import LayerSpec, PartSpec, Runtime

    g = torch.Generator().manual_seed(21)

    def rnd(*shape, s=0.2):
        return torch.randn(*shape, generator=g) * s

    tensors = {"emb": rnd(V, D, s=0.5), "nf.g": 1 + rnd(D), "nf.b": rnd(D), "gate": rnd(D, 2, s=1.0)}
    for e in range(2):
        tensors.update({f"e{e}.w1": rnd(D, F), f"e{e}.w2": rnd(F, D)})
    for i in range(2):
        tensors.update({f"l{i}.n1.g": 1 + rnd(D), f"l{i}.n1.b": rnd(D), f"l{i}.n2.g": 1 + rnd(D), f"l{i}.n2.b": rnd(D),
                        f"l{i}.qkv.w": rnd(D, 3 * D), f"l{i}.qkv.b": rnd(3 * D), f"l{i}.o.w": rnd(D, D), f"l{i}.o.b": rnd(D)})
    tensors.update({"l1.fc.w": rnd(D, F), "l1.fc.b": rnd(F), "l1.pr.w": rnd(F, D), "l1.pr.b": rnd(D)})

    def layer(i, feed_forward):
        return LayerSpec(
            block="pre_norm",
            mixer=PartSpec("attention", {"n_heads": HEADS, "n_kv_heads": HEADS, "head_dim": HD, "scale": 0.25, "window": 0},
                           {"w_qkv": f"l{i}.qkv.w", "b_qkv": f"l{i}.qkv.b", "w_out": f"l{i}.o.w", "b_out": f"l{i}.o.b"}),
            norm_1=PartSpec("layer_norm", {"eps": 1e-5}, {"gamma": f"l{i}.n1.g", "beta": f"l{i}.n1.b"}),
            norm_2=PartSpec("layer_norm", {"eps": 1e-5}, {"gamma": f"l{i}.n2.g", "beta": f"l{i}.n2.b"}),
            feed_forward=feed_forward)

    experts = PartSpec("toy_two_experts", {}, {"gate": "gate", "e0.w1": "e0.w1", "e0.w2": "e0.w2", "e1.w1": "e1.w1", "e1.w2": "e1.w2"})
    dense_ff = PartSpec("mlp", {"activation": "gelu_new"}, {"w_in": "l1.fc.w", "b_in": "l1.fc.b", "w_out": "l1.pr.w", "b_out": "l1.pr.b"})
    spec = ModelSpec(
        vocab_size=V, hidden=D, max_seq_len=64, eos_token=None, embedding="emb", head="emb",
        positions=PartSpec("toy_rotation", {}, {}),
        layers=(layer(0, experts), layer(1, dense_ff)),
        final_norm=PartSpec("layer_norm", {"eps": 1e-5}, {"gamma": "nf.g", "beta": "nf.b"}))
    return DecoderModel(spec, tensors, Runtime(DEV, dtype)), tensors


def dense(tensors, ids):
    """The same model as a plain statement over a whole sequence."""
    n = len(ids)
    pos = torch.arange(n)
    x = plain.embed_tokens(torch.tensor(ids), tensors["emb"])
    for i in range(2):
        h = plain.layer_norm(x, tensors[f"l{i}.n1.g"], tensors[f"l{i}.n1.b"], 1e-5)
        q, k, v = plain.linear(h, tensors[f"l{i}.qkv.w"], tensors[f"l{i}.qkv.b"]).split(D, -1)
        q, k = rotate_pairs(q, pos), rotate_pairs(k, pos)
        mixed = plain.causal_attention(q.reshape(n, HEADS, HD), k.reshape(n, HEADS, HD), v.reshape(n, HEADS, HD), 0.25)
        x = x + plain.linear(mixed, tensors[f"l{i}.o.w"], tensors[f"l{i}.o.b"])
        h = plain.layer_norm(x, tensors[f"l{i}.n2.g"], tensors[f"l{i}.n2.b"], 1e-5)
        if i == 0:
            logits = h @ tensors["gate"]
            prob, pick = torch.softmax(logits, -1), logits.argmax(-1)
            y = torch.stack([plain.gelu_new(h[t] @ tensors[f"e{int(pick[t])}.w1"]) @ tensors[f"e{int(pick[t])}.w2"] * prob[t, pick[t]]
                             for t in range(n)])
            x = x + y
        else:
            x = x + plain.linear(plain.gelu_new(plain.linear(h, tensors["l1.fc.w"], tensors["l1.fc.b"])), tensors["l1.pr.w"], tensors["l1.pr.b"])
    return plain.tied_head(plain.layer_norm(x, tensors["nf.g"], tensors["nf.b"], 1e-5), tensors["emb"]).numpy()


def run_in_steps(model, seqs, plan):
    from research_2_b200.cache.manager import CacheManager
    from research_2_b200.engine.step import StepFunction

    step_fn = StepFunction(model, 8, 16, 3, capture=False)
    cache = CacheManager(step_fn.cache_groups(), 3, 64)
    step_fn.arena.fill_(64.0)
    got, fed = {r: [] for r in seqs}, {r: 0 for r in seqs}
    for r in seqs:
        cache.open(r)
    for step in plan:
        reqs, starts, toks = [], [], []
        for r, n in step:
            cache.reserve(r, fed[r], fed[r] + n)
            reqs.append(r); starts.append(fed[r]); toks.append(seqs[r][fed[r]: fed[r] + n])
        total = sum(len(t) for t in toks)
        batch = step_fn.new_batch(total, len(reqs), total)
        batch.set_entries(reqs, starts, toks)
        cache.fill(batch)
        batch.set_logit_rows(list(range(total)))
        logits = step_fn(batch).cpu().numpy()
        at = 0
        for r, n in step:
            got[r].append(logits[at: at + n])
            at += n
            fed[r] += n
    assert all(fed[r] == len(ids) for r, ids in seqs.items())
    return {r: np.concatenate(got[r]) for r in seqs}


@pytest.mark.parametrize("dtype,tolerance", [(torch.float32, 3e-4), (torch.bfloat16, 5e-2)])
def test_routed_feed_forward_and_rotating_positions_are_registered_built_and_stepped(dtype, tolerance):
    from research_2_b200.parts import registry

    register_toys()
    assert "toy_two_experts" in registry("feed_forward") and "toy_rotation" in registry("positions")
    model, tensors = toy_model(dtype)
    assert all(block.mixer.rotary is model.positions for block in model.blocks), "the rotation was not attached to the mixers"
    seqs = {0: torch.randint(0, V, (37,), generator=torch.Generator().manual_seed(4)).tolist(),
            1: torch.randint(0, V, (22,), generator=torch.Generator().manual_seed(5)).tolist()}
    want = {r: dense(tensors, ids) for r, ids in seqs.items()}
    # both experts are in use, or the routing is not tested
    h = plain.layer_norm(plain.embed_tokens(torch.tensor(seqs[0]), tensors["emb"]), tensors["l0.n2.g"], tensors["l0.n2.b"], 1e-5)
    assert len(set((h @ tensors["gate"]).argmax(-1).tolist())) == 2
    plan = [[(0, 11), (1, 2)], [(1, 9), (0, 1)], [(0, 1), (1, 1)], [(0, 24)], [(1, 10)]]
    got = run_in_steps(model, seqs, plan)
    for r in seqs:
        scale = max(1.0, float(np.abs(want[r]).max()))
        assert np.abs(got[r] - want[r]).max() < tolerance * scale, (r, float(np.abs(got[r] - want[r]).max()))
    assert math.isfinite(float(np.abs(got[0]).sum()))
