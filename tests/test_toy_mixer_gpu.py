"""A toy mixer with state of its own, defined HERE, is registered, built and stepped without a
change to the framework's files: it keeps a running (decayed) sum of its inputs per request in
a state slot of fixed size, beside an ordinary attention layer with a paged cache. It is a toy
and no model of anyone's; it shows that the cache manager's state slots, the step function and
the layer schedule serve a mixer that is not attention."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from tests.plain import gpt2_plain as plain

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DECAY = 0.9


def register_toy():
    from research_2_b200.parts import StateSpec, register_mixer

    @register_mixer("toy_running_sum")
    class RunningSum:
        """y[t] = w * s[t], s[t] = DECAY * s[t - 1] + h[t], with s carried across steps in the
        request's state slot. Entries are folded in order, row by row, with torch ops."""

        def __init__(self, params, weights, rt):
            self.width = int(params["width"])
            self.w = weights["w"].to(rt.device, torch.float32)

        cache_spec = None
        capturable = False

        @property
        def state_spec(self):
            return StateSpec((self.width,), torch.float32)

        def forward(self, h, residual, ctx, cache, state, writes_cache=True):
            out = residual.clone()
            host = ctx.host
            for e in range(host.n_entries):
                a, b = int(host.q_start[e]), int(host.q_start[e + 1])
                slot = int(host.state_slot[e])
                s = torch.zeros(self.width, device=h.device) if host.fresh[e] else state[slot].clone()
                for t in range(a, b):
                    s = DECAY * s + h[t].float()
                    out[t] += self.w * s
                state[slot] = s
            return out

    return RunningSum


def register_toy_on_device():
    from research_2_b200.parts import StateSpec, register_mixer

    @register_mixer("toy_running_sum_on_device")
    class RunningSumOnDevice:
        """The same sum with nothing read on the host: rows of one entry are tied by a lower-triangular
        matrix of powers of DECAY, an entry's carried state comes in by its slot, and the last row of
        each entry writes it back. Every shape is the batch's capacity, padding rows (entry -1) and
        padding entries (no rows) change nothing: the part may be captured in a CUDA graph."""

        def __init__(self, params, weights, rt):
            self.width = int(params["width"])
            self.w = weights["w"].to(rt.device, torch.float32)
            self.decay = torch.tensor(DECAY, device=rt.device)   # (made here: a capture allows no copy from the host)

        cache_spec = None
        capturable = True

        @property
        def state_spec(self):
            return StateSpec((self.width,), torch.float32)

        def forward(self, h, residual, ctx, cache, state, writes_cache=True):
            n = h.shape[0]
            i = torch.arange(n, device=h.device)
            entry = ctx.row_entry.long()
            live = entry >= 0
            e = entry.clamp(min=0)
            q_start, slots = ctx.q_start.long(), ctx.state_slot.long()
            first, end = q_start[e], q_start[e + 1]
            tied = (entry[:, None] == entry[None, :]) & live[:, None] & (i[None, :] <= i[:, None])
            powers = torch.pow(self.decay, (i[:, None] - i[None, :]).clamp(min=0).float())
            lower = torch.where(tied, powers, torch.zeros_like(powers))
            carried = torch.where(ctx.fresh.bool()[:, None], torch.zeros_like(state[slots]), state[slots])   # per entry
            grown = torch.pow(self.decay, (i - first + 1).clamp(min=0).float())
            s = lower @ h.float() + (grown * live)[:, None] * carried[e]
            # the last row of each entry writes its slot: a 0/1 matrix [slot, row] instead of a scatter,
            # so that padding entries, which all name slot 0, write nothing
            last = live & (i + 1 == end)
            writes = (last[None, :] & (slots[e][None, :] == torch.arange(state.shape[0], device=h.device)[:, None])).float()
            state.copy_(state * (1 - writes.sum(1, keepdim=True)) + writes @ s)
            return residual + self.w * s

    return RunningSumOnDevice


def toy_model(dtype, mixer="toy_running_sum"):
    from research_2_b200.models.decoder import DecoderModel, ModelSpec
    from research_2_b200.parts import LayerSpec, PartSpec, Runtime

    d, v, f = 32, 101, 48
    g = torch.Generator().manual_seed(8)

    def rnd(*shape, s=0.2):
        return torch.randn(*shape, generator=g) * s

    tensors = {"emb": rnd(v, d, s=0.5), "pos": rnd(64, d, s=0.5), "nf.g": 1 + rnd(d), "nf.b": rnd(d), "toy.w": rnd(d)}
    for i in range(2):
        tensors.update({f"l{i}.n1.g": 1 + rnd(d), f"l{i}.n1.b": rnd(d), f"l{i}.n2.g": 1 + rnd(d), f"l{i}.n2.b": rnd(d),
                        f"l{i}.fc.w": rnd(d, f), f"l{i}.fc.b": rnd(f), f"l{i}.pr.w": rnd(f, d), f"l{i}.pr.b": rnd(d)})
    tensors.update({"l1.qkv.w": rnd(d, 3 * d), "l1.qkv.b": rnd(3 * d), "l1.o.w": rnd(d, d), "l1.o.b": rnd(d)})

    def layer(i, mixer):
        return LayerSpec(
            block="pre_norm", mixer=mixer,
            norm_1=PartSpec("layer_norm", {"eps": 1e-5}, {"gamma": f"l{i}.n1.g", "beta": f"l{i}.n1.b"}),
            norm_2=PartSpec("layer_norm", {"eps": 1e-5}, {"gamma": f"l{i}.n2.g", "beta": f"l{i}.n2.b"}),
            feed_forward=PartSpec("mlp", {"activation": "gelu_new"},
                                  {"w_in": f"l{i}.fc.w", "b_in": f"l{i}.fc.b", "w_out": f"l{i}.pr.w", "b_out": f"l{i}.pr.b"}))

    spec = ModelSpec(
        vocab_size=v, hidden=d, max_seq_len=64, eos_token=None, embedding="emb", head="emb",
        positions=PartSpec("learned", {"n_positions": 64}, {"table": "pos"}),
        layers=(layer(0, PartSpec(mixer, {"width": d}, {"w": "toy.w"})),
                layer(1, PartSpec("attention", {"n_heads": 2, "n_kv_heads": 2, "head_dim": 16, "scale": 0.25, "window": 0},
                                  {"w_qkv": "l1.qkv.w", "b_qkv": "l1.qkv.b", "w_out": "l1.o.w", "b_out": "l1.o.b"}))),
        final_norm=PartSpec("layer_norm", {"eps": 1e-5}, {"gamma": "nf.g", "beta": "nf.b"}))
    return DecoderModel(spec, tensors, Runtime(DEV, dtype)), tensors


def dense(tensors, ids):
    n, d = len(ids), 32
    x = plain.learned_positions(plain.embed_tokens(torch.tensor(ids), tensors["emb"]), torch.arange(n), tensors["pos"])
    h = plain.layer_norm(x, tensors["l0.n1.g"], tensors["l0.n1.b"], 1e-5)
    s, rows = torch.zeros(d), []
    for t in range(n):
        s = DECAY * s + h[t]
        rows.append(tensors["toy.w"] * s)
    x = x + torch.stack(rows)
    x = x + plain.linear(plain.gelu_new(plain.linear(plain.layer_norm(x, tensors["l0.n2.g"], tensors["l0.n2.b"], 1e-5),
                                                      tensors["l0.fc.w"], tensors["l0.fc.b"])), tensors["l0.pr.w"], tensors["l0.pr.b"])
    h = plain.layer_norm(x, tensors["l1.n1.g"], tensors["l1.n1.b"], 1e-5)
    q, k, v = (t.reshape(n, 2, 16) for t in plain.linear(h, tensors["l1.qkv.w"], tensors["l1.qkv.b"]).split(32, -1))
    x = x + plain.linear(plain.causal_attention(q, k, v, 0.25), tensors["l1.o.w"], tensors["l1.o.b"])
    x = x + plain.linear(plain.gelu_new(plain.linear(plain.layer_norm(x, tensors["l1.n2.g"], tensors["l1.n2.b"], 1e-5),
                                                      tensors["l1.fc.w"], tensors["l1.fc.b"])), tensors["l1.pr.w"], tensors["l1.pr.b"])
    return plain.tied_head(plain.layer_norm(x, tensors["nf.g"], tensors["nf.b"], 1e-5), tensors["emb"]).numpy()


def test_toy_mixer_with_state_is_registered_built_and_stepped():
    from research_2_b200.cache.manager import CacheManager
    from research_2_b200.engine.step import StepFunction
    from research_2_b200.parts import registry

    register_toy()
    assert "toy_running_sum" in registry("mixer")
    model, tensors = toy_model(torch.float32)
    assert len(model.state_members) == 1 and len(model.cache_members) == 1
    step_fn = StepFunction(model, 8, 16, 3, capture=True)
    assert step_fn.capture is False, "a mixer that folds rows on the host keeps the model out of CUDA graphs"
    assert step_fn.state_tensors[0].shape == (3, 32)
    cache = CacheManager(step_fn.cache_groups(), 3, 64)
    step_fn.arena.fill_(64.0)
    seqs = {0: torch.randint(0, 101, (40,), generator=torch.Generator().manual_seed(1)).tolist(),
            2: torch.randint(0, 101, (25,), generator=torch.Generator().manual_seed(2)).tolist()}
    want = {r: dense(tensors, ids) for r, ids in seqs.items()}
    got = {r: [] for r in seqs}
    fed = {r: 0 for r in seqs}
    for r in seqs:
        cache.open(r)
    plan = [[(0, 13), (2, 1)], [(2, 9), (0, 1)], [(0, 1), (2, 1)], [(0, 25)], [(2, 14)]]
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
    for r, ids in seqs.items():
        assert fed[r] == len(ids)
        out = np.concatenate(got[r])
        assert np.abs(out - want[r]).max() < 2e-4 * max(1.0, np.abs(want[r]).max()), (r, np.abs(out - want[r]).max())
    # a request slot that is used again starts from a fresh state
    cache.close(0)
    cache.open(0)
    cache.reserve(0, 0, 5)
    batch = step_fn.new_batch(5, 1, 5)
    batch.set_entries([0], [0], [seqs[2][:5]])
    cache.fill(batch)
    batch.set_logit_rows(list(range(5)))
    again = step_fn(batch).cpu().numpy()
    assert np.abs(again - want[2][:5]).max() < 2e-4 * max(1.0, np.abs(want[2]).max())


def test_toy_mixer_that_walks_entries_on_the_device_runs_inside_cuda_graphs():
    """The stateful toy in its device-only form: the step function captures the model (decode-only
    steps and steps with portions) and replays it; logits at each entry's last row against the dense
    statement, across steps that carry the state, with a request slot given to another request
    in between."""
    from research_2_b200.cache.manager import CacheManager
    from research_2_b200.engine.step import StepFunction

    register_toy_on_device()
    model, tensors = toy_model(torch.float32, "toy_running_sum_on_device")
    step_fn = StepFunction(model, 8, 16, 3, capture=True)
    assert step_fn.capture is True
    step_fn.capture_after = 0   # every shape runs as its graph from its first step on
    cache = CacheManager(step_fn.cache_groups(), 3, 64)
    step_fn.arena.fill_(64.0)
    # sequences a and b run side by side in request slots 0 and 2; c then takes slot 0, which a has left
    seqs = {"a": torch.randint(0, 101, (40,), generator=torch.Generator().manual_seed(1)).tolist(),
            "b": torch.randint(0, 101, (25,), generator=torch.Generator().manual_seed(2)).tolist(),
            "c": torch.randint(0, 101, (30,), generator=torch.Generator().manual_seed(3)).tolist()}
    slot = {"a": 0, "b": 2, "c": 0}
    want = {name: dense(tensors, ids) for name, ids in seqs.items()}
    fed = {name: 0 for name in seqs}
    cache.open(0), cache.open(2)
    plan = [[("a", 13), ("b", 1)], [("b", 9), ("a", 1)], [("a", 1), ("b", 1)], [("a", 1), ("b", 1)], [("a", 24)], [("b", 13)],
            [("c", 11)], [("c", 1)], [("c", 18)]]
    n_graphs = 0
    for step in plan:
        if step[0][0] == "c" and fed["c"] == 0:
            cache.close(0)      # its state must start fresh, whatever a left in the slot
            cache.open(0)
        reqs, starts, toks = [], [], []
        for name, n in step:
            cache.reserve(slot[name], fed[name], fed[name] + n)
            reqs.append(slot[name]); starts.append(fed[name]); toks.append(seqs[name][fed[name]: fed[name] + n])
        total = sum(len(t) for t in toks)
        batch = step_fn.new_batch(total, len(reqs), len(reqs), decode_only=all(len(t) == 1 for t in toks))
        batch.set_entries(reqs, starts, toks)
        cache.fill(batch)
        ends = np.cumsum([len(t) for t in toks]) - 1
        batch.set_logit_rows(ends.tolist())
        n_graphs += step_fn._graph_of(batch) is not None
        logits = step_fn(batch).cpu().numpy()
        for (name, n), row in zip(step, logits):
            fed[name] += n
            err = np.abs(row - want[name][fed[name] - 1]).max()
            assert err < 2e-4 * max(1.0, np.abs(want[name]).max()), (name, fed[name] - 1, err)
    assert n_graphs == len(plan), f"{n_graphs} of {len(plan)} steps ran as graphs"
    assert all(fed[name] == len(ids) for name, ids in seqs.items())
