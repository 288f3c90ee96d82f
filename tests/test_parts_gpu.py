"""Each part of a layer alone, built through the registry with sizes of its own, against the
plain implementation's function for the same part; then a model whose layers differ from one
another (a window in one, grouped heads in another, a layer run twice, a layer that reads
another layer's cache), stepped in portions against one dense pass."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from tests.plain import gpt2_plain as plain

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def rt(dtype):
    from research_2_b200.parts import Runtime

    return Runtime(DEV, dtype)


def tolerance(dtype):
    return dict(atol=3e-5, rtol=3e-5) if dtype == torch.float32 else dict(atol=4e-2, rtol=4e-2)


def one_entry_ctx(step_fn, cache, req, start, n_tokens, ids=None):
    batch = step_fn.new_batch(n_tokens, 1, n_tokens)
    batch.set_entries([req], [start], [ids if ids is not None else [0] * n_tokens])
    cache.fill(batch)
    batch.set_logit_rows(list(range(n_tokens)))
    return step_fn.upload(batch)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layer_norm_part(dtype):
    from research_2_b200.parts import PartSpec, build_part

    torch.manual_seed(0)
    tensors = {"g": torch.randn(100) + 1, "b": torch.randn(100)}
    part = build_part("norm", PartSpec("layer_norm", {"eps": 3e-4}, {"gamma": "g", "beta": "b"}), tensors, rt(dtype))
    x = torch.randn(9, 100)
    got = part.forward(x.to(DEV), dtype)
    torch.testing.assert_close(got.float().cpu(), plain.layer_norm(x, tensors["g"], tensors["b"], 3e-4), **tolerance(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("activation", ["gelu_new", "gelu"])
def test_mlp_part(dtype, activation):
    from research_2_b200.parts import PartSpec, build_part

    torch.manual_seed(1)
    d, f = 48, 200
    tensors = {"a": torch.randn(d, f) * 0.2, "ab": torch.randn(f) * 0.1, "c": torch.randn(f, d) * 0.1, "cb": torch.randn(d) * 0.1}
    tensors = {k: v.to(dtype).float() for k, v in tensors.items()}
    part = build_part("feed_forward", PartSpec("mlp", {"activation": activation},
                                               {"w_in": "a", "b_in": "ab", "w_out": "c", "b_out": "cb"}), tensors, rt(dtype))
    h = torch.randn(11, d).to(dtype)
    residual = torch.randn(11, d)
    got = part.forward(h.to(DEV), residual.to(DEV), None)
    act = plain.ACTIVATIONS[activation]
    want = residual + plain.linear(act(plain.linear(h.float(), tensors["a"], tensors["ab"])), tensors["c"], tensors["cb"])
    assert got.dtype == torch.float32
    torch.testing.assert_close(got.cpu(), want, **tolerance(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_with_learned_positions(dtype):
    from research_2_b200.parts import PartSpec, build_part
    from research_2_b200.parts.embedding import TokenEmbedding

    torch.manual_seed(2)
    table, wpe = torch.randn(300, 40).to(dtype), torch.randn(50, 40).to(dtype)
    emb = TokenEmbedding(table, rt(dtype))
    pos = build_part("positions", PartSpec("learned", {"n_positions": 50}, {"table": "wpe"}), {"wpe": wpe}, rt(dtype))

    class Ctx:
        input_ids = torch.tensor([5, 299, 0, 17], dtype=torch.int32, device=DEV)
        positions = torch.tensor([49, 0, 7, 7], dtype=torch.int32, device=DEV)

    got = emb.forward(Ctx, pos.additive_table()).cpu()
    want = plain.learned_positions(plain.embed_tokens(Ctx.input_ids.cpu(), table.float()), Ctx.positions.cpu(), wpe.float())
    torch.testing.assert_close(got, want, atol=0, rtol=0)


class TinyHost:
    """A model-less holder of a cache for part tests: one attention member."""

    def __init__(self, member, page, pages, dtype, max_seq_len=128):
        from research_2_b200.cache.manager import CacheManager
        from research_2_b200.engine.step import StepFunction

        class Shell:
            pass

        model = Shell()
        model.rt = rt(dtype)
        model.cache_members, model.state_members = [member], []
        model.max_seq_len, model.vocab_size, model.blocks = max_seq_len, 10, []
        self.step_fn = StepFunction(model, page, pages, 2)
        self.cache = CacheManager(self.step_fn.cache_groups(), 2, max_seq_len)
        self.step_fn.arena.fill_(64.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_heads,n_kv,hd,window", [(4, 4, 16, 0), (6, 2, 32, 0), (3, 1, 48, 9), (2, 2, 64, 20)])
def test_attention_part_in_portions(dtype, n_heads, n_kv, hd, window):
    """The attention part fed in portions over its paged cache equals dense attention."""
    from research_2_b200.parts import MemberSpec, PartSpec, build_part

    torch.manual_seed(hd)
    d = 40
    qkv_out = (n_heads + 2 * n_kv) * hd
    tensors = {"w": torch.randn(d, qkv_out) * 0.3, "b": torch.randn(qkv_out) * 0.1,
               "o": torch.randn(n_heads * hd, d) * 0.1, "ob": torch.randn(d) * 0.1}
    tensors = {k: v.to(dtype).float() for k, v in tensors.items()}
    scale = hd**-0.5 / 2
    part = build_part("mixer", PartSpec("attention", {"n_heads": n_heads, "n_kv_heads": n_kv, "head_dim": hd,
                                                      "scale": scale, "window": window},
                                        {"w_qkv": "w", "b_qkv": "b", "w_out": "o", "b_out": "ob"}), tensors, rt(dtype))
    assert part.cache_spec == MemberSpec(n_kv, hd, window)
    host = TinyHost(part.cache_spec, 8, 12, dtype)
    n = 50
    h = torch.randn(n, d).to(dtype)
    residual = torch.randn(n, d)
    qkv = plain.linear(h.float(), tensors["w"], tensors["b"])
    q = qkv[:, : n_heads * hd].reshape(n, n_heads, hd)
    k = qkv[:, n_heads * hd: (n_heads + n_kv) * hd].reshape(n, n_kv, hd)
    v = qkv[:, (n_heads + n_kv) * hd:].reshape(n, n_kv, hd)
    if dtype == torch.bfloat16:  # the engine rounds q, k, v to bfloat16 before attention
        q, k, v = (t.to(dtype).float() for t in (q, k, v))
    want = residual + plain.linear(plain.causal_attention(q, k, v, scale, window), tensors["o"], tensors["ob"])
    host.cache.open(1)
    at, outs = 0, []
    for rows in (17, 2, 1, 23, 1, 6):
        host.cache.slide(1, at)
        host.cache.reserve(1, at, at + rows)
        ctx = one_entry_ctx(host.step_fn, host.cache, 1, at, rows)
        outs.append(part.forward(h[at: at + rows].to(DEV), residual[at: at + rows].to(DEV), ctx, host.step_fn.arena.members[0]))
        at += rows
    got = torch.cat(outs).cpu()
    assert torch.isfinite(got).all()
    torch.testing.assert_close(got, want, **tolerance(dtype))
    if window:
        assert host.cache.pages_held(1) <= -(-(window + 6) // 8) + 1, "pages behind the window were kept"


def mixed_layers_spec(n_layers_cfg):
    """A model whose layers differ: full attention, a window with grouped heads, then layer 0
    again (same weights, cache of its own), then a layer that reads layer 1's cache."""
    from research_2_b200.models.decoder import ModelSpec, ScheduleEntry
    from research_2_b200.parts import LayerSpec, PartSpec

    d = n_layers_cfg["d"]

    def layer(i, n_heads, n_kv, hd, window, act):
        return LayerSpec(
            block="pre_norm",
            norm_1=PartSpec("layer_norm", {"eps": 1e-5}, {"gamma": f"l{i}.n1.g", "beta": f"l{i}.n1.b"}),
            mixer=PartSpec("attention", {"n_heads": n_heads, "n_kv_heads": n_kv, "head_dim": hd, "scale": hd**-0.5, "window": window},
                           {"w_qkv": f"l{i}.qkv.w", "b_qkv": f"l{i}.qkv.b", "w_out": f"l{i}.o.w", "b_out": f"l{i}.o.b"}),
            norm_2=PartSpec("layer_norm", {"eps": 1e-5}, {"gamma": f"l{i}.n2.g", "beta": f"l{i}.n2.b"}),
            feed_forward=PartSpec("mlp", {"activation": act},
                                  {"w_in": f"l{i}.fc.w", "b_in": f"l{i}.fc.b", "w_out": f"l{i}.pr.w", "b_out": f"l{i}.pr.b"}))

    layers = (layer(0, 4, 4, 16, 0, "gelu_new"), layer(1, 4, 2, 32, 12, "gelu"), layer(2, 4, 2, 32, 12, "gelu_new"))
    schedule = (ScheduleEntry(0, cache=0), ScheduleEntry(1, cache=1), ScheduleEntry(0, cache=2),
                ScheduleEntry(2, cache=1, writes_cache=False))
    return ModelSpec(vocab_size=n_layers_cfg["v"], hidden=d, max_seq_len=96, eos_token=None, embedding="emb", head="emb",
                     positions=PartSpec("learned", {"n_positions": 96}, {"table": "pos"}), layers=layers,
                     final_norm=PartSpec("layer_norm", {"eps": 1e-5}, {"gamma": "nf.g", "beta": "nf.b"}), schedule=schedule)


def mixed_layers_tensors(d, v):
    g = torch.Generator().manual_seed(3)

    def rnd(*shape, s=0.1):
        return torch.randn(*shape, generator=g) * s

    t = {"emb": rnd(v, d, s=0.5), "pos": rnd(96, d, s=0.5), "nf.g": 1 + rnd(d), "nf.b": rnd(d)}
    for i, (h, kv, hd, f) in enumerate(((4, 4, 16, 100), (4, 2, 32, 72), (4, 2, 32, 64))):
        t.update({f"l{i}.n1.g": 1 + rnd(d), f"l{i}.n1.b": rnd(d), f"l{i}.n2.g": 1 + rnd(d), f"l{i}.n2.b": rnd(d),
                  f"l{i}.qkv.w": rnd(d, (h + 2 * kv) * hd, s=0.2), f"l{i}.qkv.b": rnd((h + 2 * kv) * hd),
                  f"l{i}.o.w": rnd(h * hd, d, s=0.2), f"l{i}.o.b": rnd(d),
                  f"l{i}.fc.w": rnd(d, f, s=0.2), f"l{i}.fc.b": rnd(f), f"l{i}.pr.w": rnd(f, d, s=0.2), f"l{i}.pr.b": rnd(d)})
    return t


def mixed_layers_plain(t, ids, d):
    """The same model as one dense pass with the plain implementation's functions."""
    n = len(ids)
    x = plain.learned_positions(plain.embed_tokens(torch.tensor(ids), t["emb"]), torch.arange(n), t["pos"])
    shapes = {0: (4, 4, 16, 0, "gelu_new"), 1: (4, 2, 32, 12, "gelu"), 2: (4, 2, 32, 12, "gelu_new")}
    kv_of = {}
    for layer, reads in ((0, None), (1, None), (0, None), (2, 1)):
        h_, kvh, hd, window, act = shapes[layer]
        h = plain.layer_norm(x, t[f"l{layer}.n1.g"], t[f"l{layer}.n1.b"], 1e-5)
        qkv = plain.linear(h, t[f"l{layer}.qkv.w"], t[f"l{layer}.qkv.b"])
        q = qkv[:, : h_ * hd].reshape(n, h_, hd)
        k = qkv[:, h_ * hd: (h_ + kvh) * hd].reshape(n, kvh, hd)
        v = qkv[:, (h_ + kvh) * hd:].reshape(n, kvh, hd)
        if reads is None:
            kv_of[layer] = (k, v)
        else:
            k, v = kv_of[reads]
        x = x + plain.linear(plain.causal_attention(q, k, v, hd**-0.5, window), t[f"l{layer}.o.w"], t[f"l{layer}.o.b"])
        h = plain.layer_norm(x, t[f"l{layer}.n2.g"], t[f"l{layer}.n2.b"], 1e-5)
        x = x + plain.linear(plain.ACTIVATIONS[act](plain.linear(h, t[f"l{layer}.fc.w"], t[f"l{layer}.fc.b"])),
                             t[f"l{layer}.pr.w"], t[f"l{layer}.pr.b"])
    return plain.tied_head(plain.layer_norm(x, t["nf.g"], t["nf.b"], 1e-5), t["emb"])


def test_layers_that_differ_a_layer_twice_and_a_shared_cache():
    from research_2_b200.cache.manager import CacheManager
    from research_2_b200.engine.step import StepFunction
    from research_2_b200.models.decoder import DecoderModel

    d, v = 64, 203
    tensors = mixed_layers_tensors(d, v)
    model = DecoderModel(mixed_layers_spec({"d": d, "v": v}), tensors, rt(torch.float32))
    assert len(model.cache_members) == 3 and [m.window for m in model.cache_members] == [0, 12, 0]
    step_fn = StepFunction(model, 8, 12, 2)
    assert len(step_fn.groups) == 2 and sorted(g.window for g in step_fn.groups) == [0, 12]
    cache = CacheManager(step_fn.cache_groups(), 2, 96)
    step_fn.arena.fill_(64.0)
    ids = torch.randint(0, v, (70,), generator=torch.Generator().manual_seed(4)).tolist()
    want = mixed_layers_plain(tensors, ids, d).numpy()
    cache.open(0)
    at, outs = 0, []
    for rows in (20, 3, 1, 1, 30, 2, 13):
        cache.slide(0, at)
        cache.reserve(0, at, at + rows)
        batch = step_fn.new_batch(rows, 1, rows)
        batch.set_entries([0], [at], [ids[at: at + rows]])
        cache.fill(batch)
        batch.set_logit_rows(list(range(rows)))
        outs.append(step_fn(batch).cpu().numpy())
        at += rows
    got = np.concatenate(outs)
    window_group = [g for g, spec in enumerate(step_fn.groups) if spec.window][0]
    assert cache.pages_held(0, window_group) <= 4, "the window group kept pages that the window has passed"
    assert np.abs(got - want).max() < 2e-4 * max(1.0, np.abs(want).max()), np.abs(got - want).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_window_group_beside_a_full_one_in_portions_and_long_decoding(dtype):
    """A model with a windowed layer and full layers has two cache groups, each with block tables,
    slots and a pool of its own. Two requests are stepped together, in portions and then token by
    token to the model's limit, while the window group gives pages back as the
    window passes them (block-table entries behind the window read as the null page), so that the
    second request's window pages are ones that the first has left. Unwritten slots hold inf. Every position's
    logits against one dense pass of the plain implementation's functions."""
    from research_2_b200.cache.manager import CacheManager
    from research_2_b200.engine.step import StepFunction
    from research_2_b200.models.decoder import DecoderModel

    d, v = 64, 203
    tensors = {k: t.to(dtype).float() for k, t in mixed_layers_tensors(d, v).items()}
    model = DecoderModel(mixed_layers_spec({"d": d, "v": v}), tensors, rt(dtype))
    step_fn = StepFunction(model, 8, 18, 2)   # 18 pages a group: a request of 96 tokens (12 pages) beside one of 41 (6)
    cache = CacheManager(step_fn.cache_groups(), 2, 96)
    window_group = [g for g, spec in enumerate(step_fn.groups) if spec.window][0]
    step_fn.arena.fill_(float("inf"))
    gen = torch.Generator().manual_seed(8)
    ids = {r: torch.randint(0, v, (n,), generator=gen).tolist() for r, n in ((0, 96), (1, 41))}
    want = {r: mixed_layers_plain(tensors, seq, d).numpy() for r, seq in ids.items()}
    # request 0 in portions and then one by one; request 1 joins after request 0 has slid its window
    plan = [[(0, 20)], [(0, 3)], [(0, 29)], [(0, 1)], [(0, 1)], [(0, 2)]] + [[(0, 1)]] * 16
    plan += [[(0, 1), (1, 17)], [(0, 1), (1, 2)], [(0, 1), (1, 16)]] + [[(0, 1), (1, 1)]] * 6
    plan += [[(0, 1)]] * 15
    assert all(sum(n for q, n in sum(plan, []) if q == r) == len(seq) for r, seq in ids.items())
    at = {0: 0, 1: 0}
    got = {0: [], 1: []}
    most_window_pages = 0
    for entries in plan:
        reqs, starts, toks = [], [], []
        for r, rows in entries:
            rows = min(rows, len(ids[r]) - at[r])
            if rows <= 0:
                continue
            if not cache.is_open(r):
                cache.open(r)
            cache.slide(r, at[r])
            cache.reserve(r, at[r], at[r] + rows)
            reqs.append(r), starts.append(at[r]), toks.append(ids[r][at[r]: at[r] + rows])
        if not reqs:
            continue
        n = sum(len(t) for t in toks)
        batch = step_fn.new_batch(n, len(reqs), n, decode_only=all(len(t) == 1 for t in toks))
        batch.set_entries(reqs, starts, toks)
        cache.fill(batch)
        batch.set_logit_rows(list(range(n)))
        logits = step_fn(batch).float().cpu().numpy()
        row = 0
        for r, t in zip(reqs, toks):
            got[r].append(logits[row: row + len(t)])
            row += len(t)
            at[r] += len(t)
            if len(t) == 1:  # (a portion of n rows holds the pages of n + window - 1 keys while it runs)
                most_window_pages = max(most_window_pages, cache.pages_held(r, window_group))
            if at[r] == len(ids[r]):
                cache.close(r)
    assert most_window_pages <= 3, "while decoding, the window group kept pages that the window (12 keys, pages of 8) has passed"
    assert cache.check() == "" and all(cache.n_free(g) == 18 for g in range(2))
    for r in ids:
        out = np.concatenate(got[r])
        assert out.shape == want[r].shape and np.isfinite(out).all(), "an unwritten or returned slot leaked in"
        limit = (2e-4 if dtype == torch.float32 else 4e-2) * max(1.0, np.abs(want[r]).max())
        err = np.abs(out - want[r]).max(axis=1)
        assert err.max() < limit, f"request {r}: first position over the limit is {int(np.argmax(err >= limit))} ({err.max():.3g} >= {limit:.3g})"


def test_a_two_group_model_through_the_engine():
    """The same model through the scheduler and the engine (native batches with two groups' block tables
    and slots, admission by the worst case of each group, pages given back as the window slides):
    greedy tokens of three requests in a small pool equal the plain implementation's."""
    from research_2_b200.config.engine_options import EngineOptions
    from research_2_b200.engine.api import generate_with
    from research_2_b200.engine.engine import Engine
    from research_2_b200.models.decoder import DecoderModel

    d, v = 64, 203
    tensors = {k: t * (4.0 if k in ("emb",) else 1.0) for k, t in mixed_layers_tensors(d, v).items()}  # clear argmax gaps
    model = DecoderModel(mixed_layers_spec({"d": d, "v": v}), tensors, rt(torch.float32))
    gen = torch.Generator().manual_seed(12)
    prompts = [torch.randint(0, v, (n,), generator=gen).tolist() for n in (30, 9, 50)]
    n_new = 24

    def plain_generate(prompt):
        seq = list(prompt)
        for _ in range(n_new):
            seq.append(int(mixed_layers_plain(tensors, seq, d)[-1].argmax()))
        return seq[len(prompt):]

    want = [plain_generate(p) for p in prompts]
    opts = EngineOptions(dtype="float32", max_requests=3, block_size=8, num_slabs=18, max_batch_tokens=32, chunk_size=16)
    with Engine.for_model(model, opts) as engine:
        assert len(engine.scheduler.groups) == 2
        engine.keep_events = True
        got = generate_with(engine, prompts, n_new)
        assert engine.scheduler.cache.check() == ""
        assert all(engine.scheduler.cache.n_free(g) == 18 for g in range(2))
        events = engine.request_events()
        assert len(events) == 3 and all(e.n_generated == n_new and e.time_to_first_token_ms > 0 for e in events)
    assert got == want


def resident_spec(d, v, n_layers, heads, kv, hd, f, windows, n_positions=160):
    from research_2_b200.models.decoder import ModelSpec
    from research_2_b200.parts import LayerSpec, PartSpec

    def layer(i):
        return LayerSpec(
            block="pre_norm",
            norm_1=PartSpec("layer_norm", {"eps": 1e-5}, {"gamma": f"l{i}.n1.g", "beta": f"l{i}.n1.b"}),
            mixer=PartSpec("attention", {"n_heads": heads, "n_kv_heads": kv, "head_dim": hd, "scale": hd**-0.5 / (i + 1), "window": windows[i]},
                           {"w_qkv": f"l{i}.qkv.w", "b_qkv": f"l{i}.qkv.b", "w_out": f"l{i}.o.w", "b_out": f"l{i}.o.b"}),
            norm_2=PartSpec("layer_norm", {"eps": 3e-6}, {"gamma": f"l{i}.n2.g", "beta": f"l{i}.n2.b"}),
            feed_forward=PartSpec("mlp", {"activation": "gelu" if i % 2 else "gelu_new"},
                                  {"w_in": f"l{i}.fc.w", "b_in": f"l{i}.fc.b", "w_out": f"l{i}.pr.w", "b_out": f"l{i}.pr.b"}))

    return ModelSpec(vocab_size=v, hidden=d, max_seq_len=n_positions, eos_token=None, embedding="emb", head="emb",
                     positions=PartSpec("learned", {"n_positions": n_positions}, {"table": "pos"}),
                     layers=tuple(layer(i) for i in range(n_layers)),
                     final_norm=PartSpec("layer_norm", {"eps": 1e-5}, {"gamma": "nf.g", "beta": "nf.b"}))


def resident_tensors(d, v, n_layers, heads, kv, hd, f, n_positions=160):
    g = torch.Generator().manual_seed(21)

    def rnd(*shape, s=0.1):
        return (torch.randn(*shape, generator=g) * s).bfloat16().float()

    t = {"emb": rnd(v, d, s=0.5), "pos": rnd(n_positions, d, s=0.5), "nf.g": 1 + rnd(d), "nf.b": rnd(d)}
    for i in range(n_layers):
        t.update({f"l{i}.n1.g": 1 + rnd(d), f"l{i}.n1.b": rnd(d), f"l{i}.n2.g": 1 + rnd(d), f"l{i}.n2.b": rnd(d),
                  f"l{i}.qkv.w": rnd(d, (heads + 2 * kv) * hd, s=0.1), f"l{i}.qkv.b": rnd((heads + 2 * kv) * hd),
                  f"l{i}.o.w": rnd(heads * hd, d, s=0.1), f"l{i}.o.b": rnd(d),
                  f"l{i}.fc.w": rnd(d, f, s=0.1), f"l{i}.fc.b": rnd(f), f"l{i}.pr.w": rnd(f, d, s=0.1), f"l{i}.pr.b": rnd(d)})
    return t


def resident_plain(t, ids, n_layers, heads, kv, hd, windows):
    n = len(ids)
    x = plain.learned_positions(plain.embed_tokens(torch.tensor(ids), t["emb"]), torch.arange(n), t["pos"])
    for i in range(n_layers):
        h = plain.layer_norm(x, t[f"l{i}.n1.g"], t[f"l{i}.n1.b"], 1e-5)
        qkv = plain.linear(h, t[f"l{i}.qkv.w"], t[f"l{i}.qkv.b"])
        q = qkv[:, : heads * hd].reshape(n, heads, hd)
        k = qkv[:, heads * hd: (heads + kv) * hd].reshape(n, kv, hd)
        v = qkv[:, (heads + kv) * hd:].reshape(n, kv, hd)
        x = x + plain.linear(plain.causal_attention(q, k, v, hd**-0.5 / (i + 1), windows[i]), t[f"l{i}.o.w"], t[f"l{i}.o.b"])
        h = plain.layer_norm(x, t[f"l{i}.n2.g"], t[f"l{i}.n2.b"], 3e-6)
        act = plain.ACTIVATIONS["gelu" if i % 2 else "gelu_new"]
        x = x + plain.linear(act(plain.linear(h, t[f"l{i}.fc.w"], t[f"l{i}.fc.b"])), t[f"l{i}.pr.w"], t[f"l{i}.pr.b"])
    return plain.tied_head(plain.layer_norm(x, t["nf.g"], t["nf.b"], 1e-5), t["emb"])


@pytest.mark.parametrize("n_requests", [1, 5, 13, 30, 64])
@pytest.mark.parametrize("shape", [(64, 4, 2, 32, 80, (0, 12, 0), 8), (192, 3, 3, 64, 448, (0, 0), 16), (128, 8, 1, 16, 256, (7, 0), 4),
                                   (64, 4, 4, 16, 6416, (0,), 12)],
                         ids=["grouped_heads_of_32_with_a_window", "heads_of_64", "eight_query_heads_to_a_kv_head",
                              "an_inner_width_beyond_what_shared_memory_holds_of_the_rows_and_pages_of_12"])
def test_a_decode_steps_layers_as_one_resident_kernel(shape, n_requests):
    """Batches of one new token per row run all layers as ONE kernel whose CTAs stay resident, with
    grid barriers between a layer's phases. Requests of different lengths are prefilled (part by part)
    and then decoded for many steps, once through the resident kernel and once with every part
    launching its own kernels; both against a dense pass of the plain implementation. Grouped heads,
    a windowed layer beside full ones (two cache groups), 1 to 64 rows (one to eight token tiles), pages
    that are used again after a request has ended, unwritten slots holding inf."""
    from research_2_b200.cache.manager import CacheManager
    from research_2_b200.engine.step import StepFunction
    from research_2_b200.kernels import ops
    from research_2_b200.models.decoder import DecoderModel

    d, heads, kv, hd, f, windows, page = shape
    v, n_layers, n_decode = 211, len(windows), 24
    tensors = resident_tensors(d, v, n_layers, heads, kv, hd, f)
    model = DecoderModel(resident_spec(d, v, n_layers, heads, kv, hd, f, windows), tensors, rt(torch.bfloat16))
    gen = torch.Generator().manual_seed(n_requests)
    lengths = [int(torch.randint(1, 100, (1,), generator=gen)) + n_decode for _ in range(n_requests)]
    ids = [torch.randint(0, v, (n,), generator=gen).tolist() for n in lengths]
    want = [resident_plain(tensors, seq, n_layers, heads, kv, hd, windows).numpy() for seq in ids]
    results = {}
    for resident in (True, False):
        before, uses = ops.use_resident_decode(resident), ops.kernel_uses().get("decode_resident", 0)
        rows_before = ops.set_resident_decode_rows(64)   # (the default keeps larger batches on the chain of kernels)
        try:
            pages = sum(-(-n // page) for n in lengths) + 2
            step_fn = StepFunction(model, page, pages, n_requests)
            cache = CacheManager(step_fn.cache_groups(), n_requests, 160)
            step_fn.arena.fill_(float("inf"))
            out = [[] for _ in ids]
            for r, seq in enumerate(ids):   # prompts, one request a step
                cache.open(r)
                n = len(seq) - n_decode
                cache.reserve(r, 0, n)
                batch = step_fn.new_batch(n, 1, n)
                batch.set_entries([r], [0], [seq[:n]])
                cache.fill(batch)
                batch.set_logit_rows(list(range(n)))
                out[r].append(step_fn(batch).float().cpu().numpy())
            for i in range(n_decode):        # then all requests together, one token each
                reqs = list(range(n_requests))
                for r in reqs:
                    at = len(ids[r]) - n_decode + i
                    cache.slide(r, at)
                    cache.reserve(r, at, at + 1)
                batch = step_fn.new_batch(n_requests, n_requests, n_requests, decode_only=True)
                batch.set_entries(reqs, [len(ids[r]) - n_decode + i for r in reqs], [[ids[r][len(ids[r]) - n_decode + i]] for r in reqs])
                cache.fill(batch)
                batch.set_logit_rows(list(range(n_requests)))
                logits = step_fn(batch).float().cpu().numpy()
                for r in reqs:
                    out[r].append(logits[r: r + 1])
            assert ops.device_errors() == 0
            used = ops.kernel_uses().get("decode_resident", 0) - uses
            assert used == (n_decode if resident else 0), f"the resident kernel ran {used} times"
            results[resident] = [np.concatenate(o) for o in out]
        finally:
            ops.use_resident_decode(before)
            ops.set_resident_decode_rows(rows_before)
    for r in range(n_requests):
        limit = 4e-2 * max(1.0, np.abs(want[r]).max())
        for resident in (True, False):
            got = results[resident][r]
            assert np.isfinite(got).all(), f"resident={resident}: an unwritten slot leaked into request {r}"
            err = np.abs(got - want[r]).max(axis=1)
            other = np.abs(results[not resident][r] - want[r]).max(axis=1)
            assert err.max() < limit, (f"resident={resident} request {r} of {lengths[r]} tokens: position {int(np.argmax(err >= limit))} is off by "
                                       f"{err.max():.3g} (limit {limit:.3g}); the other path is off by {other[int(np.argmax(err >= limit))]:.3g} there")
