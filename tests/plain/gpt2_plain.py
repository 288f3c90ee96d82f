"""A plain, slow GPT-2: whole sequences, no cache, one function per part.

Written from the formulas of arb8020/research-2 (`kelpie/`); each function cites the file and
lines it restates. It shares no code with the product package: it reads model folders with the
`safetensors` library, computes with dense torch ops on the CPU, and knows nothing about pages,
batches or kernels. Tests compare the engine against it.

Options that the reference's GPT-2 does not model (`n_inner`, `activation_function`,
`scale_attn_weights`, `scale_attn_by_inverse_layer_idx`, a sliding window, grouped KV heads)
follow their usual config.json meaning and are stated in each function's docstring.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


# ---------------------------------------------------------------------------------------------
# parts


def embed_tokens(ids: torch.Tensor, wte: torch.Tensor) -> torch.Tensor:
    """x[t] = wte[ids[t]]. kelpie-models/kelpie_models/models/torch/gpt2.py:90."""
    return wte[ids.long()]


def learned_positions(x: torch.Tensor, positions: torch.Tensor, wpe: torch.Tensor) -> torch.Tensor:
    """x[t] + wpe[positions[t]], absolute positions given per row.
    kelpie-models/kelpie_models/models/torch/gpt2.py:90."""
    return x + wpe[positions.long()]


def layer_norm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(var + eps) * gamma + beta over the last dim, biased variance.
    kelpie-models/kelpie_models/kernels/ops/layer_norm.py:21-23;
    blogs/engine/ref/ch01/files/gpt2.py:135-139."""
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * gamma + beta


def gelu_new(x: torch.Tensor) -> torch.Tensor:
    """0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))).
    kelpie-models/kelpie_models/kernels/ops/gelu.py:17-19; blogs/engine/ref/ch01/files/gpt2.py:127-131."""
    inner = math.sqrt(2.0 / math.pi) * (x + 0.044715 * x**3)
    return 0.5 * x * (1.0 + torch.tanh(inner))


def gelu_erf(x: torch.Tensor) -> torch.Tensor:
    """The exact GELU 0.5 x (1 + erf(x / sqrt 2)): config.json `activation_function = "gelu"`.
    The reference pins the tanh form (kernels/ops/gelu.py:1-6); this is the other standard one."""
    return 0.5 * x * (1.0 + torch.erf(x / math.sqrt(2.0)))


ACTIVATIONS = {"gelu_new": gelu_new, "gelu": gelu_erf}


def linear(x: torch.Tensor, w_in_out: torch.Tensor, b: torch.Tensor | None) -> torch.Tensor:
    """x @ w + b with w stored [in, out] (Conv1D).
    kelpie-models/kelpie_models/models/torch/gpt2.py:52-55,113."""
    y = x @ w_in_out
    return y if b is None else y + b


def causal_attention(  # noqa: PLR0913
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    scale: float,
    window: int = 0,
    positions: torch.Tensor | None = None,
) -> torch.Tensor:
    """q [T, H, hd], k/v [T, Hkv, hd] of one whole sequence -> [T, H * hd].

    scores = q . k * scale; key j visible to query t iff j <= t (and j > t - window when
    window > 0); softmax over visible keys; out = probs @ v. Query head h reads kv head
    h // (H / Hkv). kelpie-models/kelpie_models/kernels/ops/paged_attention.py:160-212
    (scores 179, mask 186-212, PV 182-183)."""
    t_len, n_heads, head_dim = q.shape
    n_kv = k.shape[1]
    rep = n_heads // n_kv
    pos = torch.arange(t_len) if positions is None else positions.long()
    kk = k.repeat_interleave(rep, dim=1)
    vv = v.repeat_interleave(rep, dim=1)
    scores = torch.einsum("thd,shd->hts", q, kk) * scale
    visible = pos[None, :] <= pos[:, None]
    if window > 0:
        visible = visible & (pos[None, :] > pos[:, None] - window)
    scores = scores.masked_fill(~visible[None], -math.inf)
    probs = torch.softmax(scores, dim=-1)
    out = torch.einsum("hts,shd->thd", probs, vv)
    return out.reshape(t_len, n_heads * head_dim)


def attention_scale(head_dim: int, layer_idx: int, scale_attn_weights: bool, by_inverse_layer: bool) -> float:
    """hd^-1/2 when `scale_attn_weights` (the reference always scales so:
    kernels/ops/paged_attention.py:179), further divided by (layer_idx + 1) when
    `scale_attn_by_inverse_layer_idx` (config.json meaning; absent from the reference)."""
    s = head_dim**-0.5 if scale_attn_weights else 1.0
    if by_inverse_layer:
        s = s / float(layer_idx + 1)
    return s


def self_attention(h: torch.Tensor, w: dict, prefix: str, cfg: dict, layer_idx: int) -> torch.Tensor:
    """qkv = h @ c_attn + b; split in the order q, k, v; heads are contiguous hd-slices of D;
    attend; project with c_proj. kelpie-models/kelpie_models/models/torch/gpt2.py:104-131."""
    d = cfg["n_embd"]
    n_head = cfg["n_head"]
    hd = d // n_head
    qkv = linear(h, w[f"{prefix}.attn.c_attn.weight"], w[f"{prefix}.attn.c_attn.bias"])
    q, k, v = (t.reshape(h.shape[0], n_head, hd) for t in qkv.split(d, dim=-1))
    scale = attention_scale(
        hd, layer_idx, cfg.get("scale_attn_weights", True), cfg.get("scale_attn_by_inverse_layer_idx", False)
    )
    out = causal_attention(q, k, v, scale)
    return linear(out, w[f"{prefix}.attn.c_proj.weight"], w[f"{prefix}.attn.c_proj.bias"])


def mlp(h: torch.Tensor, w: dict, prefix: str, cfg: dict) -> torch.Tensor:
    """act(h @ c_fc + b) @ c_proj + b. kelpie-models/kelpie_models/models/torch/gpt2.py:94-96."""
    act = ACTIVATIONS[cfg.get("activation_function", "gelu_new")]
    inner = act(linear(h, w[f"{prefix}.mlp.c_fc.weight"], w[f"{prefix}.mlp.c_fc.bias"]))
    return linear(inner, w[f"{prefix}.mlp.c_proj.weight"], w[f"{prefix}.mlp.c_proj.bias"])


def block(x: torch.Tensor, w: dict, layer_idx: int, cfg: dict) -> torch.Tensor:
    """Pre-norm residual block: x + attn(ln_1 x), then x + mlp(ln_2 x).
    kelpie-models/kelpie_models/models/torch/gpt2.py:91-97."""
    p = f"h.{layer_idx}"
    eps = cfg["layer_norm_epsilon"]
    x = x + self_attention(layer_norm(x, w[f"{p}.ln_1.weight"], w[f"{p}.ln_1.bias"], eps), w, p, cfg, layer_idx)
    x = x + mlp(layer_norm(x, w[f"{p}.ln_2.weight"], w[f"{p}.ln_2.bias"], eps), w, p, cfg)
    return x


def tied_head(x: torch.Tensor, wte: torch.Tensor) -> torch.Tensor:
    """logits = x @ wte^T (the embedding is the head). models/torch/gpt2.py:98-101."""
    return x @ wte.T


def forward(w: dict, cfg: dict, ids: torch.Tensor) -> torch.Tensor:
    """Token ids [T] of one whole sequence -> logits [T, V] at every position.
    kelpie-models/kelpie_models/models/torch/gpt2.py:80-101 (which keeps only the last row);
    blogs/engine/ref/ch01/files/gpt2.py:182-191 (all rows)."""
    t_len = ids.shape[0]
    assert t_len <= cfg["n_positions"], (t_len, cfg["n_positions"])
    x = learned_positions(embed_tokens(ids, w["wte.weight"]), torch.arange(t_len), w["wpe.weight"])
    for i in range(cfg["n_layer"]):
        x = block(x, w, i, cfg)
    x = layer_norm(x, w["ln_f.weight"], w["ln_f.bias"], cfg["layer_norm_epsilon"])
    return tied_head(x, w["wte.weight"])


# ---------------------------------------------------------------------------------------------
# reading a model folder


def read_model(folder: str | Path, dtype: torch.dtype = torch.float32) -> tuple[dict, dict]:
    """(weights by bare tensor name, config dict) from config.json + model.safetensors. Names
    may carry a `transformer.` prefix (models/torch/gpt2.py:163-165). Values are converted to
    `dtype` (a bf16 file is upcast: the values stay the bf16-rounded ones)."""
    from safetensors.torch import load_file

    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    raw = load_file(str(folder / "model.safetensors"))
    weights = {}
    for name, tensor in raw.items():
        bare = name[len("transformer."):] if name.startswith("transformer.") else name
        weights[bare] = tensor.to(dtype)
    return weights, cfg


# ---------------------------------------------------------------------------------------------
# sampling


PHILOX_M0, PHILOX_M1 = 0xD2511F53, 0xCD9E8D57
PHILOX_W0, PHILOX_W1 = 0x9E3779B9, 0xBB67AE85
MASK32 = (1 << 32) - 1


def philox_4x32_10(counter: tuple[int, int, int, int], key: tuple[int, int]) -> tuple[int, int, int, int]:
    """Philox-4x32-10 on Python ints. kelpie-models/kelpie_models/kernels/ops/sample.py:23-49."""
    c0, c1, c2, c3 = counter
    k0, k1 = key
    for rnd in range(10):
        if rnd > 0:
            k0 = (k0 + PHILOX_W0) & MASK32
            k1 = (k1 + PHILOX_W1) & MASK32
        p0 = c0 * PHILOX_M0
        p1 = c2 * PHILOX_M1
        hi0, lo0 = (p0 >> 32) & MASK32, p0 & MASK32
        hi1, lo1 = (p1 >> 32) & MASK32, p1 & MASK32
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & MASK32, lo1, (hi0 ^ c3 ^ k1) & MASK32, lo0
    return c0, c1, c2, c3


def uniform_for(position: int, token: int, key: tuple[int, int]) -> float:
    """u = ((c0 & 0xFFFFFF) + 0.5) * 2^-24 with counter (position, 0, token, 0).
    kernels/ops/sample.py:26-30,51 (there the first counter word is the batch row; here it is
    the position of the token being drawn, so a request's draws do not depend on its batch)."""
    c0 = philox_4x32_10((position & MASK32, 0, token, 0), key)[0]
    low = torch.tensor(float(c0 & 0xFFFFFF), dtype=torch.float32)  # float32 arithmetic, as the reference
    return float((low + 0.5) * (1.0 / (1 << 24)))


def sample_token(  # noqa: PLR0913
    logits: torch.Tensor, temperature: float, top_k: int, key: tuple[int, int], position: int
) -> int:
    """One draw from fp32 logits [V]. temperature < 1e-6 or top_k == 1: argmax, first index on
    ties (kernels/ops/sample.py:103-108; the T=0 rule, kelpie-core/src/request.zig:140-144).
    Otherwise Gumbel-max over the kept tokens: top_k == 0 keeps all, k > 1 keeps every token
    >= the k-th largest value; score = logit / T + g, g = -log(-log u); filtered tokens are
    selected out, never added to (kernels/ops/sample.py:114-137)."""
    lg = logits.to(torch.float32)
    if temperature < 1e-6 or top_k == 1:
        return int(torch.argmax(lg).item())
    vocab = lg.shape[0]
    keep = torch.ones(vocab, dtype=torch.bool)
    if top_k > 1:
        kth = torch.topk(lg, top_k).values[-1]
        keep = lg >= kth
    u = torch.tensor([uniform_for(position, t, key) for t in range(vocab)], dtype=torch.float32)
    gumbel = -torch.log(-torch.log(u))
    scores = torch.where(keep, lg / torch.tensor(temperature, dtype=torch.float32) + gumbel,
                         torch.tensor(-math.inf))
    return int(torch.argmax(scores).item())


def generate(  # noqa: PLR0913
    w: dict, cfg: dict, prompt: list[int], max_new_tokens: int, temperature: float = 0.0,
    top_k: int = 0, key: tuple[int, int] = (0, 0), stop_token_ids: tuple[int, ...] = (),
) -> list[int]:
    """Re-runs the whole sequence for every new token. Stops after `max_new_tokens` (at least
    one token is produced: kelpie-core/src/scheduler.zig:613-616) or on a stop token, which is
    kept (scheduler.zig:640-644)."""
    seq = list(prompt)
    out: list[int] = []
    while True:
        logits = forward(w, cfg, torch.tensor(seq))[-1]
        tok = sample_token(logits, temperature, top_k, key, position=len(seq))
        seq.append(tok)
        out.append(tok)
        if tok in stop_token_ids or len(out) >= max(1, max_new_tokens):
            return out
