"""Plain, slow, whole-sequence implementation of the dense Qwen3 decoder.

It is the oracle of the test suite.  It has no cache, no batching and no
chunking, runs on the CPU with ordinary tensor arithmetic, and shares no code
with the engine: it parses ``config.json`` and reads ``model.safetensors`` by
itself.  Every function restates one formula of RicardoMin/tiny-vLLM and cites
the file and lines (paths inside that project) it was taken from.

``dt`` is the storage dtype that the engine under test runs in.  With
``torch.float32`` nothing is rounded.  With ``torch.bfloat16`` every value
that the reference materialises between two operations is rounded to bfloat16
and brought back to float32, so that the oracle follows the same rounding
points while all arithmetic itself stays in float32.

One thing goes beyond the reference: a sliding window on chosen layers.  The
reference refuses ``use_sliding_window`` (tinyvllm/models/qwen3.py:186-189);
here a layer with window ``W`` lets the query at position ``p`` see the keys
``p-W+1 .. p``.  The list ``order`` of (layer, cache_from) pairs restates the
engine's run list: a layer may run twice, and a run may attend over the keys
and values that an earlier run produced.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

F32 = torch.float32


def rnd(x: torch.Tensor, dt: torch.dtype) -> torch.Tensor:
    """Round to the storage dtype and return float32 again."""
    if dt == F32:
        return x
    return x.to(dt).to(F32)


# --------------------------------------------------------------------------
# configuration and weights (own parsing, nothing shared with the engine)
# --------------------------------------------------------------------------

def read_config(model_dir) -> dict:
    """config.json keys of tinyvllm/models/qwen3.py:25-36 plus the optional
    ones the reference reads through its passthrough (:203-204)."""
    raw = json.loads((Path(model_dir) / "config.json").read_text())
    cfg = {
        "V": raw["vocab_size"],
        "H": raw["hidden_size"],
        "I": raw["intermediate_size"],
        "L": raw["num_hidden_layers"],
        "nq": raw["num_attention_heads"],
        "nkv": raw["num_key_value_heads"],
        "d": raw["head_dim"],
        "max_pos": raw["max_position_embeddings"],
        "theta": float(raw.get("rope_theta", 1_000_000.0)),   # tinyvllm/layers.py:175
        "eps": float(raw.get("rms_norm_eps", 1e-6)),          # tinyvllm/layers.py:136
        "tied": bool(raw.get("tie_word_embeddings", False)),
    }
    windows = [None] * cfg["L"]
    if raw.get("use_sliding_window", False):
        size = raw["sliding_window"]
        kinds = raw.get("layer_types")
        if kinds is None:
            first = raw.get("max_window_layers", cfg["L"])
            kinds = ["full_attention" if i < first else "sliding_attention"
                     for i in range(cfg["L"])]
        windows = [size if k == "sliding_attention" else None for k in kinds]
    cfg["windows"] = windows
    return cfg


def read_weights(model_dir) -> dict[str, torch.Tensor]:
    """All tensors of the folder by checkpoint name, as float32 (names of
    tinyvllm/models/qwen3.py:569-648)."""
    from safetensors.torch import load_file

    out = {}
    for path in sorted(Path(model_dir).glob("*.safetensors")):
        for name, tensor in load_file(str(path)).items():
            out[name] = tensor.to(F32)
    return out


# --------------------------------------------------------------------------
# one function for each part
# --------------------------------------------------------------------------

def embed(table: torch.Tensor, ids: torch.Tensor, dt) -> torch.Tensor:
    """h = E[ids]  (tinyvllm/models/qwen3.py:480); the rows are rounded after the gather, which is
    the same values as gathering from the rounded table."""
    return rnd(table[ids], dt)


def rope_tables(d: int, max_pos: int, theta: float):
    """float32 cos/sin of p * theta^(-2j/d), j < d/2
    (tinyvllm/layers.py:192-226)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=F32) / d))
    ang = torch.outer(torch.arange(max_pos, dtype=F32), inv_freq)
    return ang.cos(), ang.sin()


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, dt) -> torch.Tensor:
    """y = round(round(x * rsqrt(mean(x^2) + eps)) * w), sums in float32
    (tinyvllm/kernels/pointwise.cu:153-211)."""
    n = x.shape[-1]
    var = (x * x).sum(-1, keepdim=True) * (1.0 / n)
    r = torch.rsqrt(var + eps)
    return rnd(rnd(x * r, dt) * w, dt)


def add_rms_norm(x, res, w, eps, dt):
    """m = round(x + res); returns (RMSNorm(m), m)
    (tinyvllm/kernels/pointwise.cu:159-164, :203-205; tinyvllm/layers.py:159-164)."""
    m = rnd(x + res, dt)
    return rms_norm(m, w, eps, dt), m


def linear(x: torch.Tensor, w: torch.Tensor, dt) -> torch.Tensor:
    """x . W^T without bias, float32 accumulation, result rounded
    (tinyvllm/layers.py:84-85)."""
    return rnd(x @ rnd(w, dt).T, dt)


def rotate_half_split(x, cos, sin, dt):
    """y1 = round(round(x1 c) - round(x2 s)), y2 = round(round(x2 c) + round(x1 s))
    with x1, x2 the two halves of the head (tinyvllm/kernels/pointwise.cu:94-116).
    x: [T, heads, d]; cos, sin: [T, d/2], rounded to the storage dtype first
    (tinyvllm/layers.py:235-243)."""
    half = x.shape[-1] // 2
    c = rnd(cos, dt)[:, None, :]
    s = rnd(sin, dt)[:, None, :]
    x1, x2 = x[..., :half], x[..., half:]
    y1 = rnd(rnd(x1 * c, dt) - rnd(x2 * s, dt), dt)
    y2 = rnd(rnd(x2 * c, dt) + rnd(x1 * s, dt), dt)
    return torch.cat([y1, y2], dim=-1)


def qk_norm_rope(q, k, qw, kw, cos, sin, eps, dt):
    """Per (token, head) RMSNorm over the head, then rotation, for q and k
    (tinyvllm/models/qwen3.py:284-293; tinyvllm/kernels/pointwise.cu:366-449)."""
    q = rotate_half_split(rms_norm(q, qw, eps, dt), cos, sin, dt)
    k = rotate_half_split(rms_norm(k, kw, eps, dt), cos, sin, dt)
    return q, k


def causal_attention(q, k, v, scale: float, window, dt,
                     q_positions: torch.Tensor | None = None) -> torch.Tensor:
    """softmax(scale * q.K^T) V over the keys j <= p (and j > p - window),
    q head h reading kv head h // (nq/nkv); scores and softmax in float32
    (scale tinyvllm/models/qwen3.py:228; group map
    tinyvllm/kernels/paged_decode.cu:120; mask tinyvllm/runtime/attention.py:34-55;
    softmax tinyvllm/kernels/paged_decode.cu:302-356, :457-465).
    q: [Tq, nq, d]; k, v: [Tk, nkv, d]; query i stands at position
    q_positions[i] (default i), key j at position j."""
    tq, nq, d = q.shape
    tk, nkv, _ = k.shape
    group = nq // nkv
    pos_q = torch.arange(tq) if q_positions is None else q_positions
    pos_k = torch.arange(tk)
    keep = pos_k[None, :] <= pos_q[:, None]
    if window is not None:
        keep &= pos_k[None, :] > (pos_q[:, None] - window)
    out = torch.empty_like(q)
    for h in range(nq):
        g = h // group
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        s = s.masked_fill(~keep, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, g, :]
    return rnd(out, dt)


def swiglu(gate_up: torch.Tensor, dt) -> torch.Tensor:
    """round(round(silu(gate)) * up), silu(g) = g / (1 + exp(-g))
    (tinyvllm/kernels/pointwise.cu:274-285)."""
    inter = gate_up.shape[-1] // 2
    gate, up = gate_up[..., :inter], gate_up[..., inter:]
    act = rnd(gate / (1.0 + torch.exp(-gate)), dt)
    return rnd(act * up, dt)


# --------------------------------------------------------------------------
# blocks and the whole model
# --------------------------------------------------------------------------

def attention_block(cfg, w, prefix, x, cos, sin, window, dt, kv_from=None):
    """QKV projection, q/k norm, rotation, attention, output projection
    (tinyvllm/models/qwen3.py:273-303).  Returns (output, (k, v)); with
    ``kv_from`` the keys and values of another run are attended instead."""
    t = x.shape[0]
    nq, nkv, d = cfg["nq"], cfg["nkv"], cfg["d"]
    q = linear(x, w[f"{prefix}.self_attn.q_proj.weight"], dt).view(t, nq, d)
    k = linear(x, w[f"{prefix}.self_attn.k_proj.weight"], dt).view(t, nkv, d)
    v = linear(x, w[f"{prefix}.self_attn.v_proj.weight"], dt).view(t, nkv, d)
    q, k = qk_norm_rope(
        q, k,
        rnd(w[f"{prefix}.self_attn.q_norm.weight"], dt),
        rnd(w[f"{prefix}.self_attn.k_norm.weight"], dt),
        cos, sin, cfg["eps"], dt,
    )
    if kv_from is not None:
        k, v = kv_from
    a = causal_attention(q, k, v, d ** -0.5, window, dt)
    o = linear(a.reshape(t, nq * d), w[f"{prefix}.self_attn.o_proj.weight"], dt)
    return o, (k, v)


def mlp_block(w, prefix, x, dt):
    """down(silu(gate(x)) * up(x))  (tinyvllm/models/qwen3.py:316-346)."""
    gate_up = torch.cat(
        [linear(x, w[f"{prefix}.mlp.gate_proj.weight"], dt),
         linear(x, w[f"{prefix}.mlp.up_proj.weight"], dt)], dim=-1)
    return linear(swiglu(gate_up, dt), w[f"{prefix}.mlp.down_proj.weight"], dt)


def forward(cfg: dict, w: dict, ids, dt=F32, order=None, rows=None) -> torch.Tensor:
    """Logits [T, V] of one whole sequence, float32; with ``rows`` (positions) only those rows,
    in that order (every layer still runs over the whole sequence).

    Layer arrangement of tinyvllm/models/qwen3.py:386-412 and :458-494: the
    first layer norms the embedding and keeps it as the residual stream;
    every later norm first adds the previous output to the stream; the
    feed-forward output is added by the next layer's norm or the final one.
    Head: tinyvllm/models/qwen3.py:703-717 (tied: :514-525)."""
    ids = torch.as_tensor(ids, dtype=torch.long)
    t = ids.shape[0]
    h = embed(w["model.embed_tokens.weight"], ids, dt)
    cos, sin = rope_tables(cfg["d"], cfg["max_pos"], cfg["theta"])
    cos, sin = cos[:t], sin[:t]
    if order is None:
        order = [(i, None) for i in range(cfg["L"])]
    res = None
    produced = []
    for layer, cache_from in order:
        p = f"model.layers.{layer}"
        win = rnd(w[f"{p}.input_layernorm.weight"], dt)
        wpost = rnd(w[f"{p}.post_attention_layernorm.weight"], dt)
        if res is None:
            res = h
            x = rms_norm(h, win, cfg["eps"], dt)
        else:
            x, res = add_rms_norm(h, res, win, cfg["eps"], dt)
        kv_from = None if cache_from is None else produced[cache_from]
        a, kv = attention_block(cfg, w, p, x, cos, sin, cfg["windows"][layer], dt, kv_from)
        produced.append(kv)
        x, res = add_rms_norm(a, res, wpost, cfg["eps"], dt)
        h = mlp_block(w, p, x, dt)
    if rows is not None:
        keep = torch.as_tensor(list(rows), dtype=torch.long)
        h, res = h[keep], res[keep]
    x, _ = add_rms_norm(h, res, rnd(w["model.norm.weight"], dt), cfg["eps"], dt)
    head = w["model.embed_tokens.weight"] if cfg["tied"] else w["lm_head.weight"]
    return x @ rnd(head, dt).T


def greedy_generate(cfg, w, prompt, new_tokens: int, dt=F32) -> list[int]:
    """argmax decoding by running the whole sequence again for every token
    (tinyvllm/sampling.py:42-43)."""
    seq = list(prompt)
    out = []
    for _ in range(new_tokens):
        logits = forward(cfg, w, seq, dt)
        nxt = int(torch.argmax(logits[-1]))
        out.append(nxt)
        seq.append(nxt)
    return out


# --------------------------------------------------------------------------
# sampling (tinyvllm/sampling.py:75-164), with the engine's counter-based noise
# --------------------------------------------------------------------------

_M32 = 0xFFFFFFFF


def _mulhilo(a: int, b: int):
    p = a * b
    return (p >> 32) & _M32, p & _M32


def philox4x32(counter, key, rounds: int = 10):
    """Philox-4x32-10 (Salmon et al., 2011), on Python integers."""
    c = list(counter)
    k = list(key)
    for _ in range(rounds):
        hi0, lo0 = _mulhilo(0xD2511F53, c[0])
        hi1, lo1 = _mulhilo(0xCD9E8D57, c[2])
        c = [hi1 ^ c[1] ^ k[0], lo1, hi0 ^ c[3] ^ k[1], lo0]
        k = [(k[0] + 0x9E3779B9) & _M32, (k[1] + 0xBB67AE85) & _M32]
    return c


def exponential_noise(seed: int, draw: int, vocab: int) -> torch.Tensor:
    """Exp(1) noise of one draw: token i takes word i%4 of
    philox(counter=(i//4, draw_lo, draw_hi, 0), key=(seed_lo, seed_hi));
    u = ((x >> 9) + 0.5) / 2^23 (exact in float32); noise = -log(u) in float32."""
    key = (seed & _M32, (seed >> 32) & _M32)
    words = []
    for block in range((vocab + 3) // 4):
        words.extend(philox4x32((block, draw & _M32, (draw >> 32) & _M32, 0), key))
    x = torch.tensor([word >> 9 for word in words[:vocab]], dtype=torch.float64)
    u = ((x + 0.5) / 8388608.0).to(F32)
    return -torch.log(u)


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float,
           seed: int, draw: int) -> int:
    """One token from one row of logits.

    temperature 0: argmax (tinyvllm/sampling.py:42-43).  Else scores =
    (logits - max) / temperature (:82-104); keep the top_k largest (:107-112);
    softmax over what is kept; top_p drops every token before which, in
    descending stable order, more than top_p of the mass already lies
    (:125-139); the draw is argmax(p / noise) with Exp(1) noise (:141-157).
    Ties go to the smaller token id throughout."""
    logits = logits.to(F32)
    vocab = logits.shape[0]
    if temperature == 0.0:
        return int(torch.argmax(logits))
    scores = (logits - logits.max()) / temperature
    order = torch.sort(scores, descending=True, stable=True).indices
    keep = torch.ones(vocab, dtype=torch.bool)
    if 0 < top_k < vocab:
        keep[:] = False
        keep[order[:top_k]] = True
    p = torch.softmax(scores.masked_fill(~keep, float("-inf")), dim=0)
    if top_p < 1.0:
        sorted_p = p[order]
        before = sorted_p.cumsum(0) - sorted_p
        drop = before > top_p
        drop[0] = False
        p[order[drop]] = 0.0
    noise = exponential_noise(seed, draw, vocab)
    return int(torch.argmax(p / noise))
