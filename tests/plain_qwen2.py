"""Plain, slow implementation of the Qwen2.5 dense decoder, used only as a test oracle.

Whole sequences, no cache, no batching, one function per part, torch on the CPU.
It shares no code with the package under test: it parses config.json keys itself,
reads tensors from a plain ``{name: tensor}`` dict and keeps everything in one
floating-point type (float32 by default; float64 gives a truth to measure float32
error against).

Every function cites the place in puneethgv/DiSpec (path inside that project) whose
behaviour it restates.  DiSpec borrows its weight modules (RMSNorm, projections,
rotary tables) from a model object of an installed package; those formulas were
pinned numerically against DiSpec's own runner, see ``tests/golden/make_golden.py``
and the outputs committed beside it.

Sliding-window layers are an extension: DiSpec refuses them
(dispec/engine/model_runner.py:79-84).  Here a layer with window W lets the query
at position p see keys b with p - W < b <= p.
"""

from __future__ import annotations

import torch


# --------------------------------------------------------------------------- config

def read_config(cfg: dict) -> dict:
    """Pick the keys the decoder needs out of a config.json dict.

    Key names as the reference reads them from the model's config object:
    dispec/engine/model_runner.py:68-72 (heads, head_dim fallback),
    dispec/kv/paged_cache.py:44-55 (layers, kv heads), :79-84 (layer_types).
    ``rope_theta`` may sit at the top level or under ``rope_parameters``
    (dispec/engine/model_runner.py:86-87 notes the layout moved).
    """
    heads = cfg["num_attention_heads"]
    head_dim = cfg.get("head_dim") or cfg["hidden_size"] // heads
    if "rope_theta" in cfg:
        theta = cfg["rope_theta"]
    else:
        theta = cfg["rope_parameters"]["rope_theta"]
    layers = cfg["num_hidden_layers"]
    windows = [0] * layers
    layer_types = cfg.get("layer_types")
    if layer_types is not None:
        windows = [cfg["sliding_window"] if t == "sliding_attention" else 0 for t in layer_types]
    elif cfg.get("use_sliding_window", False):
        first = cfg["max_window_layers"]
        windows = [cfg["sliding_window"] if i >= first else 0 for i in range(layers)]
    return dict(
        layers=layers, hidden=cfg["hidden_size"], heads=heads,
        kv_heads=cfg["num_key_value_heads"], head_dim=head_dim,
        inter=cfg["intermediate_size"], vocab=cfg["vocab_size"],
        eps=cfg["rms_norm_eps"], theta=float(theta),
        tied=bool(cfg["tie_word_embeddings"]), windows=windows,
    )


# ---------------------------------------------------------------------------- parts

def embed(table: torch.Tensor, token_ids: torch.Tensor) -> torch.Tensor:
    """x0[t] = E[token_ids[t]], no scaling. dispec/engine/model_runner.py:63,199."""
    return table[token_ids]


def rope_tables(positions: torch.Tensor, head_dim: int, theta: float, dtype=torch.float32):
    """cos/sin tables of shape (T, head_dim).

    inv_freq[i] = theta^(-2i/D); f[t,i] = pos[t]*inv_freq[i]; cos(cat(f,f)), sin(cat(f,f)).
    dispec/engine/model_runner.py:121-124 (tables), dispec/kv/transfer.py:50-58 (the
    same formula written out in float32).
    """
    exponent = torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim
    inv_freq = (1.0 / (theta ** exponent)).to(dtype)
    freqs = positions.to(dtype)[:, None] * inv_freq[None, :]
    emb = torch.cat([freqs, freqs], dim=-1)
    return emb.cos(), emb.sin()


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """cat(-x[D/2:], x[:D/2]): half-split pairs. dispec/engine/model_runner.py:35-37."""
    half = x.shape[-1] // 2
    return torch.cat([-x[..., half:], x[..., :half]], dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x*cos + rotate_half(x)*sin, tables broadcast over heads.
    dispec/engine/model_runner.py:40-44."""
    return x * cos[:, None, :] + rotate_half(x) * sin[:, None, :]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """w * x * rsqrt(mean(x^2) + eps), plain gain (no 1+w).
    Applied at dispec/engine/model_runner.py:215,218,220."""
    var = x.pow(2).mean(dim=-1, keepdim=True)
    return weight * (x * torch.rsqrt(var + eps))


def qkv_projection(h, wq, bq, wk, bk, wv, bv, heads, kv_heads, head_dim):
    """q,k,v = h W^T + b, viewed per head. dispec/engine/model_runner.py:131-140."""
    t = h.shape[0]
    q = (h @ wq.T + bq).view(t, heads, head_dim)
    k = (h @ wk.T + bk).view(t, kv_heads, head_dim)
    v = (h @ wv.T + bv).view(t, kv_heads, head_dim)
    return q, k, v


def causal_attention(q, k, v, window: int = 0) -> torch.Tensor:
    """Whole-sequence causal grouped-query attention.

    Query head j reads KV head j // G; scores scaled by head_dim**-0.5
    (dispec/engine/model_runner.py:71-72); key b visible to query a iff b <= a
    (dispec/engine/model_runner.py:172-181 with ctx_len == q_len), softmax over the
    visible keys, weighted sum of values.  ``window`` > 0 additionally hides keys
    with b <= a - window.
    """
    t, heads, d = q.shape
    kv_heads = k.shape[1]
    group = heads // kv_heads
    scale = d ** -0.5
    a = torch.arange(t)[:, None]
    b = torch.arange(t)[None, :]
    visible = b <= a
    if window > 0:
        visible &= b > a - window
    out = torch.empty_like(q)
    for j in range(heads):
        kj, vj = k[:, j // group], v[:, j // group]
        s = (q[:, j] @ kj.T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        out[:, j] = torch.softmax(s, dim=-1) @ vj
    return out


def swiglu_mlp(h, w_gate, w_up, w_down) -> torch.Tensor:
    """down( silu(h Wg^T) * (h Wu^T) ). dispec/engine/model_runner.py:222-226."""
    g = h @ w_gate.T
    u = h @ w_up.T
    return ((g * torch.sigmoid(g)) * u) @ w_down.T


def decoder_layer(x, w: dict, prefix: str, c: dict, cos, sin, window: int) -> torch.Tensor:
    """norm -> attention -> residual -> norm -> MLP -> residual.
    dispec/engine/model_runner.py:214-219."""
    h = rms_norm(x, w[prefix + "input_layernorm.weight"], c["eps"])
    a = prefix + "self_attn."
    q, k, v = qkv_projection(
        h, w[a + "q_proj.weight"], w[a + "q_proj.bias"], w[a + "k_proj.weight"],
        w[a + "k_proj.bias"], w[a + "v_proj.weight"], w[a + "v_proj.bias"],
        c["heads"], c["kv_heads"], c["head_dim"])
    q = apply_rope(q, cos, sin)
    k = apply_rope(k, cos, sin)
    o = causal_attention(q, k, v, window)
    x = x + o.reshape(x.shape[0], -1) @ w[a + "o_proj.weight"].T
    h = rms_norm(x, w[prefix + "post_attention_layernorm.weight"], c["eps"])
    m = prefix + "mlp."
    return x + swiglu_mlp(h, w[m + "gate_proj.weight"], w[m + "up_proj.weight"],
                          w[m + "down_proj.weight"])


def forward_logits(weights: dict, config: dict, token_ids, dtype=torch.float32, rows=None) -> torch.Tensor:
    """Logits (T, vocab) of one whole sequence starting at position 0; with ``rows`` (a list of
    positions) only those rows, (len(rows), vocab), as the reference's ``logits(hidden, indices)``
    does.  dispec/engine/model_runner.py:188-231."""
    c = read_config(config)
    w = {k: v.to(dtype) for k, v in weights.items()}
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    positions = torch.arange(ids.shape[0])
    cos, sin = rope_tables(positions, c["head_dim"], c["theta"], dtype)
    x = embed(w["model.embed_tokens.weight"], ids)
    for i in range(c["layers"]):
        x = decoder_layer(x, w, f"model.layers.{i}.", c, cos, sin, c["windows"][i])
    if rows is not None:
        x = x[torch.as_tensor(list(rows), dtype=torch.long)]
    x = rms_norm(x, w["model.norm.weight"], c["eps"])
    head = w["model.embed_tokens.weight"] if c["tied"] else w["lm_head.weight"]
    return x @ head.T


# ------------------------------------------------------------------------- sampling

def apply_top_k_top_p(logits: torch.Tensor, top_k: int, top_p: float) -> torch.Tensor:
    """Mask by top-k (ties with the k-th value stay) and then top-p (drop a token when the
    mass before it in descending order exceeds top_p; the first always stays).
    dispec/sampling.py:26-45."""
    if top_k and top_k > 0:
        k = min(top_k, logits.shape[-1])
        kth = torch.topk(logits, k, dim=-1).values[..., -1, None]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p < 1.0:
        sorted_logits, order = torch.sort(logits, descending=True, dim=-1, stable=True)
        probs = torch.softmax(sorted_logits, dim=-1)
        before = probs.cumsum(dim=-1) - probs
        drop = before > top_p
        drop[..., 0] = False
        logits = logits.masked_fill(drop.scatter(-1, order, drop), float("-inf"))
    return logits


def sampling_distribution(logits: torch.Tensor, temperature: float, top_k: int = 0,
                          top_p: float = 1.0) -> torch.Tensor:
    """Distribution a token is drawn from: one-hot argmax when temperature <= 0, else
    softmax(mask(logits / T)). dispec/sampling.py:48-59."""
    logits = logits.to(torch.float64)
    if temperature <= 0.0:
        out = torch.zeros_like(logits)
        out.scatter_(-1, logits.argmax(dim=-1, keepdim=True), 1.0)
        return out
    return torch.softmax(apply_top_k_top_p(logits / temperature, top_k, top_p), dim=-1)


def draw_inverse_cdf(probs: torch.Tensor, u: float) -> int:
    """Index of the first token whose cumulative probability (vocabulary order) reaches
    u * total.  DiSpec draws with torch.multinomial (dispec/sampling.py:62-67); any
    exact sampler of the same distribution is equivalent, and this one is replayable."""
    cdf = probs.to(torch.float64).cumsum(-1)
    idx = int(torch.searchsorted(cdf, torch.tensor(u * float(cdf[-1]), dtype=torch.float64)))
    idx = min(idx, probs.shape[-1] - 1)
    while probs[idx] == 0 and idx > 0:
        idx -= 1
    return idx


def greedy_generate(weights: dict, config: dict, prompt_ids, max_new_tokens: int,
                    eos_id=None, dtype=torch.float32):
    """Prefill, argmax, feed back; stop at max_new_tokens or after emitting eos.
    dispec/engine/engine.py:46-101 without its cache.  Returns (tokens, top-2 gaps)."""
    ids = list(prompt_ids)
    out, gaps = [], []
    while len(out) < max_new_tokens:
        last = forward_logits(weights, config, ids, dtype)[-1]
        top2 = torch.topk(last, 2).values
        gaps.append(float(top2[0] - top2[1]))
        nxt = int(last.argmax())
        out.append(nxt)
        ids.append(nxt)
        if eos_id is not None and nxt == eos_id:
            break
    return out, gaps


# ------------------------------------------------------------------- random weights

def tensor_shapes(config: dict) -> dict:
    """Names and shapes of a Qwen2ForCausalLM state dict ((out, in) matrices, y = x W^T + b):
    the modules the reference picks at dispec/engine/model_runner.py:62-66,104-118."""
    c = read_config(config)
    h, d = c["hidden"], c["head_dim"]
    shapes = {"model.embed_tokens.weight": (c["vocab"], h)}
    for i in range(c["layers"]):
        p = f"model.layers.{i}."
        shapes[p + "input_layernorm.weight"] = (h,)
        shapes[p + "self_attn.q_proj.weight"] = (c["heads"] * d, h)
        shapes[p + "self_attn.q_proj.bias"] = (c["heads"] * d,)
        shapes[p + "self_attn.k_proj.weight"] = (c["kv_heads"] * d, h)
        shapes[p + "self_attn.k_proj.bias"] = (c["kv_heads"] * d,)
        shapes[p + "self_attn.v_proj.weight"] = (c["kv_heads"] * d, h)
        shapes[p + "self_attn.v_proj.bias"] = (c["kv_heads"] * d,)
        shapes[p + "self_attn.o_proj.weight"] = (h, c["heads"] * d)
        shapes[p + "post_attention_layernorm.weight"] = (h,)
        shapes[p + "mlp.gate_proj.weight"] = (c["inter"], h)
        shapes[p + "mlp.up_proj.weight"] = (c["inter"], h)
        shapes[p + "mlp.down_proj.weight"] = (h, c["inter"])
    shapes["model.norm.weight"] = (h,)
    if not c["tied"]:
        shapes["lm_head.weight"] = (c["vocab"], h)
    return shapes


def random_weights(config: dict, seed: int, std: float, head_std: float | None = None) -> dict:
    """Matrices, embedding and biases N(0, std); norm gains 1 + N(0, std).
    ``head_std`` redraws the output matrix wider so that argmax is not a near-tie, as
    the reference's own fixture does (tests/tiny_models.py:1-6,17-23)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        t = torch.randn(shape, generator=g, dtype=torch.float32) * std
        if name.endswith("layernorm.weight") or name == "model.norm.weight":
            t = t + 1.0
        if head_std is not None and name == "lm_head.weight":
            t = t * (head_std / std)
        out[name] = t
    return out



# ------------------------------------------------ counter-based random weights (scalar restatement)

def _philox4x32_10(counter, key):
    """Philox-4x32 with ten rounds on Python integers (the published algorithm: two 32x32 -> 64
    multiplications per round, the key bumped by the golden-ratio and sqrt(3) constants)."""
    c0, c1, c2, c3 = counter
    k0, k1 = key
    for _ in range(10):
        p0, p1 = 0xD2511F53 * c0, 0xCD9E8D57 * c2
        c0, c1, c2, c3 = (p1 >> 32) ^ c1 ^ k0, p1 & 0xFFFFFFFF, (p0 >> 32) ^ c3 ^ k1, p0 & 0xFFFFFFFF
        k0, k1 = (k0 + 0x9E3779B9) & 0xFFFFFFFF, (k1 + 0xBB67AE85) & 0xFFFFFFFF
    return c0, c1, c2, c3


def counter_normal_element(seed: int, ordinal: int, index: int):
    """Element ``index`` of tensor ``ordinal`` under ``seed`` as the engine's random-weights mode
    defines it, one element at a time with numpy float32 scalars (every operation rounded once):
    Philox block index // 4, Box-Muller on words (0, 1) for elements 0 and 1 of the block and on
    words (2, 3) for elements 2 and 3, uniforms = odd multiples of 2^-24 from the top 23 bits,
    logarithm by the atanh series, sine and cosine by octant reduction and Taylor polynomials."""
    import numpy as np
    f = np.float32
    block, lane = divmod(index, 4)
    words = _philox4x32_10((block & 0xFFFFFFFF, block >> 32, ordinal, 0), (seed & 0xFFFFFFFF, seed >> 32))
    w0, w1 = words[2 * (lane // 2)], words[2 * (lane // 2) + 1]
    u = f(2 * (w0 >> 9) + 1) * f(5.96046448e-08)
    bits = int(np.array(u, dtype=np.float32).view(np.uint32))
    e = (bits >> 23) - 127
    m = np.array((bits & 0x007FFFFF) | 0x3F800000, dtype=np.uint32).view(np.float32)[()]
    if m > f(1.41421354):
        m, e = m * f(0.5), e + 1
    t = m - f(1.0)
    s = t / (t + f(2.0))
    z = s * s
    p = z * f(0.222222224) + f(0.285714298)
    p = z * p + f(0.400000006)
    p = z * p + f(0.666666687)
    p = z * p + f(2.0)
    log_u = f(e) * f(0.693147182) + s * p
    radius = np.sqrt(f(-2.0) * log_u)
    n = 2 * (w1 >> 9) + 1
    octant, r = n >> 21, n & 0x1FFFFF
    if octant & 1:
        r = 0x200000 - r
    a = (f(r) * f(4.76837158e-07)) * f(0.785398185)
    a2 = a * a
    ps = a2 * f(2.75573188e-06) + f(-1.98412701e-04)
    ps = a2 * ps + f(8.33333377e-03)
    ps = a2 * ps + f(-0.166666672)
    ps = a2 * ps + f(1.0)
    sin_a = a * ps
    pc = a2 * f(-2.75573188e-07) + f(2.48015876e-05)
    pc = a2 * pc + f(-1.38888892e-03)
    pc = a2 * pc + f(4.16666679e-02)
    pc = a2 * pc + f(-0.5)
    cos_a = a2 * pc + f(1.0)
    sin_t, cos_t = {0: (sin_a, cos_a), 1: (cos_a, sin_a), 2: (cos_a, -sin_a), 3: (sin_a, -cos_a),
                    4: (-sin_a, -cos_a), 5: (-cos_a, -sin_a), 6: (-cos_a, sin_a), 7: (-sin_a, cos_a)}[octant]
    return radius * (cos_t if lane % 2 == 0 else sin_t)


def counter_random_tensor(names, name: str, shape, seed: int, std: float, mean: float = 0.0,
                          indices=None) -> torch.Tensor:
    """Float32 values (before the rounding to the storage type) of tensor ``name`` of a checkpoint
    whose tensor names are ``names``: ordinal = place of the name in sorted order; value =
    mean + std * z.  ``indices``: flat element indices to compute (default: all)."""
    import numpy as np
    ordinal = sorted(names).index(name)
    total = 1
    for d in shape:
        total *= d
    idx = range(total) if indices is None else indices
    vals = [np.float32(mean) + np.float32(std) * counter_normal_element(seed, ordinal, int(i)) for i in idx]
    t = torch.tensor(np.array(vals, dtype=np.float32))
    return t.reshape(shape) if indices is None else t
