"""Plain, slow implementation of the Qwen3 dense decoder, used only as the test oracle.

Whole sequences, no cache, one function per part, plain torch on the CPU.  It
shares no code with ``ondeviceinfer_b200``: it takes a raw ``config.json``
dictionary and a ``{checkpoint tensor name: tensor}`` mapping and nothing else.
Every function restates a formula of UESlubei/ondeviceinfer and cites the place
(path inside that project, ``file:line``).

``tests/golden/make_golden.py`` ran this file against the reference project's own
model code (imported on the CPU) for two tiny random models; the outputs it
committed under ``tests/golden/`` are re-checked by ``tests/test_plain.py``.

``dtype`` selects the arithmetic: ``torch.float32`` is the exact oracle;
``torch.bfloat16`` rounds after every operation exactly where the reference's
eager code does, which is what a bf16 engine is compared with.
"""

from __future__ import annotations

import math

import torch

MASK64 = (1 << 64) - 1


# --------------------------------------------------------------------------- parts


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm: square/mean/rsqrt in fp32, cast back, then scale in the model dtype.

    ondeviceinfer/layers.py:28-33 and ondeviceinfer/functional.py:17-22; the order
    (normalise in fp32 -> cast -> multiply by the weight) is what
    tests/test_foundations.py:43-45 of the reference asserts.
    """
    x32 = x.float()
    variance = (x32 * x32).mean(dim=-1, keepdim=True)
    y = x32 * torch.rsqrt(variance + eps)
    return weight * y.to(x.dtype)


def rope_tables(positions: torch.Tensor, head_dim: int, theta: float, dtype: torch.dtype):
    """cos/sin tables [T, head_dim] for integer positions.

    ondeviceinfer/layers.py:44-46 (inv_freq = 1 / theta**(arange(0,d,2)/d), fp32) and
    ondeviceinfer/layers.py:59-63 (angles in fp32, the half table repeated twice, cast
    to the model dtype).
    """
    exponent = torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim
    inv_freq = 1.0 / (theta**exponent)
    freqs = positions.to(torch.float32).unsqueeze(-1) * inv_freq
    angles = torch.cat((freqs, freqs), dim=-1)
    return angles.cos().to(dtype), angles.sin().to(dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Half-split rotation of x [heads, T, d]: x*cos + cat(-x2, x1)*sin.

    ondeviceinfer/layers.py:66-69 (rotate_half) and ondeviceinfer/layers.py:79-83.
    """
    half = x.shape[-1] // 2
    rotated = torch.cat((-x[..., half:], x[..., :half]), dim=-1)
    return x * cos.unsqueeze(0) + rotated * sin.unsqueeze(0)


def causal_gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """softmax(q k^T / sqrt(d) + causal mask) v with grouped heads.

    q [nq, T, d], k and v [nkv, T, d].  Query head h reads key/value head h // g with
    g = nq // nkv (ondeviceinfer/config.py:76-79; shown equal to repeat_interleave in
    the reference's tests/test_model.py:40-53).  Key j is visible to query t iff
    j <= t (ondeviceinfer/attention.py:29-33 with no past).  The scale 1/sqrt(d) is the
    default of the scaled-dot-product call at ondeviceinfer/attention.py:77-85, which
    passes no scale.  Softmax is taken in fp32.
    """
    nq, T, d = q.shape
    nkv = k.shape[0]
    g = nq // nkv
    kk = k.repeat_interleave(g, dim=0)
    vv = v.repeat_interleave(g, dim=0)
    scores = (q.float() @ kk.float().transpose(-1, -2)) / math.sqrt(d)
    visible = torch.arange(T).unsqueeze(0) <= torch.arange(T).unsqueeze(1)
    scores = scores.masked_fill(~visible, float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    return (probs @ vv.float()).to(q.dtype)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """y = x W^T (+ b) for an [out, in] weight (nn.Linear; the four attention projections carry a bias
    when ``attention_bias`` is set, ondeviceinfer/attention.py:106-129; no other product has one)."""
    y = x @ weight.t()
    return y if bias is None else y + bias


def attention_block(x, w, prefix, cfg, cos, sin):
    """Projections, per-head Q/K norm, RoPE, attention, output projection.

    ondeviceinfer/attention.py:149-177: q/k/v projections viewed as [T, heads, d];
    q_norm and k_norm over d with one [d] weight for all heads, before RoPE (:159-160);
    V untouched (:161); rotation (:162); heads merged as column h*d + j (:173-176);
    o_proj (:177).
    """
    T = x.shape[0]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], head_dim_of(cfg)
    eps = cfg["rms_norm_eps"]
    q = linear(x, w[prefix + "q_proj.weight"], w.get(prefix + "q_proj.bias")).view(T, nq, d)
    k = linear(x, w[prefix + "k_proj.weight"], w.get(prefix + "k_proj.bias")).view(T, nkv, d)
    v = linear(x, w[prefix + "v_proj.weight"], w.get(prefix + "v_proj.bias")).view(T, nkv, d)
    q = rms_norm(q, w[prefix + "q_norm.weight"], eps).transpose(0, 1)
    k = rms_norm(k, w[prefix + "k_norm.weight"], eps).transpose(0, 1)
    v = v.transpose(0, 1)
    q = apply_rope(q, cos, sin)
    k = apply_rope(k, cos, sin)
    o = causal_gqa_attention(q, k, v)
    o = o.transpose(0, 1).reshape(T, nq * d)
    return linear(o, w[prefix + "o_proj.weight"], w.get(prefix + "o_proj.bias"))


def swiglu(x, w, prefix):
    """down(silu(gate(x)) * up(x)), no biases (ondeviceinfer/layers.py:109-113)."""
    gate = linear(x, w[prefix + "gate_proj.weight"])
    up = linear(x, w[prefix + "up_proj.weight"])
    return linear(torch.nn.functional.silu(gate) * up, w[prefix + "down_proj.weight"])


def decoder_layer(h, w, i, cfg, cos, sin):
    """Pre-norm residual block: attention, then feed-forward (ondeviceinfer/model.py:49-63)."""
    p = f"model.layers.{i}."
    eps = cfg["rms_norm_eps"]
    a = rms_norm(h, w[p + "input_layernorm.weight"], eps)
    h = h + attention_block(a, w, p + "self_attn.", cfg, cos, sin)
    m = rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
    return h + swiglu(m, w, p + "mlp.")


def head_dim_of(cfg) -> int:
    """head_dim, defaulting to hidden_size // num_attention_heads (ondeviceinfer/config.py:52-54)."""
    return cfg.get("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])


# --------------------------------------------------------------------------- whole model


def forward_logits(weights, cfg, token_ids, dtype=torch.float32) -> torch.Tensor:
    """Logits [T, vocab] (fp32) at every position of one whole sequence.

    ondeviceinfer/model.py:100-118 (embedding, positions from 0, rotary table, layers,
    final norm) and ondeviceinfer/model.py:161-163 (lm_head without bias); with
    tie_word_embeddings the head is the embedding table (ondeviceinfer/weights.py:77-78).
    """
    w = {k: v.to(dtype) for k, v in weights.items()}
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    h = w["model.embed_tokens.weight"][ids]
    cos, sin = rope_tables(torch.arange(len(ids)), head_dim_of(cfg), cfg["rope_theta"], dtype)
    for i in range(cfg["num_hidden_layers"]):
        h = decoder_layer(h, w, i, cfg, cos, sin)
    h = rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return linear(h, head).float()


# --------------------------------------------------------------------------- sampling


def uniform_draw(seed: int, stream: int, step: int) -> float:
    """The library's counter-based uniform in [0, 1): 24 bits of a 64-bit mix of
    (seed, stream, step).  The reference samples greedily only
    (ondeviceinfer/generation.py:47,58); temperature sampling and its random numbers
    are this library's own definition, restated here from its documentation.
    """
    x = (seed * 0x9E3779B97F4A7C15 + stream * 0xBF58476D1CE4E5B9 + step * 0x94D049BB133111EB
         + 0x2545F4914F6CDD1D) & MASK64
    x ^= x >> 30
    x = (x * 0xBF58476D1CE4E5B9) & MASK64
    x ^= x >> 27
    x = (x * 0x94D049BB133111EB) & MASK64
    x ^= x >> 31
    return (x >> 40) / float(1 << 24)


def sample(logits: torch.Tensor, temperature: float, u: float) -> int:
    """Greedy (temperature 0: first index of the maximum, as the argmax at
    ondeviceinfer/generation.py:47) or inverse-CDF sampling of softmax(logits / T) in
    vocabulary order: the first index whose cumulative weight exceeds u * total."""
    logits = logits.double()
    if temperature == 0.0:
        return int(torch.argmax(logits))
    z = (logits - logits.max()) / temperature
    p = torch.exp(z)
    c = torch.cumsum(p, 0)
    idx = int(torch.searchsorted(c, torch.tensor(u, dtype=torch.float64) * c[-1], right=True))
    return min(idx, logits.numel() - 1)


def generate(weights, cfg, prompt, max_new_tokens, temperature=0.0, seed=0, stream=0,
             stop_ids=(), dtype=torch.float32):
    """Token-by-token generation by recomputing the whole sequence each time.

    ondeviceinfer/generation.py:46-59: max_new_tokens counts the token the prompt
    produces; a stop token is kept in the output and ends the sequence.
    """
    ids = list(prompt)
    out = []
    for step in range(max_new_tokens):
        logits = forward_logits(weights, cfg, ids, dtype)[-1]
        tok = sample(logits, temperature, uniform_draw(seed, stream, step))
        out.append(tok)
        ids.append(tok)
        if tok in stop_ids:
            break
    return out


# --------------------------------------------------------------------------- test models


TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 128, "vocab_size": 256,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 128, "hidden_act": "silu",
}

TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 6,
    "num_key_value_heads": 3, "head_dim": 32, "intermediate_size": 160, "vocab_size": 389,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "max_position_embeddings": 256, "hidden_act": "silu", "eos_token_id": 7,
}

# A third shape for long contexts: head_dim 128 like the large models, 1 q head per kv
# head group of 3, a width and a vocabulary that are no power of two.
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 80, "num_attention_heads": 3,
    "num_key_value_heads": 1, "head_dim": 128, "intermediate_size": 208, "vocab_size": 523,
    "rope_theta": 50000.0, "rms_norm_eps": 3e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 4096, "hidden_act": "silu",
}


# The same three with a bias on the four attention projections (``attention_bias``,
# ondeviceinfer/config.py:59 and ondeviceinfer/attention.py:106-129), under seeds of their own.
TINY_A_BIAS = dict(TINY_A, attention_bias=True)
TINY_B_BIAS = dict(TINY_B, attention_bias=True)
TINY_C_BIAS = dict(TINY_C, attention_bias=True)


# A shape that the tensor-core kernels refuse in places: a width of 100 (no multiple of 8, so its products go to the
# vendor library and its logits through the fp32 kernel), heads of 48, as many key/value heads as query heads,
# biases on the attention projections.
TINY_D = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 100, "num_attention_heads": 5,
    "num_key_value_heads": 5, "head_dim": 48, "intermediate_size": 136, "vocab_size": 301,
    "rope_theta": 20000.0, "rms_norm_eps": 2e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 512, "hidden_act": "silu", "attention_bias": True,
}


def tensor_shapes(cfg):
    """Checkpoint tensor names and shapes, in file order (module tree of
    ondeviceinfer/model.py:27-38,77-89,137-144)."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], head_dim_of(cfg)
    shapes = {"model.embed_tokens.weight": (V, H)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        shapes[p + "input_layernorm.weight"] = (H,)
        shapes[p + "self_attn.q_proj.weight"] = (nq * d, H)
        shapes[p + "self_attn.k_proj.weight"] = (nkv * d, H)
        shapes[p + "self_attn.v_proj.weight"] = (nkv * d, H)
        shapes[p + "self_attn.o_proj.weight"] = (H, nq * d)
        if cfg.get("attention_bias", False):          # bias=config.attention_bias, ondeviceinfer/attention.py:106-129
            shapes[p + "self_attn.q_proj.bias"] = (nq * d,)
            shapes[p + "self_attn.k_proj.bias"] = (nkv * d,)
            shapes[p + "self_attn.v_proj.bias"] = (nkv * d,)
            shapes[p + "self_attn.o_proj.bias"] = (H,)
        shapes[p + "self_attn.q_norm.weight"] = (d,)
        shapes[p + "self_attn.k_norm.weight"] = (d,)
        shapes[p + "post_attention_layernorm.weight"] = (H,)
        shapes[p + "mlp.gate_proj.weight"] = (I, H)
        shapes[p + "mlp.up_proj.weight"] = (I, H)
        shapes[p + "mlp.down_proj.weight"] = (H, I)
    shapes["model.norm.weight"] = (H,)
    if not cfg["tie_word_embeddings"]:
        shapes["lm_head.weight"] = (V, H)
    return shapes


def random_weights(cfg, seed, std=0.02, norm_std=0.01):
    """The tests' own random weights: normal(0, std) matrices, 1 + normal(0, norm_std)
    norm weights, rounded to bfloat16 so that a bf16 and an fp32 run hold the same values."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        t = torch.randn(shape, generator=gen, dtype=torch.float32)
        t = 1.0 + norm_std * t if len(shape) == 1 and not name.endswith(".bias") else std * t
        out[name] = t.to(torch.bfloat16)
    return out


def random_prompts(cfg, lengths, seed):
    gen = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist() for n in lengths]
