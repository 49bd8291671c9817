"""An independent float64 numpy model of a Llama forward pass (no KV cache: the whole sequence is
recomputed with a causal mask).  Used to cross-check the C oracle's structure (head mapping, RoPE
convention, cache bookkeeping); it shares no code with it."""
import numpy as np


def rope(x, positions, theta):
    # x [..., S, D]; half-split convention: pairs (j, j + D/2)
    d = x.shape[-1]
    half = d // 2
    freq = 1.0 / theta ** (np.arange(half, dtype=np.float64) * 2.0 / d)
    ang = positions[:, None].astype(np.float64) * freq[None, :]
    c, s = np.cos(ang), np.sin(ang)
    x1, x2 = x[..., :half], x[..., half:]
    return np.concatenate([x1 * c - x2 * s, x2 * c + x1 * s], axis=-1)


def rmsnorm(x, w, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


def llama_logits(cfg, params, ids):
    """ids [B,S] -> logits [B,S,V] in float64."""
    P = {k: v.astype(np.float64) for k, v in params.items()}
    H, hq, hkv = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = cfg.get("head_dim") or H // hq
    eps, theta = cfg["rms_norm_eps"], cfg["rope_theta"]
    b, s = ids.shape
    x = P["model.embed_tokens.weight"][ids.astype(np.int64)]
    pos = np.arange(s)
    mask = np.triu(np.full((s, s), -np.inf), k=1)
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        nx = rmsnorm(x, P[p + "input_layernorm.weight"], eps)
        q = (nx @ P[p + "self_attn.q_proj.weight"].T).reshape(b, s, hq, d).transpose(0, 2, 1, 3)
        k = (nx @ P[p + "self_attn.k_proj.weight"].T).reshape(b, s, hkv, d).transpose(0, 2, 1, 3)
        v = (nx @ P[p + "self_attn.v_proj.weight"].T).reshape(b, s, hkv, d).transpose(0, 2, 1, 3)
        if cfg.get("qk_norm"):
            q = rmsnorm(q, P[p + "self_attn.q_norm.weight"], eps)
            k = rmsnorm(k, P[p + "self_attn.k_norm.weight"], eps)
        q, k = rope(q, pos, theta), rope(k, pos, theta)
        k = np.repeat(k, hq // hkv, axis=1)
        v = np.repeat(v, hq // hkv, axis=1)
        sc = q @ k.transpose(0, 1, 3, 2) / np.sqrt(d) + mask
        sc = np.exp(sc - sc.max(-1, keepdims=True))
        pr = sc / sc.sum(-1, keepdims=True)
        att = (pr @ v).transpose(0, 2, 1, 3).reshape(b, s, hq * d)
        x = x + att @ P[p + "self_attn.o_proj.weight"].T
        nh = rmsnorm(x, P[p + "post_attention_layernorm.weight"], eps)
        g = nh @ P[p + "mlp.gate_proj.weight"].T
        u = nh @ P[p + "mlp.up_proj.weight"].T
        x = x + ((g / (1.0 + np.exp(-g))) * u) @ P[p + "mlp.down_proj.weight"].T
    x = rmsnorm(x, P["model.norm.weight"], eps)
    return x @ P["lm_head.weight"].T
