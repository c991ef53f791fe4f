"""Plain, slow implementation of the Llama decoder for the tests: whole sequences,
no cache, one function per part, double precision, no code shared with the
product path (it imports nothing from mstar_b200).

Written from the reference's formulas; every function cites the file and lines
of t-avil/mstar it restates.  Where the reference delegates the arithmetic to a
library (RMSNorm, rotary encoding with llama3 scaling, attention, sampling) the
function says so and states the formula it rests on.  The one deliberate
deviation from exact real arithmetic: rotary angles are float32(position) *
float32(inv_freq) rounded to float32, because the engine's contract is that
rotation angles are 32-bit; sine and cosine of that angle are then taken in
double precision.

Weights are a dict of checkpoint-named tensors (model.layers.N.self_attn.q_proj.weight
and so on); ``cfg`` is the dict of config.json keys.  Everything is computed where the
weights live (the large-size tests keep them on the GPU to have the float64 products
done there; the arithmetic is the same).

``act``: an optional function applied to every activation at the places where the engine
stores one in its compute dtype (normed rows; q, k, v; rotated q and k; the attention
output; each projection's output; gate, up and their product).  With ``round_bf16`` it
gives the second oracle of the bfloat16 tests: the same float64 arithmetic on activations
that were rounded where the engine rounds them, so that what remains between it and the
engine is the order of the sums and the attention kernels' internal roundings.
"""
from __future__ import annotations

import math

import torch

DT = torch.float64


def _keep(x):
    return x


def round_bf16(x: torch.Tensor) -> torch.Tensor:
    """Round to bfloat16 (nearest even) and return to float64."""
    return x.to(torch.bfloat16).to(DT)


def plain_rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2, -1) + eps) * weight -- Llama mode, multiply by the weight.
    mstar/model/components/norm.py:45-59 (the library call) and the same formula spelled
    out at mstar/utils/attention.py:457-474 and norm.py:48-51."""
    x = x.to(DT)
    var = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * weight.to(DT)


def plain_rope_frequencies(cfg: dict) -> torch.Tensor:
    """inv_freq_j = theta^(-2j/hd), then the llama3 rule when rope_scaling asks for it.
    Unscaled formula: mstar/utils/attention.py:224-253.  The reference passes factor,
    low_freq_factor, high_freq_factor and the original context length to a library
    (mstar/engine/cache_manager.py:752-759; values mstar/model/orpheus/config.py:17-23)
    and does not spell the rule out; it is: wavelength L = 2*pi/inv_freq; L < C/high keeps
    inv_freq; L > C/low gives inv_freq/factor; between, s = (C/L - low)/(high - low) and
    inv_freq' = (1-s)*inv_freq/factor + s*inv_freq."""
    hd = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
    j = torch.arange(0, hd, 2, dtype=DT)
    inv = float(cfg["rope_theta"]) ** (-j / hd)
    rs = cfg.get("rope_scaling")
    if rs and rs.get("rope_type", rs.get("type")) == "llama3":
        factor, low, high = float(rs["factor"]), float(rs["low_freq_factor"]), float(
            rs["high_freq_factor"])
        ctx = float(rs["original_max_position_embeddings"])
        wavelen = 2 * math.pi / inv
        smooth = (ctx / wavelen - low) / (high - low)
        mid = (1 - smooth) * inv / factor + smooth * inv
        inv = torch.where(wavelen < ctx / high, inv, torch.where(wavelen > ctx / low,
                                                                 inv / factor, mid))
    return inv


def plain_apply_rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor):
    """Split-half rotation of x [T, heads, hd]: pairs (x[j], x[j+hd/2]);
    out1 = x1 cos - x2 sin, out2 = x2 cos + x1 sin (mstar/utils/attention.py:224-253;
    the same rotate-half form in test/modular/test_fused_rmsnorm.py:12-45).  Angles are
    rounded to float32 (see the module docstring)."""
    hd = x.shape[-1]
    ang32 = (positions.to(torch.float32)[:, None]
             * inv_freq.to(positions.device, torch.float32)[None, :])
    ang = ang32.to(DT)
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x1, x2 = x[..., : hd // 2].to(DT), x[..., hd // 2:].to(DT)
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


def plain_attention(q, k, v, scale=None, window=None, round_probs=None):
    """Causal grouped-query attention of a whole sequence.  q [T, nh, hd], k, v
    [T, nkv, hd]; query head i uses kv head i // (nh/nkv); scores * hd^-0.5 (the
    reference passes no scale, i.e. the library default; its own kernels and tests use
    hd^-0.5: mstar/utils/attention.py:116-117, test/modular/
    test_pi05_reference_equivalence.py:692); causal mask (mstar/model/orpheus/
    submodules.py:122); softmax; P.V (mstar/engine/cache_manager.py:653-701).
    ``window`` W lets token p see keys p-W+1..p (not used by Llama).
    ``round_probs``: a function applied to the unnormalised probabilities exp(s - max)
    before they multiply V (tensor-core attention kernels hold them in bfloat16 there);
    the normaliser is the sum of the unrounded ones.  Only the tests' yardstick for what
    such a kernel-internal rounding can do uses it."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    scale = hd ** -0.5 if scale is None else scale
    out = torch.empty(T, nh, hd, dtype=DT, device=q.device)
    idx = torch.arange(T, device=q.device)
    mask = idx[None, :] <= idx[:, None]
    if window is not None:
        mask &= idx[None, :] > idx[:, None] - window
    for h in range(nh):
        kh, vh = k[:, h // group].to(DT), v[:, h // group].to(DT)
        s = (q[:, h].to(DT) @ kh.T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        if round_probs is None:
            out[:, h] = torch.softmax(s, dim=-1) @ vh
        else:
            e = torch.exp(s - s.max(dim=-1, keepdim=True).values)
            out[:, h] = (round_probs(e) @ vh) / e.sum(dim=-1, keepdim=True)
    return out


def plain_swiglu(x, w_gate, w_up, w_down, act=_keep):
    """down(silu(gate(x)) * up(x)), no bias (mstar/model/components/distributed/
    mlp.py:78-81; activation "silu" fixed at mstar/model/orpheus/components/
    language_model.py:48)."""
    x = x.to(DT)
    g = act(x @ w_gate.to(DT).T)
    u = act(x @ w_up.to(DT).T)
    return act(act((g * torch.sigmoid(g)) * u) @ w_down.to(DT).T)


def plain_self_attention(x, w, prefix, cfg, positions, inv_freq, window=None, act=_keep,
                         round_probs=None):
    """q/k/v projections, view as heads, rotary on q and k, attention, output
    projection (mstar/model/components/distributed/attention.py:98-110, 138-149)."""
    nh, nkv = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg[
        "num_attention_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // nh
    T = x.shape[0]
    x = x.to(DT)
    q = act((x @ w[f"{prefix}.q_proj.weight"].to(DT).T)).view(T, nh, hd)
    k = act((x @ w[f"{prefix}.k_proj.weight"].to(DT).T)).view(T, nkv, hd)
    v = act((x @ w[f"{prefix}.v_proj.weight"].to(DT).T)).view(T, nkv, hd)
    q = act(plain_apply_rope(q, positions, inv_freq))
    k = act(plain_apply_rope(k, positions, inv_freq))
    a = act(plain_attention(q, k, v, window=window, round_probs=round_probs).reshape(T, nh * hd))
    return act(a @ w[f"{prefix}.o_proj.weight"].to(DT).T)


def plain_decoder_layer(h, w, i, cfg, positions, inv_freq, act=_keep, round_probs=None):
    """Pre-norm block with plain residual adds
    (mstar/model/components/decoder_layer.py:58-71)."""
    p = f"model.layers.{i}"
    eps = cfg["rms_norm_eps"]
    x = act(plain_rms_norm(h, w[f"{p}.input_layernorm.weight"], eps))
    h = h + plain_self_attention(x, w, f"{p}.self_attn", cfg, positions, inv_freq, act=act,
                                 round_probs=round_probs)
    y = act(plain_rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], eps))
    return h + plain_swiglu(y, w[f"{p}.mlp.gate_proj.weight"], w[f"{p}.mlp.up_proj.weight"],
                            w[f"{p}.mlp.down_proj.weight"], act=act)


def plain_hidden_states(w: dict, cfg: dict, token_ids, act=_keep, round_probs=None) -> torch.Tensor:
    """embed -> layers -> final norm (mstar/model/orpheus/components/
    language_model.py:72-83; embedding lookup without scaling, mstar/model/components/
    distributed/embedding.py:98-99)."""
    table = w["model.embed_tokens.weight"]
    ids = torch.as_tensor(token_ids, dtype=torch.long, device=table.device)
    positions = torch.arange(ids.numel(), device=table.device)
    inv_freq = plain_rope_frequencies(cfg)
    h = table[ids].to(DT)
    for i in range(cfg["num_hidden_layers"]):
        h = plain_decoder_layer(h, w, i, cfg, positions, inv_freq, act=act,
                                round_probs=round_probs)
    return act(plain_rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"]))


def plain_logits(w: dict, cfg: dict, token_ids, act=_keep, round_probs=None) -> torch.Tensor:
    """Logits at every position, [T, vocab], float64.  The head is lm_head.weight, or
    the embedding table when the configuration ties them (the reference has no tying
    code: mstar/model/orpheus/components/language_model.py:95-101; tying is this
    engine's reading of config.json's tie_word_embeddings)."""
    hidden = plain_hidden_states(w, cfg, token_ids, act=act, round_probs=round_probs)
    head = w.get("lm_head.weight")
    if head is None or cfg.get("tie_word_embeddings"):
        head = w["model.embed_tokens.weight"]
    return hidden @ head.to(DT).T


def plain_greedy(w: dict, cfg: dict, prompt, num_new: int) -> list:
    """Greedy continuation by recomputing the whole sequence for every token."""
    ids = list(prompt)
    out = []
    for _ in range(num_new):
        nxt = int(torch.argmax(plain_logits(w, cfg, ids)[-1]))
        out.append(nxt)
        ids.append(nxt)
    return out


# ----------------------------------------------------------------- sampling
def plain_philox4x32_10(key: int, counter: int) -> list:
    """Philox4x32-10 with a 64-bit key and a 64-bit counter in the low two words."""
    M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
    mask = 0xFFFFFFFF
    k0, k1 = key & mask, (key >> 32) & mask
    c = [counter & mask, (counter >> 32) & mask, 0, 0]
    for _ in range(10):
        p0, p1 = M0 * c[0], M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k0) & mask, p1 & mask, ((p0 >> 32) ^ c[3] ^ k1) & mask,
             p0 & mask]
        k0, k1 = (k0 + W0) & mask, (k1 + W1) & mask
    return c


def plain_uniform(seed: int, offset: int) -> float:
    return (plain_philox4x32_10(seed, offset)[0] >> 8) / 16777216.0


def plain_sampling_distribution(logits, temperature, top_k=0, top_p=1.0, penalty=1.0,
                                seen=None) -> torch.Tensor:
    """Probabilities a token is drawn from (float64, zeros outside the kept set).
    Penalty on seen tokens x>0 ? x/p : x*p (mstar/utils/sampling.py:97-98); division by
    the temperature and softmax (:131-150); top-k then top-p on the renormalised rest
    (the reference hands both to a library, :484-502); ties with the last kept token are
    kept."""
    x = logits.to(DT).clone()
    if seen is not None and penalty != 1.0:
        pen = torch.where(x > 0, x / penalty, x * penalty)
        x = torch.where(seen.bool(), pen, x)
    p = torch.softmax(x / temperature, dim=-1)
    if top_k and top_k < x.numel():
        kth = torch.topk(p, top_k).values[-1]
        p = torch.where(p >= kth, p, torch.zeros_like(p))
        p = p / p.sum()
    if top_p < 1.0:
        sp, _ = torch.sort(p, descending=True)
        csum = torch.cumsum(sp, 0)
        n_keep = int((csum < top_p).sum()) + 1
        cut = sp[min(n_keep, sp.numel()) - 1]
        p = torch.where(p >= cut, p, torch.zeros_like(p))
        p = p / p.sum()
    return p
