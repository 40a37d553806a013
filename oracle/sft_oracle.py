"""CPU restatement of the reference's LoRA-SFT step (Qwen3 branch). TEST INFRASTRUCTURE ONLY.

Nothing under llm.metal_b200/ may import this file; it is the checker the GPU engine is compared with.

It follows, operation by operation, src/nn/fast_sft.c (forward_to_logits :616-752 Qwen3 branch,
sft_apply_ce_loss :754-760, sft_backward_ex :766-982 LoRA branch, clip_grad_norm :1060-1088,
adamw_update :1045-1058, lora_update :1090-1107, sft_train_step :1113-1157, sft_save_lora :1255-1285)
with the per-kernel arithmetic of shaders/q8_kernels.metal (line numbers at each function).

It also restates the Gemma3 block order of the same functions (four norms per layer, GeGLU, scaled and tied
embeddings, a RoPE base per layer: the is_gemma3 branches of :697-738 and :797-888), the full-parameter mode (every
matrix stepped inside the backward pass, or accumulated and applied: :778-785 and the like, :996-1039) and the
GRPO step's policy-gradient kernel.

Parity status: PINNED. The reference's own fast_sft.c, compiled unmodified over a CPU stand-in for its
Metal dispatch layer (oracle/fast_metal_cpu.c -> oracle/_ref/libllmref_fast.so), produced
tests/golden/sft_golden.npz (tests/golden/make_sft_golden.py): three training steps on the tiny Qwen3
configuration. tests/test_cpu_pinned_by_reference_engines.py holds this file to those vectors within 1e-5
(loss, per-position losses, all 4*L gradient buffers of every step, the weights and the adapter file after
the third). The same file holds the Gemma3 branch to tests/golden/sft_golden_gemma3.npz (three steps of
sft_state_create_gemma3 + sft_train_step, 1e-5 on everything) and the full-parameter mode to
tests/golden/sft_golden_full.npz (losses 1e-5; more than 99.5 % of the sampled binary16 weights bit-equal after
three stepping calls, and after two accumulating calls and one apply). Independent cross-checks remain: a float64 torch-autograd model of the same network, finite
differences, and the decode oracle's logits for the forward half.

`dtype` selects float32 (as the reference computes) or float64 (to separate rounding from logic).
A batch of S sequences is handled as S independent passes whose LoRA gradients are averaged; S = 1
is exactly the reference's step.
"""
import struct

import numpy as np


def f16_round(w):
    """Weights as the F16 WMat holds them (src/nn/wmat.c wmat_create_f16), widened again."""
    return np.asarray(w, dtype=np.float32).astype(np.float16).astype(np.float32)


class Weights:
    """Frozen base of one Qwen3-architecture model; matrices already rounded to binary16 values."""

    def __init__(self, cfg, layers, lm_head, final_norm, token_emb):
        self.cfg = dict(cfg)          # d_model n_q_heads n_kv_heads head_dim intermediate_size vocab_size n_layers rope_theta eps
        self.layers = layers          # list of dict: q k v o gate up down input_norm post_attn_norm q_norm k_norm
        self.lm_head = lm_head
        self.final_norm = final_norm
        self.token_emb = token_emb


class LoRA:
    """A_q[R,D] B_q[Hq*hd,R] A_v[R,D] B_v[Hkv*hd,R] per layer (fast_sft.c:89-131) + AdamW moments."""

    def __init__(self, layers, rank, alpha):
        self.p = [{k: np.array(v, dtype=np.float32) for k, v in l.items()} for l in layers]
        self.m = [{k: np.zeros_like(v) for k, v in l.items()} for l in self.p]
        self.v = [{k: np.zeros_like(v) for k, v in l.items()} for l in self.p]
        self.rank = rank
        self.scaling = np.float32(alpha) / np.float32(rank)      # fast_sft.c:192
        self.step_count = 0


KEYS = ("A_q", "B_q", "A_v", "B_v")


# ---- kernels -------------------------------------------------------------------------------------

def rms_norm(x, gamma, eps):
    """q8_kernels.metal:133-158: x * rsqrt(mean(x^2) + eps) * gamma, row-wise."""
    t = x.dtype.type
    ms = (x * x).sum(axis=-1, keepdims=True) / t(x.shape[-1])
    inv = t(1) / np.sqrt(ms + t(eps))
    return x * inv * gamma


def rms_norm_backward(x, dy, gamma, eps):
    """q8_kernels.metal:584-624."""
    t = x.dtype.type
    dim = t(x.shape[-1])
    inv = t(1) / np.sqrt((x * x).sum(axis=-1, keepdims=True) / dim + t(eps))
    coeff = (dy * gamma * x).sum(axis=-1, keepdims=True) * inv * inv / dim
    return (gamma * dy - coeff * x) * inv


def rope_angles(n, hd, theta, t):
    """q8_kernels.metal:531-534: freq = 1/pow(theta, 2d/hd), angle = pos*freq (fp32 arithmetic)."""
    d = np.arange(hd // 2, dtype=np.float32)
    freq = (np.float32(1.0) / np.power(np.float32(theta), (2 * d) / np.float32(hd), dtype=np.float32)).astype(np.float32)
    ang = (np.arange(n, dtype=np.float32)[:, None] * freq[None, :]).astype(np.float32)
    return np.cos(ang.astype(np.float64)).astype(t), np.sin(ang.astype(np.float64)).astype(t)


def rope(x, cos, sin, inverse=False):
    """x [H,N,hd]; rope_train :495-538 and rope_train_bwd :997-1040 (rotation by -angle)."""
    h = x.shape[-1] // 2
    x0, x1 = x[..., :h], x[..., h:]
    if inverse:
        return np.concatenate([x0 * cos + x1 * sin, -x0 * sin + x1 * cos], axis=-1)
    return np.concatenate([x0 * cos - x1 * sin, x0 * sin + x1 * cos], axis=-1)


def heads_fwd(x, H, hd):
    """[N, H*hd] -> [H, N, hd] (transpose_heads_fwd :438-454)."""
    n = x.shape[0]
    return np.ascontiguousarray(x.reshape(n, H, hd).transpose(1, 0, 2))


def heads_rev(x):
    """[H, N, hd] -> [N, H*hd] (transpose_heads_rev :457-473)."""
    H, n, hd = x.shape
    return np.ascontiguousarray(x.transpose(1, 0, 2).reshape(n, H * hd))


def attn_fwd(q, k, v, scale):
    """attn_train_fwd :769-851: causal softmax(q k^T * scale) v, probabilities kept. [H,N,hd]."""
    t = q.dtype.type
    n = q.shape[1]
    s = np.einsum("hid,hjd->hij", q, k) * t(scale)
    mask = np.tril(np.ones((n, n), dtype=bool))
    s = np.where(mask, s, t(-1e30))
    s = s - s.max(axis=-1, keepdims=True)
    e = np.where(mask, np.exp(s), t(0))
    p = e * (t(1) / e.sum(axis=-1, keepdims=True))
    return np.einsum("hij,hjd->hid", p, v), p


def attn_bwd(d_out, p, q, k, v, scale):
    """attn_bwd_dq :857-925 and attn_bwd_dkv :931-968."""
    t = q.dtype.type
    n = q.shape[1]
    mask = np.tril(np.ones((n, n), dtype=bool))
    d_raw = np.where(mask, np.einsum("hid,hjd->hij", d_out, v), t(0))
    dp_sum = (p * d_raw).sum(axis=-1, keepdims=True)
    ds = np.where(mask, p * (d_raw - dp_sum) * t(scale), t(0))
    dq = np.einsum("hij,hjd->hid", ds, k)
    dk = np.einsum("hij,hid->hjd", ds, q)
    dv = np.einsum("hij,hid->hjd", p, d_out)
    return dq, dk, dv


def silu_mul(g, u):
    """silu_mul :337-348."""
    t = g.dtype.type
    return g / (t(1) + np.exp(-g)) * u


def silu_mul_backward(dy, g, u):
    """silu_mul_backward :540-556."""
    t = g.dtype.type
    sig = t(1) / (t(1) + np.exp(-g))
    return dy * u * (sig * (t(1) + g * (t(1) - sig))), dy * (g * sig)


def gelu_mul(g, u):
    """gelu_mul, shaders/q8_kernels.metal:351-363 (Gemma3's GeGLU): tanh form, its argument clamped to +-15."""
    g = np.asarray(g, dtype=np.float32)
    inner = np.clip(np.float32(0.7978845608) * (g + np.float32(0.044715) * g * g * g), -15.0, 15.0).astype(np.float32)
    return (np.float32(0.5) * g * (np.float32(1.0) + np.tanh(inner)) * u).astype(np.float32)


def gelu_mul_backward(dy, g, u):
    """gelu_mul_backward, shaders/q8_kernels.metal:561-580: returns (d_gate, d_up)."""
    g = np.asarray(g, dtype=np.float32)
    inner = np.clip(np.float32(0.7978845608) * (g + np.float32(0.044715) * g * g * g), -15.0, 15.0).astype(np.float32)
    th = np.tanh(inner)
    gelu_g = np.float32(0.5) * g * (1.0 + th)
    grad = 0.5 * (1.0 + th) + 0.5 * g * (1.0 - th * th) * np.float32(0.7978845608) * (1.0 + 3.0 * np.float32(0.044715) * g * g)
    return (dy * u * grad).astype(np.float32), (dy * gelu_g).astype(np.float32)


def softmax_ce(logits, targets):
    """softmax_ce_train :646-690: loss = logsumexp - logit[target]; dlogits = softmax - onehot."""
    mx = logits.max(axis=-1, keepdims=True)
    lse = np.log(np.exp(logits - mx).sum(axis=-1, keepdims=True)) + mx
    rows = np.arange(logits.shape[0])
    losses = (lse[:, 0] - logits[rows, targets]).astype(logits.dtype)
    d = np.exp(logits - lse)
    d[rows, targets] -= logits.dtype.type(1)
    return losses, d


# ---- forward / backward over one sequence ----------------------------------------------------------

def grpo_policy_grad(logits, actions, old_logprobs, advantages, clip_eps):
    """grpo_policy_grad, shaders/q8_kernels.metal:698-761, one row per position: returns (new_logprobs [N],
    dlogits [N, V]). PPO clip: a position whose ratio already sits on the far side of the clip interval
    (above 1 + eps with a positive advantage, below 1 - eps with a negative one) contributes nothing.
    Pinned together with the step that uses it: tests/golden/grpo_golden.bin is the record of the reference's
    own src/nn/fast_grpo.c over its engines on the CPU stand-in for the Metal layer, and the `new log-prob`
    and gradient sections of that record come out of the C restatement of this kernel
    (oracle/fast_metal_cpu.c)."""
    logits = np.asarray(logits, dtype=np.float32)
    n, v = logits.shape
    mx = logits.max(axis=1, keepdims=True)
    lse = (np.log(np.exp(logits - mx, dtype=np.float32).sum(axis=1, dtype=np.float32)) + mx[:, 0]).astype(np.float32)
    a = np.asarray(actions, dtype=np.int64)
    new_lp = (logits[np.arange(n), a] - lse).astype(np.float32)
    ratio = np.exp(new_lp - np.asarray(old_logprobs, dtype=np.float32), dtype=np.float32)
    clipped = np.clip(ratio, np.float32(1.0 - clip_eps), np.float32(1.0 + clip_eps))
    adv = np.asarray(advantages, dtype=np.float32)
    weight = np.where(adv >= 0, np.where(ratio <= clipped, -adv, 0.0), np.where(ratio >= clipped, -adv, 0.0)).astype(np.float32)
    prob = np.exp(logits - lse[:, None], dtype=np.float32)
    prob[np.arange(n), a] -= 1.0
    return new_lp, ((weight * ratio)[:, None] * prob).astype(np.float32)


def layer_theta(c, L):
    """RoPE base of layer L: one for all (Qwen3) or per layer (Gemma3: every sixth layer global, :310-313)."""
    return c["rope_thetas"][L] if "rope_thetas" in c else c["rope_theta"]


def forward(w, lora, tokens, dtype=np.float32):
    """forward_to_logits (fast_sft.c:616-752) after the embedding gather of sft_train_step (:1118-1120).
    Returns (logits [N,V], saves)."""
    c, t = w.cfg, dtype
    D, Hq, Hkv, hd = c["d_model"], c["n_q_heads"], c["n_kv_heads"], c["head_dim"]
    eps = c["eps"]
    gemma = bool(c.get("gemma"))          # Gemma3 block order (:697-704, :716-738); lora None: a full-parameter state
    sc = t(lora.scaling) if lora is not None else t(0)
    G = Hq // Hkv
    n = len(tokens)
    scale = np.float32(1.0) / np.sqrt(np.float32(hd))
    x = w.token_emb[np.asarray(tokens, dtype=np.int64)].astype(t)
    if gemma:
        x = x * t(np.sqrt(np.float32(D)))                                        # emb_scale (:302, :1124-1126)
    saves = []
    for L, lw in enumerate(w.layers):
        W = {k: v.astype(t) for k, v in lw.items()}
        sv = {"x_in": x}
        ln1 = rms_norm(x, W["input_norm"], eps)
        sv["ln1"] = ln1
        q, k, v = ln1 @ W["q"].T, ln1 @ W["k"].T, ln1 @ W["v"].T
        if lora is not None:
            lp = {k_: v_.astype(t) for k_, v_ in lora.p[L].items()}
            q_mid, v_mid = ln1 @ lp["A_q"].T, ln1 @ lp["A_v"].T
            q = q + sc * (q_mid @ lp["B_q"].T)
            v = v + sc * (v_mid @ lp["B_v"].T)
            sv["q_mid"], sv["v_mid"] = q_mid, v_mid
        q_t, k_t, v_t = heads_fwd(q, Hq, hd), heads_fwd(k, Hkv, hd), heads_fwd(v, Hkv, hd)
        sv["q_pre"], sv["k_pre"] = q_t, k_t
        cos, sin = rope_angles(n, hd, layer_theta(c, L), t)
        q_f = rope(rms_norm(q_t, W["q_norm"], eps), cos, sin)
        k_f = rope(rms_norm(k_t, W["k_norm"], eps), cos, sin)
        k_exp, v_exp = np.repeat(k_f, G, axis=0), np.repeat(v_t, G, axis=0)      # repeat_kv :476-492
        sv["q_final"], sv["k_exp"], sv["v_exp"] = q_f, k_exp, v_exp
        att, probs = attn_fwd(q_f, k_exp, v_exp, scale)
        sv["probs"] = probs
        sv["attn_flat"] = heads_rev(att)
        if gemma:
            sv["o_out"] = sv["attn_flat"] @ W["o"].T
            x = x + rms_norm(sv["o_out"], W["post_attn_norm"], eps)
            sv["x_mid"] = x
            ln2 = rms_norm(x, W["pre_ff_norm"], eps)
        else:
            x = x + sv["attn_flat"] @ W["o"].T
            sv["x_mid"] = x
            ln2 = rms_norm(x, W["post_attn_norm"], eps)
        sv["ln2"] = ln2
        g, u = ln2 @ W["gate"].T, ln2 @ W["up"].T
        sv["gate_pre"], sv["up"] = g, u
        sv["act"] = gelu_mul(g, u).astype(t) if gemma else silu_mul(g, u)
        if gemma:
            sv["ff_raw"] = sv["act"] @ W["down"].T
            x = x + rms_norm(sv["ff_raw"], W["post_ff_norm"], eps)
        else:
            x = x + sv["act"] @ W["down"].T
        saves.append(sv)
    fin = {"x_final": x, "ln_final": rms_norm(x, w.final_norm.astype(t), eps)}
    logits = fin["ln_final"] @ w.lm_head.astype(t).T
    return logits, (saves, fin)


class SGD:
    """What a full-parameter backward pass does with a weight gradient dW = dY^T X (fast_sft.c:778-785 and the
    like): step the binary16 weight at once, W <- half(W - lr dW) (f16_sgd_fused, q8_kernels.metal:1097-1125), or,
    once accumulators exist, G <- half(G + dW) (f16_grad_accum, :1164-1191) and leave W alone."""

    def __init__(self, lr, accum=None):
        self.lr, self.accum = np.float32(lr), accum

    def take(self, holder, key, dY, X, where):
        dW = (np.asarray(dY, np.float32).T @ np.asarray(X, np.float32)).astype(np.float32)
        if self.accum is not None:
            g = self.accum[where]
            g[key] = f16_round(g[key] + dW)
        else:
            holder[key] = f16_round(holder[key] - self.lr * dW)


def new_accum(w):
    """sft_alloc_grad_accum (fast_sft.c:996-1019): zeroed accumulators, one per matrix; index = layer, -1 = LM head."""
    acc = {L: {k: np.zeros_like(lw[k], dtype=np.float32) for k in ("q", "k", "v", "o", "gate", "up", "down")}
           for L, lw in enumerate(w.layers)}
    acc[-1] = {"lm_head": np.zeros_like(w.lm_head, dtype=np.float32)}
    return acc


def apply_accum(w, acc, lr):
    """sft_apply_grad_sgd (:1021-1039): W <- half(W - lr G), G <- 0."""
    lr = np.float32(lr)
    for L, lw in enumerate(w.layers):
        for k in ("q", "k", "v", "o", "gate", "up", "down"):
            lw[k] = f16_round(lw[k] - lr * acc[L][k])
            acc[L][k][...] = 0
    w.lm_head = f16_round(w.lm_head - lr * acc[-1]["lm_head"])
    acc[-1]["lm_head"][...] = 0


def backward(w, lora, saved, dlogits, sgd=None):
    """sft_backward_ex (fast_sft.c:766-982). Returns the per-layer dict of LoRA gradients (None entries for a
    full-parameter state, lora None). With `sgd` (full-parameter mode) every matrix takes its gradient as the
    pass goes, in the reference's order: the LM head, down, gate, up and o after the product that sends the
    gradient on through them, q, k and v before it (:922-945) -- w is changed in place."""
    c = w.cfg
    t = dlogits.dtype.type
    Hq, Hkv, hd = c["n_q_heads"], c["n_kv_heads"], c["head_dim"]
    eps, G = c["eps"], Hq // Hkv
    gemma = bool(c.get("gemma"))
    sc = t(lora.scaling) if lora is not None else t(0)
    n = dlogits.shape[0]
    scale = np.float32(1.0) / np.sqrt(np.float32(hd))
    saves, fin = saved
    dx = dlogits @ w.lm_head.astype(t)                                            # :777
    if sgd is not None:
        holder = {"lm_head": w.lm_head}
        sgd.take(holder, "lm_head", dlogits, fin["ln_final"], -1)
        w.lm_head = holder["lm_head"]
    dx = rms_norm_backward(fin["x_final"], dx, w.final_norm.astype(t), eps)       # :788-790
    grads = [None] * len(w.layers)
    for L in range(len(w.layers) - 1, -1, -1):
        lw = w.layers[L]
        W = {k: v.astype(t) for k, v in lw.items()}
        sv = saves[L]
        if gemma:
            # FFN, Gemma3 (:797-838)
            dff = rms_norm_backward(sv["ff_raw"], dx, W["post_ff_norm"], eps)
            d_act = dff @ W["down"]
            if sgd is not None:
                sgd.take(lw, "down", dff, sv["act"], L)
            dg, du = gelu_mul_backward(d_act, sv["gate_pre"], sv["up"])
            dg, du = dg.astype(t), du.astype(t)
        else:
            # FFN (:841-872)
            d_act = dx @ W["down"]
            if sgd is not None:
                sgd.take(lw, "down", dx, sv["act"], L)
            dg, du = silu_mul_backward(d_act, sv["gate_pre"], sv["up"])
        dln = dg @ W["gate"]
        if sgd is not None:
            sgd.take(lw, "gate", dg, sv["ln2"], L)
        dln = dln + du @ W["up"]
        if sgd is not None:
            sgd.take(lw, "up", du, sv["ln2"], L)
        dx = dx + rms_norm_backward(sv["x_mid"], dln, W["pre_ff_norm"] if gemma else W["post_attn_norm"], eps)
        # attention (:875-918)
        d_o = rms_norm_backward(sv["o_out"], dx, W["post_attn_norm"], eps) if gemma else dx
        d_att = heads_fwd(d_o @ W["o"], Hq, hd)
        if sgd is not None:
            sgd.take(lw, "o", d_o, sv["attn_flat"], L)
        dq, dk_e, dv_e = attn_bwd(d_att, sv["probs"], sv["q_final"], sv["k_exp"], sv["v_exp"], scale)
        dk = dk_e.reshape(Hkv, G, n, hd).sum(axis=1)                              # repeat_kv_bwd :973-992
        dv = dv_e.reshape(Hkv, G, n, hd).sum(axis=1)
        cos, sin = rope_angles(n, hd, layer_theta(c, L), t)
        dq = rms_norm_backward(sv["q_pre"], rope(dq, cos, sin, inverse=True), W["q_norm"], eps)
        dk = rms_norm_backward(sv["k_pre"], rope(dk, cos, sin, inverse=True), W["k_norm"], eps)
        dq, dk, dv = heads_rev(dq), heads_rev(dk), heads_rev(dv)
        if sgd is not None:
            # q, k, v step first; the gradient then goes on through the stepped matrices (:922-945)
            sgd.take(lw, "q", dq, sv["ln1"], L)
            sgd.take(lw, "k", dk, sv["ln1"], L)
            sgd.take(lw, "v", dv, sv["ln1"], L)
            W = {k: v.astype(t) for k, v in lw.items()}
        if lora is None:
            dln = dq @ W["q"] + dk @ W["k"]
            dln = dln + dv @ W["v"]
        else:
            lp = {k: v.astype(t) for k, v in lora.p[L].items()}
            # LoRA Q (:946-952), base (:955-958), LoRA V (:961-966), base V (:968-970)
            g = {}
            g["B_q"] = (dq.T @ sv["q_mid"]) * sc
            tmp = (dq @ lp["B_q"]) * sc
            g["A_q"] = tmp.T @ sv["ln1"]
            dln = dq @ W["q"] + tmp @ lp["A_q"] + dk @ W["k"]
            g["B_v"] = (dv.T @ sv["v_mid"]) * sc
            tmp = (dv @ lp["B_v"]) * sc
            g["A_v"] = tmp.T @ sv["ln1"]
            dln = dln + dv @ W["v"] + tmp @ lp["A_v"]
            grads[L] = g
        dx = dx + rms_norm_backward(sv["x_in"], dln, W["input_norm"], eps)        # :974-976
        dx = np.clip(dx, t(-1e6), t(1e6))                                         # :979
    return grads


def full_train_step(w, inputs, targets, lr, accum=None, dtype=np.float32):
    """sft_train_step on a full-parameter state (fast_sft.c:1113-1140): forward, loss, and the backward pass that
    steps (or, with accumulators, accumulates into) every matrix. Returns (mean loss, per-position losses)."""
    logits, saved = forward(w, None, inputs, dtype)
    losses, d = softmax_ce(logits, np.asarray(targets, dtype=np.int64))
    n = len(inputs)
    d = d * dtype(np.float32(1.0) / np.float32(n))
    backward(w, None, saved, d, SGD(lr, accum))
    return float(losses.sum() / dtype(n)), losses


def loss_and_grads(w, lora, inputs, targets, dtype=np.float32):
    """Mean over the S sequences of the reference's per-sequence loss and 1/N-scaled gradients."""
    inputs, targets = np.atleast_2d(inputs), np.atleast_2d(targets)
    S, n = inputs.shape
    total, acc, logits0 = 0.0, None, None
    for s in range(S):
        logits, saved = forward(w, lora, inputs[s], dtype)
        losses, d = softmax_ce(logits, np.asarray(targets[s], dtype=np.int64))
        d = d * dtype(np.float32(1.0) / np.float32(n))                            # :759
        g = backward(w, lora, saved, d)
        total += float(losses.sum() / dtype(n))                                       # :1142-1144
        acc = g if acc is None else [{k: a[k] + b[k] for k in KEYS} for a, b in zip(acc, g)]
        if s == 0:
            logits0 = logits
    grads = [{k: (a[k] / dtype(S)) for k in KEYS} for a in acc]
    return total / S, grads, logits0


def clip_grad_norm(grads, max_norm=1.0):
    """clip_grad_norm (fast_sft.c:1060-1088): norm accumulated in double, no epsilon."""
    total = 0.0
    for g in grads:
        for k in ("A_q", "B_q", "A_v", "B_v"):                                    # buffer order dA_q dB_q dA_v dB_v
            total += float((g[k].astype(np.float64) ** 2).sum())
    norm = np.float32(np.sqrt(total))
    if norm > np.float32(max_norm):
        s = np.float32(max_norm) / norm
        grads = [{k: (g[k] * s).astype(np.float32) for k in KEYS} for g in grads]
    return grads, float(norm)


def adamw(lora, grads, lr, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.01):
    """adamw_update (fast_sft.c:1045-1058), fp32 throughout, bias correction with powf."""
    f = np.float32
    step = lora.step_count
    bc1 = f(1) - f(np.power(f(beta1), f(step), dtype=np.float32))
    bc2 = f(1) - f(np.power(f(beta2), f(step), dtype=np.float32))
    b1, b2, e, w_, lr = f(beta1), f(beta2), f(eps), f(wd), f(lr)
    for L, g in enumerate(grads):
        for k in KEYS:
            gr = g[k].astype(np.float32)
            m = b1 * lora.m[L][k] + (f(1) - b1) * gr
            v = b2 * lora.v[L][k] + (f(1) - b2) * gr * gr
            lora.m[L][k], lora.v[L][k] = m, v
            p = lora.p[L][k]
            lora.p[L][k] = (p - lr * ((m / bc1) / (np.sqrt(v / bc2) + e) + w_ * p)).astype(np.float32)


def train_step(w, lora, inputs, targets, lr, dtype=np.float32):
    """sft_train_step (fast_sft.c:1113-1157): loss, then step_count++, clip at 1.0, AdamW."""
    loss, grads, _ = loss_and_grads(w, lora, inputs, targets, dtype)
    grads = [{k: g[k].astype(np.float32) for k in KEYS} for g in grads]
    lora.step_count += 1
    clipped, norm = clip_grad_norm(grads, 1.0)
    adamw(lora, clipped, lr)
    return loss, grads, norm


def save_lora_bytes(lora):
    """sft_save_lora (fast_sft.c:1255-1285): u32 0x4C4F5241, i32 n_layers, i32 rank, then per layer
    A_q, B_q, A_v, B_v as fp32."""
    out = [struct.pack("<Iii", 0x4C4F5241, len(lora.p), lora.rank)]
    for l in lora.p:
        for k in KEYS:
            out.append(np.ascontiguousarray(l[k], dtype="<f4").tobytes())
    return b"".join(out)
