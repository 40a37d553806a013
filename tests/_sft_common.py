"""Shared helpers of the LoRA-SFT tests: seeded weights as numpy arrays, the oracle model built from
them, an independent float64 torch-autograd model of the same network, and the engine driver."""
import ctypes as C
import importlib.util
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _load(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def package():
    """The package directory name contains a dot, so it is imported by path."""
    if "llm_metal_b200" in sys.modules:
        return sys.modules["llm_metal_b200"]
    import __graft_entry__ as ge
    return ge.load_package()


sft_oracle = _load("sft_oracle", os.path.join(ROOT, "oracle", "sft_oracle.py"))

T_Q, T_K, T_V, T_O, T_GATE, T_UP, T_DOWN, T_QNORM, T_KNORM, T_INPUT_NORM, T_POST_ATTN_NORM = range(11)
T_EMB, T_LM_HEAD, T_FINAL_NORM = 100, 101, 102
T_LORA = 50          # + sub (0..3): test-only tensor ids for the LoRA matrices

# llmb200_sft_export selectors (include/llmb200_sft.h)
X_IN, LN1, QKV, Q_FINAL, K_FINAL, PROBS, X_MID, LN2, GATE_UP, MID_Q, MID_V = range(11)
LOGITS, DLOGITS, LOSSES, X_FINAL = 100, 101, 102, 103
LORA_GRADS, LORA_PARAMS = 200, 201

SMALL = dict(n_layers=2, d_model=128, n_q_heads=4, n_kv_heads=2, head_dim=64, intermediate_size=256, vocab_size=512,
             rope_theta=1e6)
TINY = dict(n_layers=4, d_model=512, n_q_heads=8, n_kv_heads=2, head_dim=64, intermediate_size=1536, vocab_size=4096,
            rope_theta=1e6)


def normal(pkg, shape, seed, layer, which, mean=0.0, std=0.02):
    S = pkg.synth()
    out = np.empty(int(np.prod(shape)), dtype=np.float32)
    S.llmb200_synth_normal(out.ctypes.data, out.size, seed, S.llmb200_synth_tensor_id(layer, which), mean, std, 4)
    return out.reshape(shape)


def tokens(pkg, n, seed, vocab):
    out = np.empty(n, dtype=np.uint32)
    pkg.synth().llmb200_synth_tokens(out.ctypes.data, n, seed, vocab)
    return out


def make_weights(pkg, cfg, seed=1234, gamma_jitter=0.1):
    """fp32 (unrounded) matrices as a loader would hand them over, as numpy arrays."""
    D, Hq, Hkv, hd, IS, V = (cfg[k] for k in ("d_model", "n_q_heads", "n_kv_heads", "head_dim", "intermediate_size",
                                               "vocab_size"))
    layers = []
    for L in range(cfg["n_layers"]):
        g = lambda which, n: normal(pkg, (n,), seed, L, which, 1.0, gamma_jitter) if gamma_jitter else np.ones(n, np.float32)
        layers.append(dict(
            q=normal(pkg, (Hq * hd, D), seed, L, T_Q), k=normal(pkg, (Hkv * hd, D), seed, L, T_K),
            v=normal(pkg, (Hkv * hd, D), seed, L, T_V), o=normal(pkg, (D, Hq * hd), seed, L, T_O),
            gate=normal(pkg, (IS, D), seed, L, T_GATE), up=normal(pkg, (IS, D), seed, L, T_UP),
            down=normal(pkg, (D, IS), seed, L, T_DOWN),
            input_norm=g(T_INPUT_NORM, D), post_attn_norm=g(T_POST_ATTN_NORM, D), q_norm=g(T_QNORM, hd),
            k_norm=g(T_KNORM, hd)))
    return dict(layers=layers, lm_head=normal(pkg, (V, D), seed, 0, T_LM_HEAD), emb=normal(pkg, (V, D), seed, 0, T_EMB),
                final_norm=(normal(pkg, (D,), seed, 0, T_FINAL_NORM, 1.0, gamma_jitter) if gamma_jitter
                            else np.ones(D, np.float32)))


T_PRE_FF_NORM, T_POST_FF_NORM = 11, 12


def gemma_cfg(sp):
    """Configuration dict of a Gemma3 SynthSpec as the SFT restatement takes it: the RoPE base per layer by
    position in the stack (src/nn/fast_sft.c:310-313), tied and scaled embeddings."""
    c = dict(n_layers=sp.n_layers, d_model=sp.d_model, n_q_heads=sp.n_q_heads, n_kv_heads=sp.n_kv_heads,
             head_dim=sp.head_dim, intermediate_size=sp.intermediate_size, vocab_size=sp.vocab_size, gemma=True)
    c["rope_thetas"] = [float(sp.local_rope_theta) if (i % 6) != 0 else float(sp.rope_theta) for i in range(sp.n_layers)]
    c["rope_theta"] = float(sp.rope_theta)
    return c


def make_weights_gemma(pkg, cfg, seed=1234, gamma_jitter=0.1):
    """The seeded tensors of a synthetic Gemma3 model (llmb200_synth_gemma3) as numpy arrays: the Qwen3 set plus the
    two feed-forward norms; the LM head is the embedding table."""
    w = make_weights(pkg, cfg, seed, gamma_jitter)
    D = cfg["d_model"]
    for L, l in enumerate(w["layers"]):
        g = lambda which: normal(pkg, (D,), seed, L, which, 1.0, gamma_jitter) if gamma_jitter else np.ones(D, np.float32)
        l["pre_ff_norm"], l["post_ff_norm"] = g(T_PRE_FF_NORM), g(T_POST_FF_NORM)
    w["lm_head"] = w["emb"]
    return w


def make_lora(pkg, cfg, rank, seed=77, b_std=0.0):
    """A ~ N(0, 0.01); B = 0 (the configured start) or N(0, b_std) so that every gradient is non-zero."""
    D, Hq, Hkv, hd = cfg["d_model"], cfg["n_q_heads"], cfg["n_kv_heads"], cfg["head_dim"]
    out = []
    for L in range(cfg["n_layers"]):
        l = dict(A_q=normal(pkg, (rank, D), seed, L, T_LORA + 0, 0.0, 0.01),
                 A_v=normal(pkg, (rank, D), seed, L, T_LORA + 2, 0.0, 0.01))
        if b_std:
            l["B_q"] = normal(pkg, (Hq * hd, rank), seed, L, T_LORA + 1, 0.0, b_std)
            l["B_v"] = normal(pkg, (Hkv * hd, rank), seed, L, T_LORA + 3, 0.0, b_std)
        else:
            l["B_q"] = np.zeros((Hq * hd, rank), np.float32)
            l["B_v"] = np.zeros((Hkv * hd, rank), np.float32)
        out.append(l)
    return out


def oracle_model(cfg, w):
    o = sft_oracle
    layers = []
    for l in w["layers"]:
        d = {k: o.f16_round(l[k]) for k in ("q", "k", "v", "o", "gate", "up", "down")}
        d.update({k: l[k] for k in ("input_norm", "post_attn_norm", "q_norm", "k_norm", "pre_ff_norm", "post_ff_norm") if k in l})
        layers.append(d)
    c = dict(cfg)
    c["eps"] = 1e-6
    return o.Weights(c, layers, o.f16_round(w["lm_head"]), w["final_norm"], w["emb"])


# ---- independent float64 model (torch autograd) ------------------------------------------------------

def torch_loss_and_grads(cfg, ow, lora_layers, scaling, inputs, targets):
    """Mean over sequences of the mean next-token cross-entropy; gradients of the LoRA matrices by
    autograd. Written against the architecture, not against the oracle's code."""
    import torch
    import torch.nn.functional as F
    f64 = torch.float64
    Hq, Hkv, hd = cfg["n_q_heads"], cfg["n_kv_heads"], cfg["head_dim"]
    eps = 1e-6

    def t(a):
        return torch.tensor(np.asarray(a, dtype=np.float64), dtype=f64)

    def rms(x, g):
        return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * g

    def rot(x, cos, sin):
        h = x.shape[-1] // 2
        return torch.cat([x[..., :h] * cos - x[..., h:] * sin, x[..., :h] * sin + x[..., h:] * cos], -1)

    params = [{k: t(v).requires_grad_(True) for k, v in l.items()} for l in lora_layers]
    inputs, targets = np.atleast_2d(inputs), np.atleast_2d(targets)
    S, n = inputs.shape
    d = np.arange(hd // 2, dtype=np.float32)
    freq = (np.float32(1.0) / np.power(np.float32(cfg["rope_theta"]), (2 * d) / np.float32(hd), dtype=np.float32))
    ang = (np.arange(n, dtype=np.float32)[:, None] * freq[None, :]).astype(np.float32).astype(np.float64)
    cos, sin = torch.tensor(np.cos(ang)), torch.tensor(np.sin(ang))
    mask = torch.tril(torch.ones(n, n, dtype=torch.bool))
    total = 0.0
    for s in range(S):
        x = t(ow.token_emb[inputs[s].astype(np.int64)])
        for L, lw in enumerate(ow.layers):
            p = params[L]
            h = rms(x, t(lw["input_norm"]))
            q = h @ t(lw["q"]).T + scaling * (h @ p["A_q"].T) @ p["B_q"].T
            k = h @ t(lw["k"]).T
            v = h @ t(lw["v"]).T + scaling * (h @ p["A_v"].T) @ p["B_v"].T
            q = rot(rms(q.view(n, Hq, hd), t(lw["q_norm"])).transpose(0, 1), cos, sin)
            k = rot(rms(k.view(n, Hkv, hd), t(lw["k_norm"])).transpose(0, 1), cos, sin)
            v = v.view(n, Hkv, hd).transpose(0, 1)
            k = k.repeat_interleave(Hq // Hkv, 0)
            v = v.repeat_interleave(Hq // Hkv, 0)
            att = (q @ k.transpose(1, 2)) / np.sqrt(np.float32(hd)).astype(np.float64)
            att = F.softmax(att.masked_fill(~mask, float("-inf")), -1) @ v
            x = x + att.transpose(0, 1).reshape(n, Hq * hd) @ t(lw["o"]).T
            h = rms(x, t(lw["post_attn_norm"]))
            x = x + (F.silu(h @ t(lw["gate"]).T) * (h @ t(lw["up"]).T)) @ t(lw["down"]).T
        logits = rms(x, t(ow.final_norm)) @ t(ow.lm_head).T
        total = total + F.cross_entropy(logits, torch.tensor(targets[s].astype(np.int64)))
    loss = total / S
    loss.backward()
    return float(loss.detach()), [{k: v.grad.numpy() for k, v in p.items()} for p in params]


# ---- the engine ------------------------------------------------------------------------------------------

def fptr(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


class Engine:
    """An SFTState built layer by layer from numpy weights."""

    def __init__(self, pkg, cfg, w, lora_layers, seq_len, n_seq, rank, alpha, tensor_cores=None):
        self.pkg, self.L, self.cfg = pkg, pkg.lib(), cfg
        self.keep = []
        gemma = bool(cfg.get("gemma"))
        c = pkg.Config(pkg.MODEL_GEMMA3 if gemma else pkg.MODEL_QWEN3, cfg["d_model"], cfg["n_q_heads"], cfg["n_kv_heads"],
                       cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"], cfg["n_layers"], seq_len, 1)
        if tensor_cores is not None:
            os.environ["LLMB200_SFT_TC"] = "1" if tensor_cores else "0"
        try:
            self.h = self.L.llmb200_sft_begin(C.byref(c), seq_len, n_seq, rank, alpha)
        finally:
            os.environ.pop("LLMB200_SFT_TC", None)
        assert self.h, "llmb200_sft_begin failed"
        D, Hq, Hkv, hd, IS = (cfg[k] for k in ("d_model", "n_q_heads", "n_kv_heads", "head_dim", "intermediate_size"))
        for i, l in enumerate(w["layers"]):
            r = pkg.LayerWeightRef()
            for name, rows, cols in (("q", Hq * hd, D), ("k", Hkv * hd, D), ("v", Hkv * hd, D), ("o", D, Hq * hd),
                                     ("gate", IS, D), ("up", IS, D), ("down", D, IS)):
                a = np.ascontiguousarray(l[name], dtype=np.float32)
                self.keep.append(a)
                setattr(r, name + "_proj", pkg.WeightRef(fptr(a), rows, cols))
            norms = [("input_norm", "input_norm_g"), ("post_attn_norm", "post_attn_norm_g"), ("q_norm", "q_norm_g"),
                     ("k_norm", "k_norm_g")]
            if gemma:
                norms += [("pre_ff_norm", "pre_ff_norm_g"), ("post_ff_norm", "post_ff_norm_g")]
            for name, field in norms:
                a = np.ascontiguousarray(l[name], dtype=np.float32)
                self.keep.append(a)
                setattr(r, field, fptr(a))
            r.d_model, r.head_dim = D, hd
            arr = (C.POINTER(C.c_float) * 4)()
            if lora_layers is not None:
                for j, k in enumerate(("A_q", "B_q", "A_v", "B_v")):
                    a = np.ascontiguousarray(lora_layers[i][k], dtype=np.float32)
                    self.keep.append(a)
                    arr[j] = fptr(a)
            rc = self.L.llmb200_sft_load_layer(self.h, i, C.byref(r), cfg["rope_thetas"][i] if "rope_thetas" in cfg else cfg["rope_theta"],
                                               C.byref(arr) if lora_layers is not None else None)
            assert rc == 0, rc
        lm, fn, emb = (np.ascontiguousarray(w[k], dtype=np.float32) for k in ("lm_head", "final_norm", "emb"))
        assert self.L.llmb200_sft_finish(self.h, fptr(lm), fptr(fn), fptr(emb), 0) == 0
        self.M = seq_len * n_seq
        self.n_seq, self.seq_len, self.rank = n_seq, seq_len, rank

    def close(self):
        if self.h:
            self.L.sft_state_free(self.h)
            self.h = None

    def __del__(self):
        self.close()

    def _tok(self, a):
        a = np.ascontiguousarray(np.asarray(a).reshape(-1), dtype=np.uint32)
        assert a.size == self.M
        return a, a.ctypes.data_as(C.POINTER(C.c_uint32))

    def forward_backward(self, inputs, targets):
        a, pa = self._tok(inputs)
        b, pb = self._tok(targets)
        loss = self.L.llmb200_sft_forward_backward(self.h, pa, pb)
        assert self.L.llmb200_sft_error(self.h) == 0
        return loss

    def train(self, inputs, targets, lr):
        a, pa = self._tok(inputs)
        b, pb = self._tok(targets)
        loss = self.L.llmb200_sft_train_batch(self.h, pa, pb, lr)
        assert self.L.llmb200_sft_error(self.h) == 0
        return loss

    def _vector(self, what):
        p = C.c_void_p()
        n = self.L.llmb200_sft_grad_vector(self.h, C.byref(p))
        return self.export(what, 0, n)

    def grads(self):
        return self._split(self._vector(LORA_GRADS))

    def params(self):
        return self._split(self._vector(LORA_PARAMS))

    def _split(self, flat):
        cfg, R = self.cfg, self.rank
        D, Hq, Hkv, hd = cfg["d_model"], cfg["n_q_heads"], cfg["n_kv_heads"], cfg["head_dim"]
        shapes = (("A_q", (R, D)), ("B_q", (Hq * hd, R)), ("A_v", (R, D)), ("B_v", (Hkv * hd, R)))
        out, o = [], 0
        for _ in range(cfg["n_layers"]):
            l = {}
            for k, sh in shapes:
                n = sh[0] * sh[1]
                l[k] = flat[o:o + n].reshape(sh).copy()
                o += n
            out.append(l)
        assert o == flat.size
        return out

    def export(self, what, layer, n):
        out = np.empty(n, dtype=np.float32)
        got = self.L.llmb200_sft_export(self.h, what, layer, out.ctypes.data, n)
        assert got == n, (got, n)
        return out


def rel_err(a, b):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))
