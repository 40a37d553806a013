"""Batched F16 decode (qwen3_generate_fast_batch and the layer-by-layer batch state): every sequence
must produce what the single-sequence CPU restatement of the reference produces for its prompt. The
projections round the activation rows to binary16 (tensor-core operands), so a token may differ from
the restatement only where its two best logits are a near-tie; logits agree to the stated 1e-2."""
import ctypes as C

import numpy as np
import pytest

import _oracle

pytestmark = pytest.mark.gpu


def oracle_tokens(pkg, synth, sp, model, prompt, n):
    m = _oracle.model_qwen3(model, 1, 64, vocab=sp.vocab_size)
    return _oracle.generate(m, prompt, n, want_logits=True)


def check_against_oracle(oracle_fn, prompt, got):
    """Every generated token must be the restatement's choice given the tokens before it, or its runner-up where
    the two best logits are a near-tie. After such a flip the restatement is run again on the engine's own prefix,
    so the whole continuation is checked, not only the part before the first flip. Returns the number of flips."""
    done, flips = 0, 0
    while done < len(got):
        ref_tokens, ref_logits = oracle_fn(np.concatenate([prompt, got[:done]]).astype(np.uint32), len(got) - done)
        for i in range(len(got) - done):
            t = int(got[done + i])
            if t == int(ref_tokens[i]):
                continue
            order = np.argsort(ref_logits[i])
            top = ref_logits[i][order[-2:]]
            assert (top[1] - top[0]) < 2e-3 * np.abs(ref_logits[i]).max(), (done + i, t, int(ref_tokens[i]))
            assert t == int(order[-2]), (done + i, t, int(order[-2]))         # the runner-up, nothing else
            flips += 1
            done += i + 1
            break
        else:
            return flips
    return flips


def test_same_prompt_batch_matches_the_single_sequence_oracle(pkg, lib, synth):
    sp = pkg.spec("tiny-qwen3", gamma_jitter=0.1)
    model = synth.llmb200_synth_qwen3(C.byref(sp), 4)
    try:
        P, G, B = 16, 24, 5
        prompt = np.zeros(P, dtype=np.uint32)
        synth.llmb200_synth_tokens(prompt.ctypes.data, P, 4321, sp.vocab_size)
        out = np.zeros((B, G), dtype=np.uint32)
        n = lib.qwen3_generate_fast_batch(model, prompt.ctypes.data_as(pkg.c_u32_p), P, out.ctypes.data_as(pkg.c_u32_p), G, 64, B)
        assert n == G
        for b in range(1, B):
            assert np.array_equal(out[b], out[0])             # same prompt, greedy: identical sequences
        flips = check_against_oracle(lambda pr, n: oracle_tokens(pkg, synth, sp, model, pr, n), prompt, out[0])
        assert flips <= 2, flips
    finally:
        synth.llmb200_synth_free_qwen3(model)


def test_different_prompts_and_logits(pkg, lib, synth):
    sp = pkg.spec("tiny-qwen3", gamma_jitter=0.1, n_layers=2)
    model = synth.llmb200_synth_qwen3(C.byref(sp), 4)
    import _sft_common as sc
    try:
        P, G, B = 8, 6, 3
        cfg = pkg.config_of(sp, pkg.MODEL_QWEN3, 32, 1)
        st = lib.llmb200_batch_begin(C.byref(cfg), B, G)
        assert st
        # the same seeded tensors the synthetic model holds, handed over layer by layer
        w = sc.make_weights(pkg, dict(sc.TINY, n_layers=2), seed=sp.seed, gamma_jitter=0.1)
        keep = []
        D, Hq, Hkv, hd, IS = sp.d_model, sp.n_q_heads, sp.n_kv_heads, sp.head_dim, sp.intermediate_size
        for i, l in enumerate(w["layers"]):
            r = pkg.LayerWeightRef()
            for name, rows, cols in (("q", Hq * hd, D), ("k", Hkv * hd, D), ("v", Hkv * hd, D), ("o", D, Hq * hd),
                                     ("gate", IS, D), ("up", IS, D), ("down", D, IS)):
                a = np.ascontiguousarray(l[name], dtype=np.float32)
                keep.append(a)
                setattr(r, name + "_proj", pkg.WeightRef(sc.fptr(a), rows, cols))
            for name, field in (("input_norm", "input_norm_g"), ("post_attn_norm", "post_attn_norm_g"),
                                ("q_norm", "q_norm_g"), ("k_norm", "k_norm_g")):
                a = np.ascontiguousarray(l[name], dtype=np.float32)
                keep.append(a)
                setattr(r, field, sc.fptr(a))
            r.d_model, r.head_dim = D, hd
            assert lib.llmb200_batch_load_layer(st, i, C.byref(r), C.c_float(sp.rope_theta)) == 0
            lib.metal_flush()
        lm, fn, emb = (np.ascontiguousarray(w[k], dtype=np.float32) for k in ("lm_head", "final_norm", "emb"))
        assert lib.llmb200_batch_finish(st, sc.fptr(lm), sc.fptr(fn), sc.fptr(emb)) == 0
        lib.llmb200_batch_set_eos(st, None, 0)
        prompts = np.zeros((B, P), dtype=np.uint32)
        synth.llmb200_synth_tokens(prompts.ctypes.data, B * P, 99, sp.vocab_size)
        out = np.zeros((B, G), dtype=np.uint32)
        n = lib.llmb200_batch_generate(st, prompts.ctypes.data_as(pkg.c_u32_p), P, out.ctypes.data_as(pkg.c_u32_p), G)
        assert n == G
        # the restatement of the SFT forward (same network, fp32 activations) gives the logits to compare with:
        # feed it each sequence's prompt + generated tokens and look at the position that produced each token
        o = sc.sft_oracle
        ow = sc.oracle_model(dict(sc.TINY, n_layers=2), w)
        zero = o.LoRA(sc.make_lora(pkg, dict(sc.TINY, n_layers=2), 4), 4, 8.0)
        last = np.zeros((B, sp.vocab_size), dtype=np.float32)
        for b in range(B):
            seq = np.concatenate([prompts[b], out[b]])
            lg, _ = o.forward(ow, zero, seq[:-1])
            for g in range(G):
                row = lg[P - 1 + g]
                if int(np.argmax(row)) != int(out[b, g]):
                    top = np.sort(row)[-2:]
                    assert (top[1] - top[0]) < 2e-3 * np.abs(row).max(), (b, g)
            last[b] = lg[-1]
        got = np.zeros((B, sp.vocab_size), dtype=np.float32)
        assert lib.llmb200_batch_logits(st, got.ctypes.data_as(pkg.c_float_p), got.size)
        assert np.abs(got - last).max() < 1e-2 * np.abs(last).max()
        lib.llmb200_batch_free(st)
    finally:
        synth.llmb200_synth_free_qwen3(model)
