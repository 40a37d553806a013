#!/usr/bin/env python
"""Headline benchmark: Qwen3-4B-shaped Q8_0 batch-1 greedy decode, tokens per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One step = one generate request of the workload (prompt 512, generate 512): a
token-by-token prefill (untimed, as in the reference's own metric) followed by
511 decode forwards (timed). Weights are seeded random N(0, 0.02) of the named
architecture, quantised to Q8_0 on the GPU; token ids are uniform random.

  value      decode tokens / second with every input resident in HBM: the
             per-token CUDA graph replayed 511 times per step, timed with CUDA
             events on the launching stream, max over ranks.
  e2e        the same metric through the reference-facing call
             inference_generate() with host buffers: prompt ids copied in,
             every generated id copied back inside the timed region.
  roofline   the dominant kernel. With the whole-token kernel (the default) that
             is the one kernel of a token: algorithmic bytes per launch (weights
             + norm weights + F16 K/V rows + embedding row) / CUDA-event time per
             launch, against the measured HBM copy bandwidth.
  secondary  (N = 1, default workload) the other configurations of the
             benchmark set, measured in child processes after the headline run:
             the standalone Q8_0 matvec sweep, Gemma3-1B F16 decode, the LoRA SFT
             step.
  parity     tokens of a two-layer full-width cut of the architecture against
             vectors the reference's own C code produced (tests/golden), checked
             on the GPU(s) of this run before anything is timed.
  cpu_baseline  the reference's own C code path (oracle/_ref) on one host
             thread, on a bounded sample of the same workload.

N > 1 runs the same model tensor-parallel over N GPUs (strong scaling).
"""
import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

WORKLOADS = {
    # name: (architecture, use_fp16, prompt, generate, max_seq)
    "qwen3-4b-q8": ("qwen3-4b", 0, 512, 512, 4096),
    "tiny-qwen3-q8": ("tiny-qwen3", 0, 16, 32, 64),
    # Gemma3-1B, binary16 weights (src/nn/gemma3.c:11-25): 4-norm blocks, GeGLU, per-layer rope base, tied LM head
    "gemma3-1b-f16": ("gemma3-1b", 1, 128, 256, 512),
    "tiny-gemma3-f16": ("tiny-gemma3", 1, 16, 32, 96),
}
# Standalone Q8_0 matvec, batch 1, the six shapes of Qwen3-4B (rows x cols), fp32 activations N(0,1)
SWEEP_SHAPES = [(4096, 2560), (1024, 2560), (2560, 4096), (9728, 2560), (2560, 9728), (151936, 2560)]
HBM_FALLBACK_GBS = 6650.0

# Libraries (NCCL's version banner, the engine's progress lines) write to file descriptor 1 too; the
# contract is ONE JSON line on stdout, so everything else is sent to stderr and the line goes to the
# original descriptor.
_JSON_FD = os.dup(1)
os.dup2(2, 1)


def emit(text):
    os.write(_JSON_FD, (text + "\n").encode())

GATEUP_TRAFFIC_BYTES = 53_014_700
# dram__bytes_read.sum + dram__bytes_write.sum of one decode_token_kernel launch, from the ncu capture of a
# 4-layer and an 8-layer cut at position ~515 (profiles/decode_token_kernel_qwen3-4b_4and8layer_cuts_full.md):
# per layer (difference of the two captures / 4) and for the rest (LM head, embedding row, logits). Traffic
# grows in proportion to the layers.
TOKEN_TRAFFIC = {"qwen3-4b": {"per_layer": 110.03e6, "rest": 420.6e6}}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return HBM_FALLBACK_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except Exception:
                continue
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            for name, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def gen_f32(S, n, seed, tid, std, threads, mean=0.0):
    a = np.empty(n, dtype=np.float32)
    S.llmb200_synth_normal(a.ctypes.data, n, seed, tid, mean, std, threads)
    return a


def build_state_streaming(pkg, L, S, sp, max_seq, use_fp16, threads):
    """Layer-by-layer construction: at most one layer (plus the LM head) of fp32 weights is held on the host."""
    cfg = pkg.config_of(sp, pkg.MODEL_QWEN3, max_seq, use_fp16)
    st = L.llmb200_state_begin(C.byref(cfg))
    if not st:
        raise RuntimeError("llmb200_state_begin failed")
    D, hd, IS, V = sp.d_model, sp.head_dim, sp.intermediate_size, sp.vocab_size
    shapes = [(sp.n_q_heads * hd, D), (sp.n_kv_heads * hd, D), (sp.n_kv_heads * hd, D), (D, sp.n_q_heads * hd),
              (IS, D), (IS, D), (D, IS)]
    ones_d, ones_h = np.ones(D, dtype=np.float32), np.ones(hd, dtype=np.float32)
    fp = pkg.c_float_p
    for layer in range(sp.n_layers):
        mats = [gen_f32(S, r * c, sp.seed, S.llmb200_synth_tensor_id(layer, w), sp.weight_std, threads)
                for w, (r, c) in enumerate(shapes)]
        ref = pkg.LayerWeightRef()
        for name, m, (r, c) in zip(["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"], mats, shapes):
            setattr(ref, name, pkg.WeightRef(m.ctypes.data_as(fp), r, c))
        ref.input_norm_g = ones_d.ctypes.data_as(fp)
        ref.post_attn_norm_g = ones_d.ctypes.data_as(fp)
        ref.q_norm_g = ones_h.ctypes.data_as(fp)
        ref.k_norm_g = ones_h.ctypes.data_as(fp)
        ref.d_model, ref.head_dim = D, hd
        if L.llmb200_state_load_layer(st, layer, C.byref(ref), C.c_float(sp.rope_theta)) != 0:
            raise RuntimeError(f"loading layer {layer} failed")
        L.metal_flush()                      # the staging copies read `mats`; keep them alive until done
    lm = gen_f32(S, V * D, sp.seed, S.llmb200_synth_tensor_id(0, 101), sp.weight_std, threads)
    emb = gen_f32(S, V * D, sp.seed, S.llmb200_synth_tensor_id(0, 100), sp.weight_std, threads)
    if L.llmb200_state_finish(st, lm.ctypes.data_as(fp), ones_d.ctypes.data_as(fp), emb.ctypes.data_as(fp)) != 0:
        raise RuntimeError("llmb200_state_finish failed")
    return st


def algorithmic_bytes_per_token(sp, n_attend, world=1, use_fp16=0, gemma=False):
    """Bytes one decode token has to move per GPU: weights (Q8_0 34 bytes per 32, or binary16) + gammas +
    F16 K/V rows + one embedding row."""
    D, hd, IS, V, Lr = sp.d_model, sp.head_dim, sp.intermediate_size, sp.vocab_size, sp.n_layers
    num, den = (2, 1) if use_fp16 else (34, 32)
    per_layer = ((sp.n_q_heads + 2 * sp.n_kv_heads) * hd * D + D * sp.n_q_heads * hd + 3 * IS * D) * num // den
    weights = (Lr * per_layer + V * D * num // den) // world
    gammas = (Lr * ((4 if gemma else 2) * D + 2 * hd) + D) * 4
    kv = Lr * 2 * (sp.n_kv_heads // world) * hd * 2 * n_attend
    return weights + gammas + kv + D * 4


def cpu_reference_sample(pkg, S, sp, threads):
    """Times the reference's C path (oracle/_ref; else the oracle port) on a bounded sample.

    Sample: models with 1 and with 3 of the architecture's layers plus the full LM head, 2 prompt + 2
    generated tokens each; the per-layer and head times are separated by differencing and the full-depth
    time per token is their linear combination.
    """
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import _oracle as O
    use_ref = O.have_ref()
    prompt = np.zeros(2, dtype=np.uint32)
    S.llmb200_synth_tokens(prompt.ctypes.data, 2, 4321, sp.vocab_size)
    per_tok = {}
    for nl in (1, 3):
        sub = pkg.SynthSpec.from_buffer_copy(sp)
        sub.n_layers = nl
        model = S.llmb200_synth_qwen3(C.byref(sub), threads)
        out = np.zeros(2, dtype=np.uint32)
        secs = np.zeros(2, dtype=np.float64)
        if use_ref:
            O.ref().ref_requant_qwen3(model, 0)
            n = O.ref().ref_qwen3_generate(model, prompt.ctypes.data, 2, out.ctypes.data, 2, 8, None, 0, None, secs.ctypes.data)
            tokens = 2 + (n - 1)
            per_tok[nl] = float(secs[0] + secs[1]) / tokens
        else:
            om = O.model_qwen3(model, 0, 8, vocab=sp.vocab_size)
            toks, _ = O.generate(om, prompt, 2)
            per_tok[nl] = sum(O.generate.last_seconds) / (2 + len(toks) - 1)
            del om
        S.llmb200_synth_free_qwen3(model)
    t_layer = max((per_tok[3] - per_tok[1]) / 2.0, 1e-9)
    t_head = max(per_tok[1] - t_layer, 0.0)
    t_full = sp.n_layers * t_layer + t_head
    return {"value": 1.0 / t_full, "unit": "tok/s", "cores": 1, "kind": "reference" if use_ref else "port",
            "sample": f"1- and 3-layer models of the architecture + full LM head, 4 forwards each (positions 0-3); "
                      f"{t_layer * 1e3:.0f} ms/layer, {t_head * 1e3:.0f} ms head, extrapolated to {sp.n_layers} layers"}


SFT_WORKLOADS = {
    # name: (architecture, seq_len, sequences per GPU, LoRA rank, alpha)
    "qwen3-4b-sft-lora": ("qwen3-4b", 64, 8, 16, 32.0),
    "tiny-qwen3-sft-lora": ("tiny-qwen3", 64, 8, 16, 32.0),
}
T_LORA = 50          # tensor ids of the seeded LoRA A matrices (+0: A_q, +2: A_v)


class _DeviceVector:
    """A flat fp32 device vector owned by the library, exposed to torch through __cuda_array_interface__."""

    def __init__(self, ptr, n):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (ptr, False), "version": 2}


def build_sft_streaming(pkg, L, S, sp, seq, n_seq, rank, alpha, threads):
    cfg = pkg.config_of(sp, pkg.MODEL_QWEN3, seq, 1)
    st = L.llmb200_sft_begin(C.byref(cfg), seq, n_seq, rank, alpha)
    if not st:
        raise RuntimeError("llmb200_sft_begin failed")
    D, hd, IS, V = sp.d_model, sp.head_dim, sp.intermediate_size, sp.vocab_size
    shapes = [(sp.n_q_heads * hd, D), (sp.n_kv_heads * hd, D), (sp.n_kv_heads * hd, D), (D, sp.n_q_heads * hd),
              (IS, D), (IS, D), (D, IS)]
    ones_d, ones_h = np.ones(D, dtype=np.float32), np.ones(hd, dtype=np.float32)
    zb_q = np.zeros(sp.n_q_heads * hd * rank, dtype=np.float32)
    zb_v = np.zeros(sp.n_kv_heads * hd * rank, dtype=np.float32)
    fp = pkg.c_float_p
    for layer in range(sp.n_layers):
        mats = [gen_f32(S, r * c, sp.seed, S.llmb200_synth_tensor_id(layer, w), sp.weight_std, threads)
                for w, (r, c) in enumerate(shapes)]
        ref = pkg.LayerWeightRef()
        for name, m, (r, c) in zip(["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"], mats, shapes):
            setattr(ref, name, pkg.WeightRef(m.ctypes.data_as(fp), r, c))
        ref.input_norm_g = ones_d.ctypes.data_as(fp)
        ref.post_attn_norm_g = ones_d.ctypes.data_as(fp)
        ref.q_norm_g = ones_h.ctypes.data_as(fp)
        ref.k_norm_g = ones_h.ctypes.data_as(fp)
        ref.d_model, ref.head_dim = D, hd
        # LoRA as configured: A ~ N(0, 0.01), B = 0
        a_q = gen_f32(S, rank * D, 77, S.llmb200_synth_tensor_id(layer, T_LORA + 0), 0.01, threads)
        a_v = gen_f32(S, rank * D, 77, S.llmb200_synth_tensor_id(layer, T_LORA + 2), 0.01, threads)
        lora = (fp * 4)(a_q.ctypes.data_as(fp), zb_q.ctypes.data_as(fp), a_v.ctypes.data_as(fp), zb_v.ctypes.data_as(fp))
        if L.llmb200_sft_load_layer(st, layer, C.byref(ref), C.c_float(sp.rope_theta), C.byref(lora)) != 0:
            raise RuntimeError(f"loading layer {layer} failed")
        L.metal_flush()
    lm = gen_f32(S, V * D, sp.seed, S.llmb200_synth_tensor_id(0, 101), sp.weight_std, threads)
    emb = gen_f32(S, V * D, sp.seed, S.llmb200_synth_tensor_id(0, 100), sp.weight_std, threads)
    if L.llmb200_sft_finish(st, lm.ctypes.data_as(fp), ones_d.ctypes.data_as(fp), emb.ctypes.data_as(fp), 0) != 0:
        raise RuntimeError("llmb200_sft_finish failed")
    return st


def sft_flops_per_token(sp):
    """Forward 2P + backward through the frozen weights 2P multiply-adds per token (LoRA and attention < 1 %)."""
    D, hd, IS, V = sp.d_model, sp.head_dim, sp.intermediate_size, sp.vocab_size
    per_layer = (sp.n_q_heads + 2 * sp.n_kv_heads) * hd * D + D * sp.n_q_heads * hd + 3 * IS * D
    return 4.0 * (per_layer * sp.n_layers + V * D)


def sft_cpu_port_sample(sp, seq, rank, alpha):
    """The CPU restatement (oracle/sft_oracle.py, numpy) timed on one sequence per step, as the reference
    trains: 1- and 2-layer cuts of the architecture with the full LM head, extrapolated to all layers."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("sft_oracle", os.path.join(ROOT, "oracle", "sft_oracle.py"))
    o = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(o)
    rng = np.random.default_rng(0)
    D, hd, IS, V = sp.d_model, sp.head_dim, sp.intermediate_size, sp.vocab_size
    Hq, Hkv = sp.n_q_heads, sp.n_kv_heads

    def mat(r, c):
        return o.f16_round((rng.standard_normal((r, c)) * 0.02).astype(np.float32))

    layer = dict(q=mat(Hq * hd, D), k=mat(Hkv * hd, D), v=mat(Hkv * hd, D), o=mat(D, Hq * hd), gate=mat(IS, D),
                 up=mat(IS, D), down=mat(D, IS), input_norm=np.ones(D, np.float32), post_attn_norm=np.ones(D, np.float32),
                 q_norm=np.ones(hd, np.float32), k_norm=np.ones(hd, np.float32))
    lm, emb = mat(V, D), mat(V, D)
    lor = dict(A_q=(rng.standard_normal((rank, D)) * 0.01).astype(np.float32), B_q=np.zeros((Hq * hd, rank), np.float32),
               A_v=(rng.standard_normal((rank, D)) * 0.01).astype(np.float32), B_v=np.zeros((Hkv * hd, rank), np.float32))
    toks = rng.integers(0, V, seq + 1)
    times = []
    for nl in (1, 2):
        cfg = dict(d_model=D, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=hd, intermediate_size=IS, vocab_size=V, n_layers=nl,
                   rope_theta=sp.rope_theta, eps=1e-6)
        w = o.Weights(cfg, [layer] * nl, lm, np.ones(D, np.float32), emb)
        lora = o.LoRA([lor] * nl, rank, alpha)
        o.train_step(w, lora, toks[:-1], toks[1:], 1e-4)
        t0 = time.time()
        o.train_step(w, lora, toks[:-1], toks[1:], 1e-4)
        times.append(time.time() - t0)
    t_layer = max(times[1] - times[0], 1e-6)
    t_head = max(times[0] - t_layer, 0.0)
    total = t_head + t_layer * sp.n_layers
    return {"value": seq / total, "unit": "tok/s", "cores": os.cpu_count() or 1, "kind": "port",
            "sample": f"numpy restatement, one sequence of {seq} tokens per step: 1- and 2-layer cuts + full LM head, "
                      f"{t_layer * 1e3:.0f} ms/layer, {t_head * 1e3:.0f} ms head+loss, extrapolated to {sp.n_layers} layers"}


BATCH_WORKLOADS = {
    # name: (architecture, batch, prompt, generate, max_seq)
    "qwen3-4b-f16-batch32": ("qwen3-4b", 32, 128, 128, 512),
    "tiny-qwen3-f16-batch8": ("tiny-qwen3", 8, 16, 32, 64),
}


def batch_main(args, rank, local_rank, world):
    """Batched F16 decode: B sequences share one read of the weights per step (replicas at N > 1)."""
    arch, B, P, G, max_seq = BATCH_WORKLOADS[args.workload]
    P, G = args.prompt_len or P, args.gen_len or G
    pkg = entry.load_package()
    S = pkg.synth()
    sp = pkg.spec(arch)
    if args.layers:
        sp.n_layers = args.layers
    threads = max(1, min(32, (os.cpu_count() or 8) // max(world, 1)))
    config = {"workload": f"{arch} F16 batched greedy decode, batch {B} per GPU, prompt {P}, generate {G}",
              "batch": B, "prompt_len": P, "gen_len": G, "parallelism": f"replicas x{world}",
              "l2": "inputs larger than L2 (all weights streamed every step); no flush needed"}
    if args.impl == "reference":
        if rank == 0:
            cb = cpu_reference_sample(pkg, S, sp, threads)
            emit(json.dumps({"impl": "reference", "metric": "batched_decode_tokens_per_s", "value": cb["value"], "unit": "tok/s",
                             "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 / cb["value"],
                             "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                             "config": config, "cpu_baseline": cb,
                             "e2e": {"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                             "gpu_launches": 0}))
        return 0
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    L = pkg.lib()
    cfg = pkg.config_of(sp, pkg.MODEL_QWEN3, max_seq, 1)
    st = L.llmb200_batch_begin(C.byref(cfg), B, G)
    if not st:
        raise RuntimeError("llmb200_batch_begin failed")
    D, hd, IS, V = sp.d_model, sp.head_dim, sp.intermediate_size, sp.vocab_size
    shapes = [(sp.n_q_heads * hd, D), (sp.n_kv_heads * hd, D), (sp.n_kv_heads * hd, D), (D, sp.n_q_heads * hd),
              (IS, D), (IS, D), (D, IS)]
    ones_d, ones_h = np.ones(D, dtype=np.float32), np.ones(hd, dtype=np.float32)
    fp = pkg.c_float_p
    for layer in range(sp.n_layers):
        mats = [gen_f32(S, r * c, sp.seed, S.llmb200_synth_tensor_id(layer, w), sp.weight_std, threads)
                for w, (r, c) in enumerate(shapes)]
        ref = pkg.LayerWeightRef()
        for name, m, (r, c) in zip(["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"], mats, shapes):
            setattr(ref, name, pkg.WeightRef(m.ctypes.data_as(fp), r, c))
        ref.input_norm_g = ones_d.ctypes.data_as(fp)
        ref.post_attn_norm_g = ones_d.ctypes.data_as(fp)
        ref.q_norm_g = ones_h.ctypes.data_as(fp)
        ref.k_norm_g = ones_h.ctypes.data_as(fp)
        ref.d_model, ref.head_dim = D, hd
        if L.llmb200_batch_load_layer(st, layer, C.byref(ref), C.c_float(sp.rope_theta)) != 0:
            raise RuntimeError(f"loading layer {layer} failed")
        L.metal_flush()
    lm = gen_f32(S, V * D, sp.seed, S.llmb200_synth_tensor_id(0, 101), sp.weight_std, threads)
    emb = gen_f32(S, V * D, sp.seed, S.llmb200_synth_tensor_id(0, 100), sp.weight_std, threads)
    if L.llmb200_batch_finish(st, lm.ctypes.data_as(fp), ones_d.ctypes.data_as(fp), emb.ctypes.data_as(fp)) != 0:
        raise RuntimeError("llmb200_batch_finish failed")
    L.llmb200_batch_set_eos(st, None, 0)
    prompts = np.zeros((B, P), dtype=np.uint32)
    S.llmb200_synth_tokens(prompts.ctypes.data, B * P, 4321 + rank, sp.vocab_size)
    out = np.zeros((B, G), dtype=np.uint32)

    def one():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        n = L.llmb200_batch_generate(st, prompts.ctypes.data_as(pkg.c_u32_p), P, out.ctypes.data_as(pkg.c_u32_p), G)
        wall = (time.perf_counter() - t0) * 1e3          # the public call: host prompts in, host tokens out
        if n != G:
            raise RuntimeError(f"batch generate returned {n}")
        ns = C.c_int(0)
        ms = L.llmb200_batch_last_decode_ms(st, C.byref(ns))
        if world > 1:
            t = torch.tensor([ms, wall], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms, wall = float(t[0].item()), float(t[1].item())
        return ms, ns.value, wall

    for _ in range(args.warmup):
        one()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    runs = [one() for _ in range(args.steps)]
    clocks = sampler.stop() if rank == 0 else None
    ms = sum(r[0] for r in runs)
    steps = sum(r[1] for r in runs)
    wall_ms = sum(r[2] for r in runs)
    # every step (prompt positions included) replays one graph of this many kernels
    launches = int(L.llmb200_batch_graph_kernels(st)) * args.steps * (P + G - 1)
    value = steps * B * world / (ms / 1e3)
    per_layer = ((sp.n_q_heads + 2 * sp.n_kv_heads) * hd * D + D * sp.n_q_heads * hd + 3 * IS * D) * 2
    step_bytes = sp.n_layers * per_layer + V * D * 2 + B * sp.n_layers * 2 * sp.n_kv_heads * hd * 2 * (P + G // 2)
    peak, peak_kind = measured_peaks()
    ach = step_bytes / (ms / 1e3 / steps) / 1e9
    line = {"metric": "batched_decode_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "binary16 weights and tensor-core operands, fp32 accumulate", "data": "synthetic",
            "config": config,
            # the call runs P + G - 1 identical steps (prompt positions go through the same step graph);
            # the device-timed value covers the generating ones, the wall clock all of them
            "e2e": {"value": args.steps * (P + G - 1) * B * world / (wall_ms / 1e3), "unit": "tok/s", "h2d_bytes_per_step": int(B * P * 4), "d2h_bytes_per_step": int(B * G * 4)},
            "gpu_launches": launches,
            "roofline": {"bound": "hbm", "kernel": "whole decode step (binary16 weights once + KV rows of all sequences)",
                         "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "peak_source": peak_kind,
                         "traffic": None, "algorithmic_bytes_per_step": step_bytes},
            "ms_per_decode_step": ms / steps, "clocks": clocks, "first_tokens": out[0, :8].tolist()}
    L.llmb200_batch_free(st)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        emit(json.dumps(line))
    return 0


def sft_main(args, rank, local_rank, world):
    arch, seq, n_seq, lrank, alpha = SFT_WORKLOADS[args.workload]
    pkg = entry.load_package()
    S = pkg.synth()
    sp = pkg.spec(arch)
    if args.layers:
        sp.n_layers = args.layers
    threads = max(1, min(32, (os.cpu_count() or 8) // max(world, 1)))
    M = seq * n_seq
    config = {"workload": f"{arch}{'' if not args.layers else f' cut to {args.layers} layers'} LoRA SFT step, frozen F16-valued "
                          f"base, rank {lrank} alpha {alpha:g} on Q and V, seq {seq}, {n_seq} sequences per GPU, AdamW lr 1e-4",
              "seq_len": seq, "sequences_per_gpu": n_seq, "global_batch": n_seq * world, "parallelism": f"dp{world}",
              "l2": "inputs larger than L2 (every step streams all frozen weights, >> 126 MB); no flush needed"}
    if args.impl == "reference":
        if rank != 0:
            return 0
        cb = sft_cpu_port_sample(sp, seq, lrank, alpha)
        emit(json.dumps({"impl": "reference", "metric": "sft_tokens_per_s", "value": cb["value"], "unit": "tok/s",
                          "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                          "ms_per_step": 1000.0 * seq / cb["value"], "higher_is_better": True, "scaling": "weak",
                          "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config, "cpu_baseline": cb,
                          "e2e": {"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                          "gpu_launches": 0}))
        return 0

    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    L = pkg.lib()
    t0 = time.time()
    st = build_sft_streaming(pkg, L, S, sp, seq, n_seq, lrank, alpha, threads)
    build_s = time.time() - t0
    gp = C.c_void_p()
    n_grad = L.llmb200_sft_grad_vector(st, C.byref(gp))
    grads = torch.as_tensor(_DeviceVector(gp.value, n_grad), device="cuda") if world > 1 else None

    n_batches = args.steps + args.warmup
    toks = np.zeros((n_batches, n_seq, seq + 1), dtype=np.uint32)
    S.llmb200_synth_tokens(toks.ctypes.data, toks.size, 4321 + rank, sp.vocab_size)    # every rank its own sequences
    xs = np.ascontiguousarray(toks[:, :, :-1]).reshape(n_batches, M)
    ys = np.ascontiguousarray(toks[:, :, 1:]).reshape(n_batches, M)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    losses = []

    def step(i):
        """One optimizer step through the public calls; returns (device ms, wall ms)."""
        barrier()
        w0 = time.perf_counter()
        loss = L.llmb200_sft_forward_backward(st, xs[i].ctypes.data_as(pkg.c_u32_p), ys[i].ctypes.data_as(pkg.c_u32_p))
        ar_ms = 0.0
        if world > 1:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            dist.all_reduce(grads, op=dist.ReduceOp.SUM)       # LoRA-gradient exchange: sum, then the mean
            grads.mul_(1.0 / world)
            e1.record()
            torch.cuda.synchronize()
            ar_ms = e0.elapsed_time(e1)
        L.llmb200_sft_apply_update(st, 1e-4)
        wall = (time.perf_counter() - w0) * 1e3
        upd = C.c_float(0)
        dev = L.llmb200_sft_last_step_ms(st, C.byref(upd)) + upd.value + ar_ms
        barrier()
        losses.append(loss)
        return max_over_ranks(dev), max_over_ranks(wall)

    for i in range(args.warmup):
        step(i)
    L.b200_launch_count(1)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    timed = [step(args.warmup + i) for i in range(args.steps)]
    clocks = sampler.stop() if rank == 0 else None
    launches = int(L.b200_launch_count(0))
    if L.llmb200_sft_error(st):
        raise RuntimeError("the SFT engine reported an error")
    dev_ms = sum(d for d, _ in timed)
    wall_ms = sum(w for _, w in timed)
    tok = args.steps * M * world
    value, e2e_v = tok / (dev_ms / 1e3), tok / (wall_ms / 1e3)

    # dominant kernel alone: the gate/up forward product [M, 2*IS] = [M, D] x [2*IS, D]^T on the tensor cores
    D, IS = sp.d_model, sp.intermediate_size
    a = torch.randn(M, D, device="cuda").half()
    ws = [(torch.randn(2 * IS, D, device="cuda") * 0.02).half() for _ in range(3)]
    cbuf = torch.empty(M, 2 * IS, device="cuda")
    errw = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    def one(wt):
        g = pkg.GemmArgs()
        g.A, g.a_row, g.a_col = a.data_ptr(), D, 1
        g.B, g.b_row, g.b_col = wt.data_ptr(), 1, D
        g.C, g.ldc, g.M, g.N, g.K, g.alpha, g.d_err = cbuf.data_ptr(), 2 * IS, M, 2 * IS, D, 1.0, errw.data_ptr()
        return L.b200_gemm_f16(C.byref(g), C.c_void_p(stream))

    tc_ok = one(ws[0]) == 0
    roofline = None
    if tc_ok:
        for i in range(3):
            one(ws[i % 3])
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 30
        torch.cuda.synchronize()
        e0.record()
        for i in range(reps):
            one(ws[i % 3])
        e1.record()
        torch.cuda.synchronize()
        sec = e0.elapsed_time(e1) / 1e3 / reps
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                peak, peak_kind = float(json.load(f)["bf16_tflops"]), "measured (cuBLAS bf16 burst)"
        except Exception:
            peak, peak_kind = 1590.0, "fallback"
        ach = 2.0 * M * 2 * IS * D / sec / 1e12
        roofline = {"bound": "tensor", "kernel": f"gemm_tf32_kernel, binary16 operands: gate/up forward (M {M}, N {2 * IS}, K {D})",
                    "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak, "peak_source": peak_kind,
                    "traffic": None, "us_per_launch": sec * 1e6}
    step_flops = sft_flops_per_token(sp) * M
    line = {
        "metric": "sft_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "binary16 tensor-core operands (weights exact, activations rounded), fp32 accumulate; fp32 elsewhere",
        "data": "synthetic", "config": config,
        "e2e": {"value": e2e_v, "unit": "tok/s", "h2d_bytes_per_step": int(2 * M * 4), "d2h_bytes_per_step": int(M * 4 + 8)},
        "gpu_launches": launches, "roofline": roofline,
        "step_tflops_per_gpu": step_flops / (dev_ms / args.steps / 1e3) / 1e12,
        "clocks": clocks, "build_seconds": build_s, "losses": [float(x) for x in losses],
        "grad_norm_last": float(L.llmb200_sft_last_grad_norm(st)),
    }
    if world == 1 and not args.no_cpu_baseline and rank == 0:
        line["cpu_baseline"] = sft_cpu_port_sample(sp, seq, lrank, alpha)
    L.sft_state_free(st)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        emit(json.dumps(line))
    return 0



def sweep_main(args):
    """Config 2: standalone Q8_0 matvec over the six Qwen3-4B shapes, one GPU. Each shape rotates over enough
    weight copies to exceed L2 (>= 256 MB footprint, at least 8 copies), so every launch streams from HBM;
    timed with CUDA events on the launching stream. Beside it the reference's CPU matvec on dequantised fp32
    weights (oracle/_ref ref_linear, one thread)."""
    import torch
    pkg = entry.load_package()
    L, S = pkg.lib(), pkg.synth()
    torch.cuda.set_device(0)
    peak, peak_kind = measured_peaks()
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    rows_out = []
    sampler = ClockSampler(0)
    sampler.start()
    launches = 0
    for rows, cols in SWEEP_SHAPES:
        stride = L.b200_packed_row_stride(pkg.B200_WT_Q8, cols)
        one = stride * rows
        copies = max(8, -(-(256 << 20) // one))
        w = gen_f32(S, rows * cols, 1234, 7, 0.02, 16).reshape(rows, cols)
        d_src = torch.from_numpy(w).cuda()
        d_w = torch.empty(copies * one, dtype=torch.uint8, device="cuda")
        for c in range(copies):
            if L.b200_q8_pack(d_src.data_ptr(), cols, rows, cols, d_w.data_ptr() + c * one, stride, 0, 1, None) != 0:
                raise RuntimeError("pack failed")
        x = torch.from_numpy(gen_f32(S, cols, 99, 1, 1.0, 1)).cuda()
        y = torch.zeros(rows, dtype=torch.float32, device="cuda")
        a = pkg.MatvecArgs()
        a.row_stride, a.rows, a.cols, a.wtype = stride, rows, cols, pkg.B200_WT_Q8
        a.in_mode, a.d_in_vec = pkg.B200_IN_VEC, x.data_ptr()
        a.out_mode, a.n_out, a.eps = pkg.B200_OUT_STORE, 1, 1e-6
        a.d_out[0] = y.data_ptr()

        def launch(c):
            a.d_w = d_w.data_ptr() + c * one
            if L.b200_matvec(C.byref(a), None) != 0:
                raise RuntimeError("matvec failed")
        for c in range(copies):
            launch(c)
        torch.cuda.synchronize()
        reps = max(3, args.steps) * copies
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(reps):
            launch(i % copies)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / reps
        launches += reps
        alg = rows * cols * 34 // 32 + 4 * cols + 4 * rows
        entry_ = {"rows": rows, "cols": cols, "us_per_launch": us, "algorithmic_bytes": alg, "gbs": alg / us / 1e3,
                  "frac_of_hbm": alg / us / 1e3 / peak, "weight_copies": copies}
        if not args.no_cpu_baseline:
            import _oracle as O
            if O.have_ref():
                wd = O.q8_dequantize(O.q8_quantize(w), rows, cols)
                xv = x.cpu().numpy()
                yv = np.zeros(rows, dtype=np.float32)
                t0 = time.perf_counter()
                O.ref().ref_linear(wd.ctypes.data, xv.ctypes.data, yv.ctypes.data, rows, cols)
                entry_["cpu_reference_us"] = (time.perf_counter() - t0) * 1e6
                got = y.cpu().numpy()
                entry_["max_rel_err_vs_reference"] = float(np.abs(got - yv).max() / np.abs(yv).max())
        rows_out.append(entry_)
        del d_w, d_src
        torch.cuda.empty_cache()
    clocks = sampler.stop()
    big = rows_out[-1]
    total_bytes = sum(r["algorithmic_bytes"] for r in rows_out)
    total_us = sum(r["us_per_launch"] for r in rows_out)
    line = {"metric": "q8_matvec_hbm_gbs", "value": total_bytes / total_us / 1e3, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": total_us / 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 accumulate over int8 (Q8_0) weights", "data": "synthetic",
            "config": {"workload": "standalone Q8_0 matvec sweep, batch 1, six Qwen3-4B shapes", "shapes": [list(sh) for sh in SWEEP_SHAPES],
                       "l2": "rotating weight copies, >= 256 MB footprint per shape"},
            "e2e": {"value": total_bytes / total_us / 1e3, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                    "note": "a kernel-level sweep: inputs are device-resident by definition of the configuration"},
            "gpu_launches": launches, "shapes": rows_out, "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": "matvec_kernel<Q8_0> 151936 x 2560", "achieved": big["gbs"], "peak": peak, "unit": "GB/s",
                         "frac": big["frac_of_hbm"], "peak_source": peak_kind, "traffic": None,
                         "algorithmic_bytes_per_launch": big["algorithmic_bytes"]}}
    emit(json.dumps(line))
    return 0


def run_secondary(args):
    """The other configurations of the benchmark set, each in a child process (one GPU, few steps)."""
    out = {}
    for key, wl, extra in (("matvec_sweep_q8", "matvec-sweep", []), ("gemma3_1b_f16_decode", "gemma3-1b-f16", []),
                           ("qwen3_4b_sft_lora", "qwen3-4b-sft-lora", [])):
        cmd = [sys.executable, os.path.join(ROOT, "bench.py"), "--workload", wl, "--steps", "2", "--warmup", "3", "--no-secondary"] + extra
        if args.no_cpu_baseline or key == "qwen3_4b_sft_lora":
            cmd.append("--no-cpu-baseline")
        try:
            r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=600)
            lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
            d = json.loads(lines[-1]) if r.returncode == 0 and lines else None
        except Exception as e:                     # a failed secondary never takes the headline down
            d, r = None, None
            sys.stderr.write(f"[bench] secondary {wl} failed: {e}\n")
        if d is None:
            out[key] = {"failed": (r.stderr[-300:] if r is not None else "exception")}
            continue
        keep = {k: d[k] for k in ("metric", "value", "unit", "dtype", "ms_per_step", "steps", "warmup") if k in d}
        keep["workload"] = d["config"]["workload"]
        for k in ("token_roofline", "roofline", "shapes", "step_tflops_per_gpu", "e2e", "clocks", "parity"):
            if k in d:
                keep[k] = d[k]
        out[key] = keep
    return out


def wide_parity(pkg, L, S, rank, world, threads, dist):
    """Greedy tokens of the two-layer full-width cut of Qwen3-4B (Q8_0) on the GPU(s) of this run against the
    vectors the reference's own C code produced (tests/golden/wide_golden.npz); sampled logits of the last step."""
    import torch
    g = np.load(os.path.join(ROOT, "tests", "golden", "wide_golden.npz"))
    sp = pkg.spec("qwen3-4b", gamma_jitter=0.1, n_layers=int(g["layers"]))
    model = S.llmb200_synth_qwen3(C.byref(sp), threads)
    st = L.inference_state_create(model, int(g["max_seq"]), 0)
    L.metal_flush()
    S.llmb200_synth_free_qwen3(model)
    if not st:
        raise RuntimeError("parity model could not be created")
    if world > 1:
        connect_ranks(pkg, L, st, world, dist)
    L.llmb200_state_set_eos(st, None, 0)
    prompt, ref = g["qwen3_prompt"], g["qwen3_tokens"]
    out = np.zeros(len(ref), dtype=np.uint32)
    n = L.inference_generate(st, prompt.ctypes.data_as(pkg.c_u32_p), len(prompt), out.ctypes.data_as(pkg.c_u32_p), len(ref))
    L.inference_state_reset(st)
    lg = None
    for t in np.concatenate([prompt, ref[:-1]]):
        p = L.inference_forward_token(st, int(t))
        lg = np.ctypeslib.as_array(p, shape=(sp.vocab_size,)).copy()
    err = float(np.abs(lg[::int(g["stride"])] - g["qwen3_logit_sample"][-1]).max() / g["qwen3_logit_absmax"][-1])
    ok = n == len(ref) and list(out) == list(ref) and L.llmb200_state_error(st) == 0
    L.inference_state_free(st)
    if world > 1:
        t = torch.tensor([1.0 if ok else 0.0, -err], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        ok, err = bool(t[0].item() > 0.5), float(-t[1].item())
    return {"workload": "qwen3-4b widths, 2 layers, Q8_0, prompt 16, generate 32 (tests/golden/wide_golden.npz)",
            "tokens_match_reference": bool(ok), "max_rel_logit_err": err, "ranks": world}


def connect_ranks(pkg, L, st, world, dist):
    import torch
    h = (C.c_ubyte * pkg.LLMB200_HANDLE_BYTES)()
    if L.llmb200_state_comm_handle(st, h) != 0:
        raise RuntimeError("comm handle failed")
    mine = torch.tensor(list(h), dtype=torch.uint8, device="cuda")
    allh = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(allh, mine)
    table = bytes(torch.cat(allh).cpu().numpy().tobytes())
    if L.llmb200_state_connect(st, table, world) != 0:
        raise RuntimeError("connect failed")
    dist.barrier()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="qwen3-4b-q8",
                    choices=sorted(WORKLOADS) + sorted(SFT_WORKLOADS) + sorted(BATCH_WORKLOADS) + ["matvec-sweep"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="skip the secondary configurations and the parity stamp")
    ap.add_argument("--prompt-len", type=int, default=0, help="override the workload's prompt length (profiling runs)")
    ap.add_argument("--gen-len", type=int, default=0, help="override the workload's generation length (profiling runs)")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (small ncu captures)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.workload in SFT_WORKLOADS:
        return sft_main(args, rank, local_rank, world)
    if args.workload in BATCH_WORKLOADS:
        return batch_main(args, rank, local_rank, world)
    if args.workload == "matvec-sweep":
        if args.impl == "reference" or world > 1:
            if rank == 0:
                emit(json.dumps({"impl": args.impl, "unavailable": "the matvec sweep is a one-GPU kernel workload; its CPU reference "
                                 "timing is part of its own line"}))
            return 0
        return sweep_main(args)
    arch, use_fp16, P, G, max_seq = WORKLOADS[args.workload]
    P, G = args.prompt_len or P, args.gen_len or G
    pkg = entry.load_package()
    S = pkg.synth()
    sp = pkg.spec(arch)
    if args.layers:
        sp.n_layers = args.layers
    threads = max(1, min(32, (os.cpu_count() or 8) // max(world, 1)))
    gemma = arch.endswith("gemma3") or arch.startswith("gemma3")
    wname = "F16" if use_fp16 else "Q8_0"
    if gemma and world > 1:
        raise SystemExit("the Gemma3 workloads have one KV head: replicas only, run them at --gpus 1")
    config = {"workload": f"{arch}{'' if not args.layers else f' cut to {args.layers} layers'} {wname} batch-1 greedy decode, "
                          f"prompt {P}, generate {G}, F16 KV cache {max_seq}",
              "prompt_len": P, "gen_len": G, "kv_cache": "f16", "parallelism": f"tp{world}",
              "l2": "inputs larger than L2 (weights streamed per token >> 126 MB); no flush needed"}

    if args.impl == "reference":
        if rank != 0:
            return 0
        if gemma:
            emit(json.dumps({"impl": "reference", "unavailable": "the reference has no CPU Gemma3 forward (src/nn/gemma3.c "
                             "holds create/load only); the checker for this workload is a restatement"}))
            return 0
        cb = cpu_reference_sample(pkg, S, sp, threads)
        line = {"impl": "reference", "metric": "decode_tokens_per_s", "value": cb["value"], "unit": "tok/s", "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 / cb["value"] * (G - 1),
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": config, "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        emit(json.dumps(line))
        return 0

    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    L = pkg.lib()
    if L.llmb200_set_tp(rank, world) != 0:
        raise RuntimeError("llmb200_set_tp failed")
    parity = None
    if arch == "qwen3-4b" and not args.layers and not args.no_secondary:
        parity = wide_parity(pkg, L, S, rank, world, threads, dist)
    t0 = time.time()
    if gemma:
        model = S.llmb200_synth_gemma3(C.byref(sp), threads)
        st = L.inference_state_create_gemma3(model, max_seq, use_fp16)
        L.metal_flush()                          # uploads read the host weights until the stream has drained
        S.llmb200_synth_free_gemma3(model)       # the state holds its own device copies, embedding table included
        if not st:
            raise RuntimeError("inference_state_create_gemma3 failed")
    else:
        st = build_state_streaming(pkg, L, S, sp, max_seq, use_fp16, threads)
    if world > 1:
        connect_ranks(pkg, L, st, world, dist)
    build_s = time.time() - t0
    L.llmb200_state_set_eos(st, None, 0)          # uniform random ids: never stop early

    prompt = np.zeros(P, dtype=np.uint32)
    S.llmb200_synth_tokens(prompt.ctypes.data, P, 4321, sp.vocab_size)
    out = np.zeros(G, dtype=np.uint32)
    pp, op = prompt.ctypes.data_as(pkg.c_u32_p), out.ctypes.data_as(pkg.c_u32_p)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def device_step():
        # prefill + first token through the public call, then the decode forwards from device memory
        if L.inference_generate(st, pp, P, op, 1) != 1:
            raise RuntimeError("prefill failed")
        barrier()
        ms = L.llmb200_state_run_device_steps(st, G - 1)
        if ms <= 0:
            raise RuntimeError("device steps failed")
        barrier()
        return max_over_ranks(ms)

    def e2e_step():
        barrier()
        t_call = time.perf_counter()
        n = L.inference_generate(st, pp, P, op, G)
        wall_ms = (time.perf_counter() - t_call) * 1e3
        nd = C.c_int(0)
        ms = L.llmb200_last_decode_ms(st, C.byref(nd))
        barrier()
        if n != G:
            raise RuntimeError(f"generate returned {n} tokens")
        return max_over_ranks(ms), nd.value, max_over_ranks(wall_ms)

    for _ in range(args.warmup):
        device_step()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    step_ms = [device_step() for _ in range(args.steps)]
    e2e = [e2e_step() for _ in range(args.steps)]
    clocks = sampler.stop() if rank == 0 else None
    first_tokens = out[:8].tolist()
    if L.llmb200_state_error(st):
        raise RuntimeError("a device-side wait timed out")

    per_token_kernels = L.llmb200_state_graph_kernels(st, 1)
    token_kernel = per_token_kernels == 1
    peak, peak_kind = measured_peaks()
    n_tok = args.steps * (G - 1)
    value = n_tok / (sum(step_ms) / 1e3)
    e2e_ms = sum(m for m, _, _ in e2e)
    e2e_tok = sum(n for _, n, _ in e2e)
    call_ms = sum(w for _, _, w in e2e)
    mean_bytes = float(np.mean([algorithmic_bytes_per_token(sp, n, world, use_fp16, gemma) for n in range(P + 1, P + G)]))
    us_per_token = 1e3 * sum(step_ms) / n_tok
    prof = {}
    if token_kernel:
        # one persistent kernel per token: its launches are the timed region itself
        prof["decode_token_kernel"] = {"us_per_launch": us_per_token, "launches_timed": n_tok, "launches_per_token": 1}
        achieved = mean_bytes / (us_per_token * 1e-6) / 1e9
        tr = TOKEN_TRAFFIC.get(arch)
        traffic = None
        if tr and world == 1 and not args.layers:
            traffic = int(tr["per_layer"] * sp.n_layers + tr["rest"])
        roofline = {"bound": "hbm", "kernel": "decode_token_kernel<%s> (whole token: %d layers + LM head)" % (wname, sp.n_layers),
                    "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_kind,
                    "traffic": traffic,
                    "traffic_source": ("ncu captures of a 4- and an 8-layer cut, scaled by layers (profiles/)" if traffic else
                                       "none at N > 1 or for cuts: DRAM bytes are only measured on one GPU"),
                    "algorithmic_bytes_per_launch": int(mean_bytes)}
    else:
        # one kernel per stage: each kind launched back to back over all layers (different weights every launch,
        # so L2 cannot serve them) between two CUDA events on the library's stream
        barrier()                                                # the ranks must enter the next request together
        L.inference_generate(st, pp, P, op, 1)
        L.llmb200_state_run_device_steps(st, (G - 1) // 2)       # to the middle of the decode range
        names = ["qkv_matvec", "attention", "o_matvec", "gateup_matvec", "down_matvec", "lm_head_matvec"]
        for i, nme in enumerate(names):
            nl = C.c_int(0)
            ms = L.llmb200_state_time_kind(st, i, 8 if i < 5 else 24, C.byref(nl))
            if ms <= 0 or nl.value <= 0:
                raise RuntimeError("kernel timing failed")
            prof[nme] = {"us_per_launch": 1e3 * ms / nl.value, "launches_timed": nl.value,
                         "launches_per_token": sp.n_layers if i < 5 else 1}
        D, IS = sp.d_model, sp.intermediate_size
        gu_rows, gu_cols = 2 * IS // world, D
        gu_bytes = int(gu_rows * gu_cols * (2 if use_fp16 else 34 / 32) + 4 * gu_cols + 4 * (gu_rows // 2))
        achieved = gu_bytes / (1e-6 * prof["gateup_matvec"]["us_per_launch"]) / 1e9
        roofline = {"bound": "hbm", "kernel": "matvec_kernel<%s> gate/up (rows %d x cols %d)" % (wname, gu_rows, gu_cols),
                    "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_kind,
                    "traffic": GATEUP_TRAFFIC_BYTES if (arch == "qwen3-4b" and world == 1) else None,
                    "traffic_source": "ncu capture of the N=1 4-layer cut (profiles/matvec_gateup_qwen3-4b_4layers_full.md)",
                    "algorithmic_bytes_per_launch": gu_bytes}
    line = {
        "metric": "decode_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sum(step_ms) / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32 accumulate over %s weights" % ("binary16" if use_fp16 else "int8 (Q8_0)"),
        "data": "synthetic", "config": config,
        # e2e.value: the reference's own metric (decode loop only, src/nn/fast_inference.c:643-672) through
        # inference_generate with host buffers; whole_call_*: wall clock around the entire call, prefill included
        "e2e": {"value": e2e_tok / (e2e_ms / 1e3), "unit": "tok/s", "h2d_bytes_per_step": int(P * 4 + 8),
                "d2h_bytes_per_step": int(G * 4), "whole_call_ms": call_ms / args.steps,
                "whole_call_tokens_per_s": args.steps * (P + G - 1) / (call_ms / 1e3)},
        "gpu_launches": int(args.steps * (G - 1) * per_token_kernels),
        "roofline": roofline,
        "token_roofline": {"bytes_per_token_per_gpu": mean_bytes, "achieved_gbs": mean_bytes * value / 1e9,
                           "frac_of_hbm": mean_bytes * value / 1e9 / peak, "peak_source": peak_kind},
        "kernels": prof, "clocks": clocks, "ms_per_token": sum(step_ms) / n_tok, "build_seconds": build_s,
        "first_tokens": first_tokens,
    }
    if parity is not None:
        line["parity"] = parity
    if world > 1:
        line["exchange"] = {"impl": "partial sums stored with their flags into every rank's slot over NVLink (plain peer stores), summed "
                                    "in rank order inside the consumer stage of the same kernel; no separate all-reduce kernel",
                            "exchanges_per_token": 2 * sp.n_layers,
                            # everything a layer costs (rows, attention, five hand-overs, both exchanges), halved:
                            # an upper bound on what one fused exchange can cost
                            "us_per_token_over_exchanges": 1e3 * sum(step_ms) / n_tok / (2 * sp.n_layers),
                            "nccl_arm": nccl_exchange_arm(torch, dist, sp.d_model, 2 * sp.n_layers, max_over_ranks)}
    if world == 1 and not args.no_cpu_baseline and not gemma:
        if rank == 0:
            line["cpu_baseline"] = cpu_reference_sample(pkg, S, sp, threads)
    L.inference_state_free(st)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if world == 1 and arch == "qwen3-4b" and not args.layers and not args.no_secondary:
        torch.cuda.empty_cache()
        line["secondary"] = run_secondary(args)
    if rank == 0:
        emit(json.dumps(line))
    return 0


def nccl_exchange_arm(torch, dist, d_model, per_token, max_over_ranks):
    """The exchange as a stage-by-stage design would do it: an NCCL all-reduce (sum) of one d_model fp32 vector
    after the o and after the down projection, i.e. 2 x layers calls per token. Timed on its own, the calls of
    one token captured in a CUDA graph (no host launch cost), CUDA events, max over ranks. A comparison figure
    beside the fused exchange of the token kernel; nothing of it is on the measured decode path."""
    try:
        x = torch.zeros(d_model, dtype=torch.float32, device="cuda")
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            for _ in range(8):
                dist.all_reduce(x)
        s.synchronize()
        mode = "the calls of one token in a CUDA graph"
        g, captured = None, 1.0
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                for _ in range(per_token):
                    dist.all_reduce(x)
        except Exception:                                         # capture refused on this rank
            captured = 0.0
            torch.cuda.synchronize()
        # every rank must time the same thing: replay only if all of them captured
        if max_over_ranks(-captured) > -1.0:
            mode = "eager launches (host launch cost included)"

            def run():
                for _ in range(per_token):
                    dist.all_reduce(x)
        else:
            run = g.replay
        reps = 20
        with torch.cuda.stream(s):
            for _ in range(3):
                run()
            s.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(s)
            for _ in range(reps):
                run()
            e1.record(s)
            e1.synchronize()
        us = max_over_ranks(1e3 * e0.elapsed_time(e1) / (reps * per_token))
        return {"us_per_allreduce": us, "us_per_token": us * per_token, "bytes": 4 * d_model, "mode": mode,
                "what": "torch.distributed all_reduce (NCCL, sum) of one d_model fp32 vector, back to back"}
    except Exception as exc:                                      # a comparison figure must not cost the bench line
        return {"unavailable": "%s: %s" % (type(exc).__name__, str(exc)[:200])}


if __name__ == "__main__":
    sys.exit(main())
