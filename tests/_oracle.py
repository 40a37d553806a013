"""ctypes access to the checkers under oracle/ (test infrastructure only).

liboracle.so is the CPU restatement; oracle/_ref/libllmref.so is the reference's
own C code compiled in place (present only where it was built).
"""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
LIB = os.path.join(ORACLE_DIR, "liboracle.so")
REF_LIB = os.path.join(ORACLE_DIR, "_ref", "libllmref.so")

_o = None
_r = None
vp, i32, sz = C.c_void_p, C.c_int, C.c_size_t


def lib():
    global _o
    if _o is None:
        if not os.path.exists(LIB):
            subprocess.run(["make", "-C", ORACLE_DIR, "liboracle.so"], check=True, stdout=subprocess.DEVNULL)
        o = C.CDLL(LIB)
        o.oracle_q8_quantize.argtypes = [vp, i32, i32, vp]
        o.oracle_q8_dequantize.argtypes = [vp, sz, vp]
        o.oracle_f16_bits.argtypes = [vp, sz, vp]
        o.oracle_q8_matvec.argtypes = [vp, vp, vp, i32, i32]
        o.oracle_f16_matvec.argtypes = [vp, vp, vp, i32, i32]
        o.oracle_linear.argtypes = [vp, vp, vp, i32, i32]
        o.oracle_rms_norm.argtypes = [vp, vp, vp, i32, C.c_float]
        o.oracle_model_qwen3.restype, o.oracle_model_qwen3.argtypes = vp, [vp, i32, i32]
        o.oracle_model_gemma3.restype, o.oracle_model_gemma3.argtypes = vp, [vp, i32, i32]
        o.oracle_model_free.argtypes = [vp]
        o.oracle_model_set_kv_f16.argtypes = [vp, i32]
        o.oracle_forward_token.argtypes = [vp, i32, i32, vp]
        o.oracle_generate.restype = i32
        o.oracle_generate.argtypes = [vp, vp, i32, vp, i32, vp, i32, vp, vp]
        _o = o
    return _o


def have_ref():
    return os.path.exists(REF_LIB)


def ref():
    global _r
    if _r is None:
        r = C.CDLL(REF_LIB)
        r.ref_q8_blocks.restype, r.ref_q8_blocks.argtypes = sz, [vp, i32, i32, vp]
        r.ref_f16_bits.restype, r.ref_f16_bits.argtypes = sz, [vp, i32, i32, vp]
        r.ref_requant_qwen3.argtypes = [vp, i32]
        r.ref_requant_gemma3.argtypes = [vp, i32]
        r.ref_qwen3_generate.restype = i32
        r.ref_qwen3_generate.argtypes = [vp, vp, i32, vp, i32, i32, vp, i32, vp, vp]
        r.ref_gemma3_generate.restype = i32
        r.ref_gemma3_generate.argtypes = [vp, i32, vp, i32, vp, i32, i32, vp, i32, vp, vp]
        r.ref_qwen3_forward_full.argtypes = [vp, vp, i32, vp]
        r.ref_linear.argtypes = [vp, vp, vp, i32, i32]
        r.ref_abi_layout.restype, r.ref_abi_layout.argtypes = i32, [C.POINTER(sz), i32]
        _r = r
    return _r


def q8_quantize(w):
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, cols = w.shape
    out = np.zeros(rows * (cols // 32) * 34, dtype=np.uint8)
    lib().oracle_q8_quantize(w.ctypes.data, rows, cols, out.ctypes.data)
    return out


def q8_dequantize(blocks, rows, cols):
    out = np.zeros((rows, cols), dtype=np.float32)
    lib().oracle_q8_dequantize(blocks.ctypes.data, rows * cols // 32, out.ctypes.data)
    return out


def f16_bits(w):
    w = np.ascontiguousarray(w, dtype=np.float32)
    out = np.zeros(w.size, dtype=np.uint16)
    lib().oracle_f16_bits(w.ctypes.data, w.size, out.ctypes.data)
    return out.reshape(w.shape)


def q8_matvec(blocks, x, rows, cols):
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.zeros(rows, dtype=np.float32)
    lib().oracle_q8_matvec(blocks.ctypes.data, x.ctypes.data, y.ctypes.data, rows, cols // 32)
    return y


def f16_matvec(wbits, x):
    rows, cols = wbits.shape
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.zeros(rows, dtype=np.float32)
    lib().oracle_f16_matvec(wbits.ctypes.data, x.ctypes.data, y.ctypes.data, rows, cols)
    return y


def linear(w, x):
    w = np.ascontiguousarray(w, dtype=np.float32)
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.zeros(w.shape[0], dtype=np.float32)
    lib().oracle_linear(w.ctypes.data, x.ctypes.data, y.ctypes.data, w.shape[0], w.shape[1])
    return y


class Model:
    def __init__(self, handle, vocab):
        self.h, self.vocab = handle, vocab

    def __del__(self):
        if self.h:
            lib().oracle_model_free(self.h)
            self.h = None


def model_qwen3(model_ptr, use_fp16, max_seq, vocab=None, kv_f16=False):
    h = lib().oracle_model_qwen3(model_ptr, use_fp16, max_seq)
    lib().oracle_model_set_kv_f16(h, 1 if kv_f16 else 0)
    return Model(h, vocab)


def model_gemma3(model_ptr, use_fp16, max_seq, vocab=None, kv_f16=False):
    h = lib().oracle_model_gemma3(model_ptr, use_fp16, max_seq)
    lib().oracle_model_set_kv_f16(h, 1 if kv_f16 else 0)
    return Model(h, vocab)


def generate(model, prompt, max_gen, eos=(), vocab=None, want_logits=False):
    """Greedy loop; returns (tokens, logits or None)."""
    prompt = np.ascontiguousarray(prompt, dtype=np.uint32)
    out = np.zeros(max_gen, dtype=np.uint32)
    e = np.asarray(list(eos), dtype=np.int32)
    V = vocab or model.vocab
    logits = np.zeros((max_gen, V), dtype=np.float32) if want_logits else None
    secs = np.zeros(2, dtype=np.float64)
    n = lib().oracle_generate(model.h, prompt.ctypes.data, len(prompt), out.ctypes.data, max_gen,
                              e.ctypes.data if len(e) else None, len(e),
                              logits.ctypes.data if want_logits else None, secs.ctypes.data)
    generate.last_seconds = (float(secs[0]), float(secs[1]))
    return out[:n], (logits[:n] if want_logits else None)


def forward_token(model, token, pos, vocab=None):
    V = vocab or model.vocab
    lg = np.zeros(V, dtype=np.float32)
    lib().oracle_forward_token(model.h, int(token), int(pos), lg.ctypes.data)
    return lg
