"""Reader of the record files tests/c_api/grpo_drop_in.c writes (one per run of the reference's GRPO loop)."""
import numpy as np

REWARD, LEN, TOKENS, LOGPROBS, REWARDS, ADVANTAGES, GRADS, NEW_LP, ADAPTER, SFT_LOSS, CKPT_HEAD, CKPT_SAMPLE, CKPT_SUMS = range(1, 14)
GROUP, MAX_GEN, STEPS = 4, 8, 2


def read(path):
    """-> list of (kind, float32 array) in file order."""
    raw = np.fromfile(path, dtype=np.int32)
    out, i = [], 0
    while i < len(raw):
        kind, n = int(raw[i]), int(raw[i + 1])
        assert 1 <= kind <= 13 and n >= 0 and i + 2 + n <= len(raw), "malformed record file"
        out.append((kind, raw[i + 2:i + 2 + n].view(np.float32).copy()))
        i += 2 + n
    return out


def by_step(sections):
    """-> (steps, tail): steps[k] maps kind -> array (GRADS: the list of all gradient buffers in order); tail maps
    the kinds written after the last step (SFT_LOSS, then ADAPTER or the CKPT_* sections) to their arrays."""
    steps, cur, tail = [], None, {}
    for kind, v in sections:
        if kind == REWARD:
            cur = {GRADS: []}
            steps.append(cur)
        if kind >= ADAPTER:
            tail[kind] = v
        elif kind == GRADS:
            cur[GRADS].append(v)
        else:
            cur[kind] = v
    return steps, tail
