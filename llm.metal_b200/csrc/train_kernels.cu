// Row-wise and attention kernels of the LoRA-SFT step (everything but the GEMMs).
//
// Arithmetic follows shaders/q8_kernels.metal: rms_norm :133-158,
// rms_norm_train_backward :584-624, rope_train :495-538, rope_train_bwd
// :997-1040, attn_train_fwd :769-851, attn_bwd_dq :857-925, attn_bwd_dkv
// :931-968, repeat_kv / repeat_kv_bwd :476-492 / :973-992 (folded into the
// indexing), silu_mul :337-348, silu_mul_backward :540-556, softmax_ce_train
// :646-690, scale_tensor :627-633, clamp_tensor :1155-1161; the optimiser
// follows src/nn/fast_sft.c:1045-1107. All fp32 (the gradient norm in double).
//
// These kernels move little data next to the projections (a few MB per layer
// against hundreds of MB of weights); they are written for fusion -- no
// transposed or repeated copies, residual adds and scalings folded in -- rather
// than for peak bandwidth.
#include "common.cuh"
#include "../../include/llmb200_train_kernels.h"

extern unsigned long long g_b200_launches;

namespace {

// ---- embedding -----------------------------------------------------------------------------
__global__ void embed_rows_kernel(const float *emb, const uint32_t *tokens, int dim, int vocab, float scale, float *x)
{
    const int m = blockIdx.x;
    uint32_t t = tokens[m];
    if (t >= (uint32_t)vocab) t = 0;                                  // never read outside the table
    const float *src = emb + (size_t)t * dim;
    float *dst = x + (size_t)m * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) dst[i] = src[i] * scale;
}

// ---- RMSNorm over rows: a group of G threads per row (G = 32 for short rows, 256 for long ones) -----
template <int G>
__device__ __forceinline__ float group_sum_f(float v, float *sh)
{
    v = warp_sum(v);
    if (G == 32) return v;
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) sh[w] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < G / 32; ++i) t += sh[i];
    return t;
}

template <int G>
__global__ void __launch_bounds__(256)
rms_norm_rows_kernel(const float *x, const float *gamma, float *out, __half *out_h, int rows, int dim, float eps)
{
    __shared__ float sh[8];
    const int row = blockIdx.x * (256 / G) + threadIdx.x / G;
    const int l = threadIdx.x % G;
    const bool on = row < rows;
    const float *xr = x + (size_t)(on ? row : 0) * dim;
    float ss = 0.f;
    if (on) for (int i = l; i < dim; i += G) { const float v = xr[i]; ss = fmaf(v, v, ss); }
    ss = group_sum_f<G>(ss, sh);
    if (!on) return;
    const float inv = rsqrtf(ss / (float)dim + eps);
    float *o = out + (size_t)row * dim;
    for (int i = l; i < dim; i += G) {
        const float v = xr[i] * inv * gamma[i];
        o[i] = v;
        if (out_h) out_h[(size_t)row * dim + i] = __float2half_rn(v);
    }
}

template <int G>
__global__ void __launch_bounds__(256)
rms_norm_bwd_rows_kernel(const float *x, const float *dy, long long dy_ld, const float *gamma, float *dx, int rows,
                         int dim, float eps, int accumulate, float clamp, __half *dx_h, float h_scale)
{
    __shared__ float sh[8];
    const int row = blockIdx.x * (256 / G) + threadIdx.x / G;
    const int l = threadIdx.x % G;
    const bool on = row < rows;
    const float *xr = x + (size_t)(on ? row : 0) * dim, *dr = dy + (size_t)(on ? row : 0) * dy_ld;
    float ss = 0.f, dot = 0.f;
    if (on) for (int i = l; i < dim; i += G) {
        const float v = xr[i];
        ss = fmaf(v, v, ss);
        dot = fmaf(dr[i] * gamma[i], v, dot);
    }
    ss = group_sum_f<G>(ss, sh);
    dot = group_sum_f<G>(dot, sh);
    if (!on) return;
    const float inv = rsqrtf(ss / (float)dim + eps);
    const float coeff = dot * inv * inv / (float)dim;
    float *o = dx + (size_t)row * dim;
    for (int i = l; i < dim; i += G) {
        float v = (gamma[i] * dr[i] - coeff * xr[i]) * inv;
        if (accumulate) v += o[i];
        if (clamp > 0.f) v = fminf(fmaxf(v, -clamp), clamp);
        o[i] = v;
        if (dx_h) dx_h[(size_t)row * dim + i] = __float2half_rn(v * h_scale);
    }
}

// ---- QK-norm + RoPE: one warp per (row, head) -----------------------------------------------
// Heads 0..n_q-1 are q heads, n_q..n_q+n_kv-1 the k heads; both sit in qkv at column head*hd.
template <int HD>
__global__ void qk_norm_rope_kernel(const float *qkv, long long ld, const float *qg, const float *kg,
                                    const float *inv_freq, int rows, int seq_len, int n_q, int n_kv, float eps,
                                    float *q_out, float *k_out)
{
    constexpr int PER = HD / 64;                       // rotation pairs per lane
    const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int nh = n_q + n_kv;
    if (unit >= rows * nh) return;
    const int row = unit / nh, h = unit % nh, l = threadIdx.x & 31;
    const float *src = qkv + (size_t)row * ld + (size_t)h * HD;
    const float *g = h < n_q ? qg : kg;
    float *dst = h < n_q ? q_out + ((size_t)row * n_q + h) * HD : k_out + ((size_t)row * n_kv + (h - n_q)) * HD;
    float a[PER], b[PER];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < PER; ++c) {
        a[c] = src[l + 32 * c];
        b[c] = src[l + 32 * c + HD / 2];
        ss = fmaf(a[c], a[c], ss);
        ss = fmaf(b[c], b[c], ss);
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)HD + eps);
    const float pos = (float)(row % seq_len);
#pragma unroll
    for (int c = 0; c < PER; ++c) {
        const int d = l + 32 * c;
        const float x0 = a[c] * inv * g[d], x1 = b[c] * inv * g[d + HD / 2];
        float sn, cs;
        sincosf(pos * inv_freq[d], &sn, &cs);
        dst[d] = x0 * cs - x1 * sn;
        dst[d + HD / 2] = x0 * sn + x1 * cs;
    }
}

template <int HD>
__global__ void qk_norm_rope_bwd_kernel(float *dqkv, const float *qkv, long long ld, long long dld, const float *qg, const float *kg,
                                        const float *inv_freq, int rows, int seq_len, int n_q, int n_kv, float eps)
{
    constexpr int PER = HD / 64;
    const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int nh = n_q + n_kv;
    if (unit >= rows * nh) return;
    const int row = unit / nh, h = unit % nh, l = threadIdx.x & 31;
    const float *x = qkv + (size_t)row * ld + (size_t)h * HD;
    float *d = dqkv + (size_t)row * dld + (size_t)h * HD;
    const float *g = h < n_q ? qg : kg;
    const float pos = (float)(row % seq_len);
    float xa[PER], xb[PER], ga[PER], gb[PER];
    float ss = 0.f, dot = 0.f;
#pragma unroll
    for (int c = 0; c < PER; ++c) {
        const int i = l + 32 * c;
        float sn, cs;
        sincosf(pos * inv_freq[i], &sn, &cs);
        const float y0 = d[i], y1 = d[i + HD / 2];
        ga[c] = y0 * cs + y1 * sn;                     // rotation by -angle
        gb[c] = -y0 * sn + y1 * cs;
        xa[c] = x[i];
        xb[c] = x[i + HD / 2];
        ss = fmaf(xa[c], xa[c], ss);
        ss = fmaf(xb[c], xb[c], ss);
        dot = fmaf(ga[c] * g[i], xa[c], dot);
        dot = fmaf(gb[c] * g[i + HD / 2], xb[c], dot);
    }
    ss = warp_sum(ss);
    dot = warp_sum(dot);
    const float inv = rsqrtf(ss / (float)HD + eps);
    const float coeff = dot * inv * inv / (float)HD;
#pragma unroll
    for (int c = 0; c < PER; ++c) {
        const int i = l + 32 * c;
        d[i] = (g[i] * ga[c] - coeff * xa[c]) * inv;
        d[i + HD / 2] = (g[i + HD / 2] * gb[c] - coeff * xb[c]) * inv;
    }
}

// ---- causal attention, training form: one warp per (sequence, head, query) ---------------------
// Dynamic shared memory per warp: HD floats (the query or d_out row) + N floats (the score row).
constexpr int ATT_WARPS = 4;

template <int HD>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attn_train_fwd_kernel(const float *q, const float *k, const float *v, long long v_ld, int n_seq, int N, int n_q,
                      int n_kv, float scale, float *probs, float *out, __half *out_h)
{
    extern __shared__ float sh[];
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    float *qs = sh + (size_t)w * (HD + N), *sc = qs + HD;
    const long long unit = (long long)blockIdx.x * ATT_WARPS + w;
    if (unit >= (long long)n_seq * n_q * N) return;
    const int i = (int)(unit % N), h = (int)((unit / N) % n_q), s = (int)(unit / ((long long)N * n_q));
    const int kvh = h / (n_q / n_kv);
    const size_t row0 = (size_t)s * N;
    const float *qr = q + ((row0 + i) * n_q + h) * HD;
    for (int d = l; d < HD; d += 32) qs[d] = qr[d];
    __syncwarp();

    float mx = -1e30f;
    for (int j = l; j <= i; j += 32) {
        const float4 *kr = reinterpret_cast<const float4 *>(k + ((row0 + j) * n_kv + kvh) * HD);
        float dot = 0.f;
#pragma unroll 8
        for (int d4 = 0; d4 < HD / 4; ++d4) {
            const float4 kk = kr[d4];
            dot = fmaf(qs[4 * d4], kk.x, dot);
            dot = fmaf(qs[4 * d4 + 1], kk.y, dot);
            dot = fmaf(qs[4 * d4 + 2], kk.z, dot);
            dot = fmaf(qs[4 * d4 + 3], kk.w, dot);
        }
        dot *= scale;
        sc[j] = dot;
        mx = fmaxf(mx, dot);
    }
    mx = warp_max(mx);
    float sum = 0.f;
    for (int j = l; j <= i; j += 32) {
        const float e = expf(sc[j] - mx);
        sc[j] = e;
        sum += e;
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    float *pr = probs + (((size_t)s * n_q + h) * N + i) * N;
    for (int j = l; j < N; j += 32) {
        const float p = j <= i ? sc[j] * inv : 0.f;
        if (j <= i) sc[j] = p;
        pr[j] = p;
    }
    __syncwarp();
    float *o = out + ((row0 + i) * n_q + h) * HD;
    for (int d = l; d < HD; d += 32) {
        float acc = 0.f;
        for (int j = 0; j <= i; ++j) acc = fmaf(sc[j], v[(row0 + j) * v_ld + (size_t)kvh * HD + d], acc);
        if (out) o[d] = acc;
        if (out_h) out_h[((row0 + i) * n_q + h) * HD + d] = __float2half_rn(acc);
    }
}

template <int HD>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attn_bwd_dq_kernel(const float *d_out, const float *probs, const float *k, const float *v, long long v_ld, int n_seq,
                   int N, int n_q, int n_kv, float scale, float *d_score, float *dqkv, long long ld)
{
    extern __shared__ float sh[];
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    float *os = sh + (size_t)w * (HD + N), *ds = os + HD;
    const long long unit = (long long)blockIdx.x * ATT_WARPS + w;
    if (unit >= (long long)n_seq * n_q * N) return;
    const int i = (int)(unit % N), h = (int)((unit / N) % n_q), s = (int)(unit / ((long long)N * n_q));
    const int kvh = h / (n_q / n_kv);
    const size_t row0 = (size_t)s * N;
    const float *dor = d_out + ((row0 + i) * n_q + h) * HD;
    for (int d = l; d < HD; d += 32) os[d] = dor[d];
    __syncwarp();
    const float *pr = probs + (((size_t)s * n_q + h) * N + i) * N;
    float dp = 0.f;
    for (int j = l; j <= i; j += 32) {
        const float4 *vr = reinterpret_cast<const float4 *>(v + (row0 + j) * v_ld + (size_t)kvh * HD);
        float dot = 0.f;
#pragma unroll 8
        for (int d4 = 0; d4 < HD / 4; ++d4) {
            const float4 vv = vr[d4];
            dot = fmaf(os[4 * d4], vv.x, dot);
            dot = fmaf(os[4 * d4 + 1], vv.y, dot);
            dot = fmaf(os[4 * d4 + 2], vv.z, dot);
            dot = fmaf(os[4 * d4 + 3], vv.w, dot);
        }
        ds[j] = dot;
        dp = fmaf(pr[j], dot, dp);
    }
    dp = warp_sum(dp);
    float *dsr = d_score + (((size_t)s * n_q + h) * N + i) * N;
    for (int j = l; j < N; j += 32) {
        const float g = j <= i ? pr[j] * (ds[j] - dp) * scale : 0.f;
        if (j <= i) ds[j] = g;
        dsr[j] = g;
    }
    __syncwarp();
    float *dq = dqkv + (row0 + i) * ld + (size_t)h * HD;
    for (int d = l; d < HD; d += 32) {
        float acc = 0.f;
        for (int j = 0; j <= i; ++j) acc = fmaf(ds[j], k[((row0 + j) * n_kv + kvh) * HD + d], acc);
        dq[d] = acc;
    }
}

// One warp per (sequence, kv head, key): dK and dV summed over the later queries of each q head
// of the group, then over the group in head order (attn_bwd_dkv followed by repeat_kv_bwd).
template <int HD>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attn_bwd_dkv_kernel(const float *d_score, const float *probs, const float *q, const float *d_out, int n_seq, int N,
                    int n_q, int n_kv, float *dqkv, long long ld)
{
    constexpr int PER = HD / 32;
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * ATT_WARPS + w;
    if (unit >= (long long)n_seq * n_kv * N) return;
    const int j = (int)(unit % N), kvh = (int)((unit / N) % n_kv), s = (int)(unit / ((long long)N * n_kv));
    const int G = n_q / n_kv;
    const size_t row0 = (size_t)s * N;
    float dk[PER], dv[PER];
#pragma unroll
    for (int c = 0; c < PER; ++c) dk[c] = dv[c] = 0.f;
    for (int g = 0; g < G; ++g) {
        const int h = kvh * G + g;
        const float *dsc = d_score + ((size_t)s * n_q + h) * N * N;
        const float *prc = probs + ((size_t)s * n_q + h) * N * N;
        float hk[PER], hv[PER];
#pragma unroll
        for (int c = 0; c < PER; ++c) hk[c] = hv[c] = 0.f;
        for (int i = j; i < N; ++i) {
            const float dsv = dsc[(size_t)i * N + j], pv = prc[(size_t)i * N + j];
            const float *qr = q + ((row0 + i) * n_q + h) * HD;
            const float *dor = d_out + ((row0 + i) * n_q + h) * HD;
#pragma unroll
            for (int c = 0; c < PER; ++c) {
                hk[c] = fmaf(dsv, qr[l + 32 * c], hk[c]);
                hv[c] = fmaf(pv, dor[l + 32 * c], hv[c]);
            }
        }
#pragma unroll
        for (int c = 0; c < PER; ++c) { dk[c] += hk[c]; dv[c] += hv[c]; }
    }
    float *dkr = dqkv + (row0 + j) * ld + (size_t)(n_q + kvh) * HD;
    float *dvr = dqkv + (row0 + j) * ld + (size_t)(n_q + n_kv + kvh) * HD;
#pragma unroll
    for (int c = 0; c < PER; ++c) { dkr[l + 32 * c] = dk[c]; dvr[l + 32 * c] = dv[c]; }
}

// ---- causal attention for short sequences (N <= 64): one block per (sequence, head) ----------------
// The whole 64 x 64 score tile of a head lives in shared memory and every product is a register-tiled
// shared-memory matmul (256 threads, 4 x 4 or 4 x HD/16 outputs each) instead of one warp walking the keys.
// Same arithmetic as the per-query kernels above (fp32 FMA, softmax with max subtraction).
constexpr int AT = 64;            // tile edge: queries and keys
constexpr int ATP = AT + 4;       // padded row of a transposed operand (keeps float4 reads aligned)

// dst[d][i] = src[i][d] for i < n (zero beyond), src rows `ld` floats apart. HD columns.
template <int HD>
__device__ __forceinline__ void load_transposed(float *dst, const float *src, long long ld, int n)
{
    for (int e = threadIdx.x; e < AT * HD; e += blockDim.x) {
        const int i = e / HD, d = e % HD;
        dst[d * ATP + i] = i < n ? src[(size_t)i * ld + d] : 0.f;
    }
}
template <int HD>
__device__ __forceinline__ void load_rows(float *dst, const float *src, long long ld, int n)
{
    for (int e = threadIdx.x; e < AT * HD; e += blockDim.x) {
        const int i = e / HD, d = e % HD;
        dst[i * HD + d] = i < n ? src[(size_t)i * ld + d] : 0.f;
    }
}

// acc[a][b] = sum_d At[d][4*ty + a] * Bt[d][4*tx + b]   (both operands transposed, ATP-padded)
template <int HD>
__device__ __forceinline__ void tile_abt(const float *At, const float *Bt, int ty, int tx, float (&acc)[4][4])
{
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
#pragma unroll 4
    for (int d = 0; d < HD; ++d) {
        const float4 av = *reinterpret_cast<const float4 *>(At + d * ATP + 4 * ty);
        const float4 bv = *reinterpret_cast<const float4 *>(Bt + d * ATP + 4 * tx);
        const float a4[4] = {av.x, av.y, av.z, av.w}, b4[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(a4[a], b4[b], acc[a][b]);
    }
}

// out[4*ty + a][CW*tx + c] = sum_j W(j, 4*ty + a) * B[j][CW*tx + c], j < n; W(j, r) = Wm[r*ATP + j] when
// !WT (the weight matrix is indexed [row][j]) or Wm[j*ATP + r] when WT (indexed [j][row]). B row-major [AT][HD].
template <int HD, bool WT>
__device__ __forceinline__ void tile_wb(const float *Wm, const float *B, int n, int ty, int tx, float (&acc)[4][HD / 16])
{
    constexpr int CW = HD / 16;
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < CW; ++c) acc[a][c] = 0.f;
    for (int j = 0; j < n; ++j) {
        float w[4];
        if (WT) {
            const float4 wv = *reinterpret_cast<const float4 *>(Wm + j * ATP + 4 * ty);
            w[0] = wv.x; w[1] = wv.y; w[2] = wv.z; w[3] = wv.w;
        } else {
#pragma unroll
            for (int a = 0; a < 4; ++a) w[a] = Wm[(4 * ty + a) * ATP + j];
        }
        float bv[CW];
#pragma unroll
        for (int c4 = 0; c4 < CW / 4; ++c4) {
            const float4 t = *reinterpret_cast<const float4 *>(B + j * HD + CW * tx + 4 * c4);
            bv[4 * c4] = t.x; bv[4 * c4 + 1] = t.y; bv[4 * c4 + 2] = t.z; bv[4 * c4 + 3] = t.w;
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int c = 0; c < CW; ++c) acc[a][c] = fmaf(w[a], bv[c], acc[a][c]);
    }
}

template <int HD>
__global__ void __launch_bounds__(256)
attn_fwd_tile_kernel(const float *q, const float *k, const float *v, long long v_ld, int N, int n_q, int n_kv,
                     float scale, float *probs, float *out, __half *out_h)
{
    extern __shared__ __align__(16) float sh[];
    // Two operand regions + the score tile: V takes over Q's region once the scores are done, which keeps
    // the block at ~87 KB (HD 128) so that two blocks share an SM.
    float *Qt = sh, *Kt = Qt + HD * ATP, *Vs = Qt, *P = Kt + HD * ATP;               // P [AT][ATP]
    const int h = blockIdx.x % n_q, s = blockIdx.x / n_q, kvh = h / (n_q / n_kv);
    const size_t row0 = (size_t)s * N;
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
    load_transposed<HD>(Qt, q + (row0 * n_q + h) * HD, (long long)n_q * HD, N);
    load_transposed<HD>(Kt, k + (row0 * n_kv + kvh) * HD, (long long)n_kv * HD, N);
    __syncthreads();
    float acc[4][4];
    tile_abt<HD>(Qt, Kt, ty, tx, acc);
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int i = 4 * ty + a, j = 4 * tx + b;
            P[i * ATP + j] = (j <= i && i < N) ? acc[a][b] * scale : -1e30f;
        }
    __syncthreads();                                          // everybody is done with Q: its region becomes V
    load_rows<HD>(Vs, v + row0 * v_ld + (size_t)kvh * HD, v_ld, N);
    {   // softmax: four threads per row, 16 columns each
        const int i = threadIdx.x / 4, part = threadIdx.x % 4;
        float *pr = P + i * ATP + 16 * part;
        float mx = -1e30f;
#pragma unroll
        for (int c = 0; c < 16; ++c) mx = fmaxf(mx, pr[c]);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        float e[16], sum = 0.f;
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            const int j = 16 * part + c;
            e[c] = (j <= i && i < N) ? expf(pr[c] - mx) : 0.f;
            sum += e[c];
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const float inv = i < N ? 1.0f / sum : 0.f;
        float *gp = probs + (((size_t)s * n_q + h) * N + i) * N;
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            const int j = 16 * part + c;
            const float p = e[c] * inv;
            pr[c] = p;
            if (i < N && j < N) gp[j] = p;
        }
    }
    __syncthreads();
    float o[4][HD / 16];
    tile_wb<HD, false>(P, Vs, N, ty, tx, o);
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        const int i = 4 * ty + a;
        if (i >= N) continue;
        const size_t base = ((row0 + i) * n_q + h) * HD + (HD / 16) * tx;
#pragma unroll
        for (int c = 0; c < HD / 16; ++c) {
            if (out) out[base + c] = o[a][c];
            if (out_h) out_h[base + c] = __float2half_rn(o[a][c]);
        }
    }
}

// Backward of one (sequence, head): dq into dqkv, this head's dK and dV into part[s][h][N][2][HD].
template <int HD>
__global__ void __launch_bounds__(256)
attn_bwd_tile_kernel(const float *d_out, const float *probs, const float *q, const float *k, const float *v,
                     long long v_ld, int N, int n_q, int n_kv, float scale, float *dqkv, long long ld, float *part)
{
    extern __shared__ __align__(16) float sh[];
    // Two operand regions (each holds a transposed [HD][ATP] or a row-major [AT][HD] tile), reloaded as the
    // four products go by, + the P and dS tiles: ~104 KB for HD 128, so that two blocks share an SM.
    float *R1 = sh, *R2 = R1 + HD * ATP, *P = R2 + HD * ATP, *dS = P + AT * ATP;
    float *dOt = R1, *Vt = R2, *Ks = R1, *Qs = R2, *dOs = R1;
    const int h = blockIdx.x % n_q, s = blockIdx.x / n_q, kvh = h / (n_q / n_kv);
    const size_t row0 = (size_t)s * N;
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
    const float *dop = d_out + (row0 * n_q + h) * HD;
    load_transposed<HD>(dOt, dop, (long long)n_q * HD, N);
    load_transposed<HD>(Vt, v + row0 * v_ld + (size_t)kvh * HD, v_ld, N);
    const float *gp = probs + ((size_t)s * n_q + h) * N * N;
    for (int e = threadIdx.x; e < AT * AT; e += blockDim.x) {
        const int i = e / AT, j = e % AT;
        P[i * ATP + j] = (i < N && j < N) ? gp[(size_t)i * N + j] : 0.f;
    }
    __syncthreads();
    float acc[4][4];
    tile_abt<HD>(dOt, Vt, ty, tx, acc);                       // d_raw[i][j] = dO_i . V_j
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int i = 4 * ty + a, j = 4 * tx + b;
            dS[i * ATP + j] = (j <= i && i < N) ? acc[a][b] : 0.f;
        }
    __syncthreads();                                          // dO^T and V^T are used up: bring in K and Q
    load_rows<HD>(Ks, k + (row0 * n_kv + kvh) * HD, (long long)n_kv * HD, N);
    load_rows<HD>(Qs, q + (row0 * n_q + h) * HD, (long long)n_q * HD, N);
    {   // d_score = p * (d_raw - sum_k p_k d_raw_k) * scale, four threads per row
        const int i = threadIdx.x / 4, part4 = threadIdx.x % 4;
        float *dr = dS + i * ATP + 16 * part4;
        const float *pr = P + i * ATP + 16 * part4;
        float dp = 0.f;
#pragma unroll
        for (int c = 0; c < 16; ++c) dp = fmaf(pr[c], dr[c], dp);
        dp += __shfl_xor_sync(0xffffffffu, dp, 1);
        dp += __shfl_xor_sync(0xffffffffu, dp, 2);
#pragma unroll
        for (int c = 0; c < 16; ++c) dr[c] = pr[c] * (dr[c] - dp) * scale;     // p is zero above the diagonal
    }
    __syncthreads();
    float o[4][HD / 16];
    tile_wb<HD, false>(dS, Ks, N, ty, tx, o);                 // dQ_i = sum_j dS[i][j] K_j
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        const int i = 4 * ty + a;
        if (i >= N) continue;
        float *dst = dqkv + (row0 + i) * ld + (size_t)h * HD + (HD / 16) * tx;
#pragma unroll
        for (int c = 0; c < HD / 16; ++c) dst[c] = o[a][c];
    }
    float *pk = part + (((size_t)s * n_q + h) * N) * 2 * HD;
    tile_wb<HD, true>(dS, Qs, N, ty, tx, o);                  // dK_j = sum_i dS[i][j] Q_i
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        const int j = 4 * ty + a;
        if (j >= N) continue;
#pragma unroll
        for (int c = 0; c < HD / 16; ++c) pk[(size_t)j * 2 * HD + (HD / 16) * tx + c] = o[a][c];
    }
    __syncthreads();                                          // K is used up: its region takes dO, row-major
    load_rows<HD>(dOs, dop, (long long)n_q * HD, N);
    __syncthreads();
    tile_wb<HD, true>(P, dOs, N, ty, tx, o);                  // dV_j = sum_i P[i][j] dO_i
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        const int j = 4 * ty + a;
        if (j >= N) continue;
#pragma unroll
        for (int c = 0; c < HD / 16; ++c) pk[(size_t)j * 2 * HD + HD + (HD / 16) * tx + c] = o[a][c];
    }
}

// dK, dV of a KV head = sum over its query heads in head order (repeat_kv_bwd), into the k and v blocks of dqkv.
__global__ void attn_bwd_reduce_kernel(const float *part, int n_seq, int N, int n_q, int n_kv, int hd, float *dqkv,
                                       long long ld)
{
    const int G = n_q / n_kv;
    const size_t total = (size_t)n_seq * N * n_kv * 2 * hd;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const int d = (int)(e % hd);
        const int which = (int)((e / hd) % 2);
        const int kvh = (int)((e / (2 * hd)) % n_kv);
        const size_t row = e / ((size_t)2 * hd * n_kv);            // s*N + j
        const int s = (int)(row / N), j = (int)(row % N);
        float sum = 0.f;
        for (int g = 0; g < G; ++g)
            sum += part[((((size_t)s * n_q + kvh * G + g) * N + j) * 2 + which) * hd + d];
        dqkv[row * ld + (size_t)(n_q + (which ? n_kv : 0) + kvh) * hd + d] = sum;
    }
}

// ---- SwiGLU ------------------------------------------------------------------------------------
__global__ void silu_mul_rows_kernel(const float *gu, int inter, float *act, __half *act_h, size_t total)
{
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const size_t m = e / inter, i = e % inter;
        const float g = gu[m * 2 * inter + i], u = gu[m * 2 * inter + inter + i];
        const float v = g / (1.0f + expf(-g)) * u;
        if (act) act[e] = v;
        if (act_h) act_h[e] = __float2half_rn(v);
    }
}

__global__ void silu_mul_bwd_rows_kernel(const float *d_act, const float *gu, int inter, float *d_gu, __half *d_gu_h,
                                         float h_scale, size_t total)
{
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const size_t m = e / inter, i = e % inter;
        const float g = gu[m * 2 * inter + i], u = gu[m * 2 * inter + inter + i], dy = d_act[e];
        const float sig = 1.0f / (1.0f + expf(-g));
        const float dg = dy * u * (sig * (1.0f + g * (1.0f - sig))), du = dy * (g * sig);
        if (d_gu) { d_gu[m * 2 * inter + i] = dg; d_gu[m * 2 * inter + inter + i] = du; }
        if (d_gu_h) {
            d_gu_h[m * 2 * inter + i] = __float2half_rn(dg * h_scale);
            d_gu_h[m * 2 * inter + inter + i] = __float2half_rn(du * h_scale);
        }
    }
}

// GeGLU (Gemma3): gelu_mul / gelu_mul_backward, shaders/q8_kernels.metal:351-363, 561-580 -- the tanh form with
// its argument clamped to +-15, on the fused [rows, 2 * inter] gate|up layout.
__global__ void gelu_mul_rows_kernel(const float *gu, int inter, float *act, size_t total)
{
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const size_t m = e / inter, i = e % inter;
        const float g = gu[m * 2 * inter + i], u = gu[m * 2 * inter + inter + i];
        float inner = 0.7978845608f * (g + 0.044715f * (g * g * g));
        inner = fminf(fmaxf(inner, -15.0f), 15.0f);
        act[e] = 0.5f * g * (1.0f + tanhf(inner)) * u;
    }
}

__global__ void gelu_mul_bwd_rows_kernel(const float *d_act, const float *gu, int inter, float *d_gu, size_t total)
{
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const size_t m = e / inter, i = e % inter;
        const float g = gu[m * 2 * inter + i], u = gu[m * 2 * inter + inter + i], dy = d_act[e];
        float inner = 0.7978845608f * (g + 0.044715f * (g * g * g));
        inner = fminf(fmaxf(inner, -15.0f), 15.0f);
        const float th = tanhf(inner);
        const float gelu_g = 0.5f * g * (1.0f + th);
        const float sech2 = 1.0f - th * th;
        const float grad = 0.5f * (1.0f + th) + 0.5f * g * sech2 * 0.7978845608f * (1.0f + 3.0f * 0.044715f * g * g);
        d_gu[m * 2 * inter + i] = dy * u * grad;
        d_gu[m * 2 * inter + inter + i] = dy * gelu_g;
    }
}

// out = a + b (residual_add :369-375 with its result in a third buffer)
__global__ void add_kernel(const float *a, const float *b, float *out, size_t n)
{
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) out[i] = a[i] + b[i];
}

// ---- LoRA up-projection added into the base projection -------------------------------------------
// One thread per output column keeps its row of B in registers and walks LORA_ROWS token rows whose
// mid vectors sit in shared memory.
constexpr int LORA_ROWS = 8;
template <int MAXR>
__global__ void __launch_bounds__(256)
lora_add_kernel(float *y, long long ld, int col0, int n_cols, const float *mid, long long mid_ld, const float *B,
                int rank, float sc, int rows)
{
    __shared__ float ms[LORA_ROWS][MAXR];
    const int m0 = blockIdx.y * LORA_ROWS;
    for (int e = threadIdx.x; e < LORA_ROWS * MAXR; e += blockDim.x) {
        const int i = e / MAXR, r = e % MAXR;
        ms[i][r] = (r < rank && m0 + i < rows) ? mid[(size_t)(m0 + i) * mid_ld + r] : 0.f;   // zero beyond the rank
    }
    __syncthreads();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= n_cols) return;
    float b[MAXR];
#pragma unroll
    for (int r = 0; r < MAXR; ++r) b[r] = r < rank ? B[(size_t)c * rank + r] : 0.f;
#pragma unroll
    for (int i = 0; i < LORA_ROWS; ++i) {
        if (m0 + i >= rows) break;
        float acc = 0.f;
#pragma unroll
        for (int r = 0; r < MAXR; ++r) acc = fmaf(ms[i][r], b[r], acc);
        y[(size_t)(m0 + i) * ld + col0 + c] += sc * acc;
    }
}

// Refreshes the LoRA rows appended to the fused q/k/v weight and to its transposed copy.
//   w_ext  [qkv + xr, d]: rows qkv..qkv+R = A_q, rows qkv+R..qkv+2R = A_v
//   wt_ext [d + xr, qkv]: row d+r = sc * B_q[:, r] over the q columns, row d+R+r = sc * B_v[:, r] over the
//                         v columns, zero elsewhere
// so that the forward product also yields ln1 A^T and the backward product also yields sc * dq B_q and
// sc * dv B_v (src/nn/fast_sft.c:639-641, 948-949, 963-964) at no extra pass over the activations.
__device__ __forceinline__ void store_as(float *p, float v) { *p = v; }
__device__ __forceinline__ void store_as(__half *p, float v) { *p = __float2half_rn(v); }

template <typename T>
__global__ void lora_pack_kernel(T *w_ext, T *wt_ext, const float *A_q, const float *B_q, const float *A_v,
                                 const float *B_v, int d, int q_cols, int kv_cols, int rank, int xr, float sc)
{
    const int qkv = q_cols + 2 * kv_cols;
    const int row = blockIdx.y;                                    // 0 .. xr-1
    const int width = d > qkv ? d : qkv;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < width; c += gridDim.x * blockDim.x) {
        if (c < d) {
            float v = 0.f;
            if (row < rank) v = A_q[(size_t)row * d + c];
            else if (row < 2 * rank) v = A_v[(size_t)(row - rank) * d + c];
            store_as(w_ext + (size_t)(qkv + row) * d + c, v);
        }
        if (c < qkv) {
            float v = 0.f;
            if (row < rank) { if (c < q_cols) v = sc * B_q[(size_t)c * rank + row]; }
            else if (row < 2 * rank) { if (c >= q_cols + kv_cols) v = sc * B_v[(size_t)(c - q_cols - kv_cols) * rank + (row - rank)]; }
            store_as(wt_ext + (size_t)(d + row) * qkv + c, v);
        }
    }
}

// ---- rank-R LoRA gradients: C(p, r) = alpha * sum_m X[m, p] * Y[m, r], X wide, Y narrow (R <= MAXR) ------
// float_matmul_tn of the reference (shaders/q8_kernels.metal:1070-1094) for dB = sc * dY^T mid and
// dA = tmp^T ln1 (src/nn/fast_sft.c:946-950, 961-965). A block owns 16 columns p; its sixteen thread groups
// take every sixteenth row m and are summed in group order through shared memory, so the result does not
// depend on scheduling. A thread keeps its R sums in registers; the rows of Y are staged in shared memory
// 4096/MAXR at a time and read as broadcasts; four X loads are in flight per thread.
template <int MAXR>
__global__ void __launch_bounds__(256)
xty_skinny_kernel(const float *X, long long ld_x, const float *Y, long long ld_y, int rows, int P, int R, float alpha,
                  float *C, long long c_p, long long c_r)
{
    constexpr int CH = 4096 / MAXR;                      // rows of Y per shared-memory chunk
    constexpr int PW = 16, NG = 16;                      // columns per block, row groups per block
    static_assert(MAXR <= 16, "the cross-group buffer is sized for MAXR <= 16");
    __shared__ float ys[CH * MAXR];
    __shared__ float red[(NG - 1) * PW * (MAXR + 1)];
    const int pl = threadIdx.x % PW, mg = threadIdx.x / PW;
    const int p = blockIdx.x * PW + pl;
    const bool on = p < P;
    float acc[MAXR];
#pragma unroll
    for (int r = 0; r < MAXR; ++r) acc[r] = 0.f;
    for (int c0 = 0; c0 < rows; c0 += CH) {
        const int cn = min(CH, rows - c0);
        __syncthreads();
        for (int e = threadIdx.x; e < cn * MAXR; e += 256) {
            const int m = e / MAXR, r = e % MAXR;
            ys[e] = r < R ? Y[(size_t)(c0 + m) * ld_y + r] : 0.f;
        }
        __syncthreads();
        if (on) {
            int m = mg;
            for (; m + 3 * NG < cn; m += 4 * NG) {       // four rows of this group in flight
                const float x0 = X[(size_t)(c0 + m) * ld_x + p], x1 = X[(size_t)(c0 + m + NG) * ld_x + p];
                const float x2 = X[(size_t)(c0 + m + 2 * NG) * ld_x + p], x3 = X[(size_t)(c0 + m + 3 * NG) * ld_x + p];
#pragma unroll
                for (int r = 0; r < MAXR; ++r) {
                    acc[r] = fmaf(x0, ys[m * MAXR + r], acc[r]);
                    acc[r] = fmaf(x1, ys[(m + NG) * MAXR + r], acc[r]);
                    acc[r] = fmaf(x2, ys[(m + 2 * NG) * MAXR + r], acc[r]);
                    acc[r] = fmaf(x3, ys[(m + 3 * NG) * MAXR + r], acc[r]);
                }
            }
            for (; m < cn; m += NG) {
                const float x0 = X[(size_t)(c0 + m) * ld_x + p];
#pragma unroll
                for (int r = 0; r < MAXR; ++r) acc[r] = fmaf(x0, ys[m * MAXR + r], acc[r]);
            }
        }
    }
    if (mg > 0) {
#pragma unroll
        for (int r = 0; r < MAXR; ++r) red[((mg - 1) * PW + pl) * (MAXR + 1) + r] = acc[r];
    }
    __syncthreads();
    if (mg == 0 && on) {
#pragma unroll
        for (int r = 0; r < MAXR; ++r) {
            if (r < R) {
                float v = acc[r];
#pragma unroll
                for (int g = 0; g < NG - 1; ++g) v += red[(g * PW + pl) * (MAXR + 1) + r];
                C[(size_t)p * c_p + (size_t)r * c_r] = alpha * v;
            }
        }
    }
}

// ---- softmax cross-entropy: one block per row ----------------------------------------------------
// Two passes over the row instead of the reference's three: the first keeps a running (max, sum of
// exponentials) per thread (merged across the block in a fixed order), the second writes the gradient.
// Rows are read four values at a time when the vocabulary allows it.
__device__ __forceinline__ void lse_add(float &m, float &s, float v)
{
    if (v > m) { s = s * expf(m - v) + 1.0f; m = v; }
    else s += expf(v - m);
}

__global__ void __launch_bounds__(1024)
softmax_ce_rows_kernel(const float *logits, const uint32_t *targets, int vocab, float grad_scale, float *losses,
                       float *dlogits, __half *dlogits_h, float h_scale)
{
    __shared__ float sh_m[32], sh_s[32];
    const size_t off = (size_t)blockIdx.x * vocab;
    const float *lr = logits + off;
    uint32_t tgt = targets[blockIdx.x];
    if (tgt >= (uint32_t)vocab) tgt = 0;
    const bool vec = (vocab & 3) == 0 && ((reinterpret_cast<uintptr_t>(logits) | reinterpret_cast<uintptr_t>(dlogits)) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(dlogits_h) & 7) == 0;
    float m = -1e30f, sum = 0.f;
    if (vec) {
        const float4 *lr4 = reinterpret_cast<const float4 *>(lr);
        for (int i = threadIdx.x; i < vocab / 4; i += blockDim.x) {
            const float4 v = lr4[i];
            lse_add(m, sum, v.x); lse_add(m, sum, v.y); lse_add(m, sum, v.z); lse_add(m, sum, v.w);
        }
    } else {
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) lse_add(m, sum, lr[i]);
    }
    // merge (max, sum) pairs: lanes of a warp by shuffles, warps through shared memory in warp order
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float mo = __shfl_xor_sync(0xffffffffu, m, o), so = __shfl_xor_sync(0xffffffffu, sum, o);
        const float mn = fmaxf(m, mo);
        sum = sum * expf(m - mn) + so * expf(mo - mn);
        m = mn;
    }
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    if (l == 0) { sh_m[w] = m; sh_s[w] = sum; }
    __syncthreads();
    float M = sh_m[0];
    for (int i = 1; i < nw; ++i) M = fmaxf(M, sh_m[i]);
    float S = 0.f;
    for (int i = 0; i < nw; ++i) S += sh_s[i] * expf(sh_m[i] - M);
    const float lse = logf(S) + M;
    if (threadIdx.x == 0) losses[blockIdx.x] = lse - lr[tgt];
    float *dr = dlogits + off;
    if (vec) {
        const float4 *lr4 = reinterpret_cast<const float4 *>(lr);
        for (int i = threadIdx.x; i < vocab / 4; i += blockDim.x) {
            const float4 v = lr4[i];
            float d[4] = {expf(v.x - lse), expf(v.y - lse), expf(v.z - lse), expf(v.w - lse)};
            if ((uint32_t)i == tgt / 4) d[tgt & 3] -= 1.0f;
#pragma unroll
            for (int c = 0; c < 4; ++c) d[c] *= grad_scale;
            reinterpret_cast<float4 *>(dr)[i] = make_float4(d[0], d[1], d[2], d[3]);
            if (dlogits_h) {
                __half2 a = __floats2half2_rn(d[0] * h_scale, d[1] * h_scale), b = __floats2half2_rn(d[2] * h_scale, d[3] * h_scale);
                uint2 o;
                o.x = *reinterpret_cast<unsigned *>(&a);
                o.y = *reinterpret_cast<unsigned *>(&b);
                reinterpret_cast<uint2 *>(dlogits_h + off)[i] = o;
            }
        }
    } else {
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float p = expf(lr[i] - lse);
            const float d = (p - ((uint32_t)i == tgt ? 1.0f : 0.0f)) * grad_scale;
            dr[i] = d;
            if (dlogits_h) dlogits_h[off + i] = __float2half_rn(d * h_scale);
        }
    }
}

// ---- GRPO: PPO-clip gradient of the sampled-token log-probability w.r.t. the logits ----------------
// One block per position (grpo_policy_grad, shaders/q8_kernels.metal:698-761): log-softmax of the row,
// new_logprob = logit[action] - logsumexp, ratio = exp(new - old), the clip decides whether the position
// contributes (weight = -advantage) or not (0), dlogits = weight * ratio * (softmax - onehot(action)).
// Positions with no contribution (prompt positions carry advantage 0) are written as zeros without a
// second pass over the logits.
__global__ void __launch_bounds__(1024)
grpo_policy_grad_rows_kernel(const float *logits, const uint32_t *actions, const float *old_logprobs, const float *advantages,
                             float *new_logprobs, float *dlogits, int vocab, float clip_eps)
{
    __shared__ float sh_m[32], sh_s[32];
    const size_t off = (size_t)blockIdx.x * vocab;
    const float *lr = logits + off;
    uint32_t action = actions[blockIdx.x];
    if (action >= (uint32_t)vocab) action = 0;                     // never index outside the row
    const bool vec = (vocab & 3) == 0 && ((reinterpret_cast<uintptr_t>(logits) | reinterpret_cast<uintptr_t>(dlogits)) & 15) == 0;
    float m = -1e30f, sum = 0.f;
    if (vec) {
        const float4 *lr4 = reinterpret_cast<const float4 *>(lr);
        for (int i = threadIdx.x; i < vocab / 4; i += blockDim.x) {
            const float4 v = lr4[i];
            lse_add(m, sum, v.x); lse_add(m, sum, v.y); lse_add(m, sum, v.z); lse_add(m, sum, v.w);
        }
    } else {
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) lse_add(m, sum, lr[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float mo = __shfl_xor_sync(0xffffffffu, m, o), so = __shfl_xor_sync(0xffffffffu, sum, o);
        const float mn = fmaxf(m, mo);
        sum = sum * expf(m - mn) + so * expf(mo - mn);
        m = mn;
    }
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    if (l == 0) { sh_m[w] = m; sh_s[w] = sum; }
    __syncthreads();
    float M = sh_m[0];
    for (int i = 1; i < nw; ++i) M = fmaxf(M, sh_m[i]);
    float S = 0.f;
    for (int i = 0; i < nw; ++i) S += sh_s[i] * expf(sh_m[i] - M);
    const float lse = logf(S) + M;

    const float new_lp = lr[action] - lse;
    if (threadIdx.x == 0) new_logprobs[blockIdx.x] = new_lp;
    const float adv = advantages[blockIdx.x];
    const float ratio = expf(new_lp - old_logprobs[blockIdx.x]);
    const float clipped = fminf(fmaxf(ratio, 1.0f - clip_eps), 1.0f + clip_eps);
    const float weight = adv >= 0.f ? (ratio <= clipped ? -adv : 0.0f) : (ratio >= clipped ? -adv : 0.0f);
    const float coef = weight * ratio;

    float *dr = dlogits + off;
    if (vec) {
        const float4 *lr4 = reinterpret_cast<const float4 *>(lr);
        for (int i = threadIdx.x; i < vocab / 4; i += blockDim.x) {
            float d[4] = {0.f, 0.f, 0.f, 0.f};
            if (coef != 0.0f) {
                const float4 v = lr4[i];
                d[0] = expf(v.x - lse); d[1] = expf(v.y - lse); d[2] = expf(v.z - lse); d[3] = expf(v.w - lse);
                if ((uint32_t)i == action / 4) d[action & 3] -= 1.0f;
#pragma unroll
                for (int c = 0; c < 4; ++c) d[c] *= coef;
            }
            reinterpret_cast<float4 *>(dr)[i] = make_float4(d[0], d[1], d[2], d[3]);
        }
    } else {
        for (int i = threadIdx.x; i < vocab; i += blockDim.x)
            dr[i] = coef != 0.0f ? coef * (expf(lr[i] - lse) - ((uint32_t)i == action ? 1.0f : 0.0f)) : 0.0f;
    }
}

// f16_sgd_apply (shaders/q8_kernels.metal:1195-1206) on fp32 holders of binary16 values:
// w <- half(w - lr * g), g <- 0
__global__ void sgd_apply_f16_kernel(float *w, float *g, size_t n, float lr)
{
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        w[i] = __half2float(__float2half_rn(w[i] - lr * g[i]));
        g[i] = 0.0f;
    }
}

// x *= alpha (scale_tensor, the 1/G of the group mean in the GRPO step)
__global__ void scale_kernel(float *x, float alpha, size_t n)
{
    const size_t i0 = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4, stride = (size_t)gridDim.x * blockDim.x * 4;
    if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        for (size_t i = i0; i < n; i += stride) {
            if (i + 4 <= n) {
                float4 v = *reinterpret_cast<float4 *>(x + i);
                v.x *= alpha; v.y *= alpha; v.z *= alpha; v.w *= alpha;
                *reinterpret_cast<float4 *>(x + i) = v;
            } else {
                for (size_t j = i; j < n; ++j) x[j] *= alpha;
            }
        }
    } else {
        for (size_t i = i0; i < n; i += stride)
            for (size_t j = i; j < n && j < i + 4; ++j) x[j] *= alpha;
    }
}

// ---- frozen weights: binary16 values held as fp32, and their transposes ---------------------------
__global__ void round_f16_kernel(float *w, size_t n)
{
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        w[i] = __half2float(__float2half_rn(w[i]));
}

// dst[c, r] = src[r, c]; 32 x 32 tiles through shared memory so that both sides coalesce.
__global__ void transpose_f32_kernel(const float *src, int rows, int cols, float *dst)
{
    __shared__ float t[32][33];
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    for (int i = threadIdx.y; i < 32; i += 8) {
        const int r = r0 + i, c = c0 + threadIdx.x;
        t[i][threadIdx.x] = (r < rows && c < cols) ? src[(size_t)r * cols + c] : 0.f;
    }
    __syncthreads();
    for (int i = threadIdx.y; i < 32; i += 8) {
        const int c = c0 + i, r = r0 + threadIdx.x;
        if (c < cols && r < rows) dst[(size_t)c * rows + r] = t[threadIdx.x][i];
    }
}

// ---- binary16 operand copies for the tensor-core products --------------------------------------------
// dst = half(src * scale), four elements per thread (n a multiple of 4 is the fast path).
__global__ void f32_to_f16_kernel(const float *src, size_t n, float scale, __half *dst)
{
    const size_t n4 = n / 4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const float4 v = reinterpret_cast<const float4 *>(src)[i];
        __half2 a = __floats2half2_rn(v.x * scale, v.y * scale), b = __floats2half2_rn(v.z * scale, v.w * scale);
        uint2 o;
        o.x = *reinterpret_cast<unsigned *>(&a);
        o.y = *reinterpret_cast<unsigned *>(&b);
        reinterpret_cast<uint2 *>(dst)[i] = o;
    }
    if (blockIdx.x == 0 && threadIdx.x < (n & 3)) dst[n4 * 4 + threadIdx.x] = __float2half_rn(src[n4 * 4 + threadIdx.x] * scale);
}

__global__ void transpose_f16_kernel(const __half *src, int rows, int cols, __half *dst)
{
    __shared__ __half t[32][34];
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    for (int i = threadIdx.y; i < 32; i += 8) {
        const int r = r0 + i, c = c0 + threadIdx.x;
        t[i][threadIdx.x] = (r < rows && c < cols) ? src[(size_t)r * cols + c] : __float2half(0.f);
    }
    __syncthreads();
    for (int i = threadIdx.y; i < 32; i += 8) {
        const int c = c0 + i, r = r0 + threadIdx.x;
        if (c < cols && r < rows) dst[(size_t)c * rows + r] = t[threadIdx.x][i];
    }
}

// ---- gradient norm, clip, AdamW ------------------------------------------------------------------
__global__ void __launch_bounds__(256) sumsq_partials_kernel(const float *g, size_t n, double *partials)
{
    __shared__ double sh[8];
    double acc = 0.0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const double v = (double)g[i];
        acc += v * v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int i = 0; i < 8; ++i) t += sh[i];
        partials[blockIdx.x] = t;
    }
}

__global__ void __launch_bounds__(256)
clip_adamw_kernel(float *p, float *g, float *m, float *v, size_t n, const double *partials, int n_partials,
                  float max_norm, float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                  int apply_update, float *norm_out)
{
    __shared__ float s_scale;
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int i = 0; i < n_partials; ++i) t += partials[i];          // same order in every block
        const float norm = (float)sqrt(t);
        s_scale = norm > max_norm ? max_norm / norm : 1.0f;
        if (blockIdx.x == 0 && norm_out) norm_out[0] = norm;
    }
    __syncthreads();
    const float scale = s_scale;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float gr = g[i];
        if (scale != 1.0f) { gr *= scale; g[i] = gr; }
        if (apply_update) {
            const float mi = beta1 * m[i] + (1.0f - beta1) * gr;
            const float vi = beta2 * v[i] + (1.0f - beta2) * gr * gr;
            m[i] = mi;
            v[i] = vi;
            const float pi = p[i];
            p[i] = pi - lr * ((mi / bc1) / (sqrtf(vi / bc2) + eps) + wd * pi);
        }
    }
}

inline int done()
{
    ++g_b200_launches;
    return (int)cudaGetLastError();
}

template <typename K>
int opt_in_smem(K kern, size_t bytes)
{
    if (bytes <= 48 * 1024) return 0;
    if (bytes > 200 * 1024) return B200_E_TOOLARGE;
    return (int)cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

}  // namespace

// ================================== C ABI =========================================================

extern "C" int b200_round_f16(float *w, size_t n, void *stream)
{
    if (!w || n == 0) return B200_E_BADARG;
    const unsigned grid = (unsigned)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    round_f16_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(w, n);
    return done();
}

extern "C" int b200_transpose_f32(const float *src, int rows, int cols, float *dst, void *stream)
{
    if (!src || !dst || rows <= 0 || cols <= 0 || (rows + 31) / 32 > 65535) return B200_E_BADARG;
    dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
    transpose_f32_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(src, rows, cols, dst);
    return done();
}

extern "C" int b200_embed_rows(const float *emb, const uint32_t *tokens, int rows, int dim, int vocab, float scale,
                               float *x, void *stream)
{
    if (!emb || !tokens || !x || rows <= 0 || dim <= 0 || vocab <= 0) return B200_E_BADARG;
    embed_rows_kernel<<<rows, 256, 0, (cudaStream_t)stream>>>(emb, tokens, dim, vocab, scale, x);
    return done();
}

extern "C" int b200_rms_norm_rows_h(const float *x, const float *gamma, float *out, void *out_h, int rows, int dim,
                                    float eps, void *stream)
{
    if (!x || !gamma || !out || rows <= 0 || dim <= 0) return B200_E_BADARG;
    cudaStream_t st = (cudaStream_t)stream;
    __half *oh = static_cast<__half *>(out_h);
    if (dim >= 1024) rms_norm_rows_kernel<256><<<rows, 256, 0, st>>>(x, gamma, out, oh, rows, dim, eps);
    else rms_norm_rows_kernel<32><<<(rows + 7) / 8, 256, 0, st>>>(x, gamma, out, oh, rows, dim, eps);
    return done();
}

extern "C" int b200_rms_norm_rows(const float *x, const float *gamma, float *out, int rows, int dim, float eps,
                                  void *stream)
{
    return b200_rms_norm_rows_h(x, gamma, out, nullptr, rows, dim, eps, stream);
}

extern "C" int b200_rms_norm_bwd_rows_h(const float *x, const float *dy, long long dy_ld, const float *gamma, float *dx,
                                        int rows, int dim, float eps, int accumulate, float clamp, void *dx_h,
                                        float h_scale, void *stream)
{
    if (!x || !dy || !gamma || !dx || rows <= 0 || dim <= 0 || dy_ld < dim) return B200_E_BADARG;
    cudaStream_t st = (cudaStream_t)stream;
    __half *dh = static_cast<__half *>(dx_h);
    if (dim >= 1024)
        rms_norm_bwd_rows_kernel<256><<<rows, 256, 0, st>>>(x, dy, dy_ld, gamma, dx, rows, dim, eps, accumulate, clamp, dh,
                                                            h_scale);
    else
        rms_norm_bwd_rows_kernel<32><<<(rows + 7) / 8, 256, 0, st>>>(x, dy, dy_ld, gamma, dx, rows, dim, eps, accumulate,
                                                                    clamp, dh, h_scale);
    return done();
}

extern "C" int b200_rms_norm_bwd_rows(const float *x, const float *dy, long long dy_ld, const float *gamma, float *dx,
                                      int rows, int dim, float eps, int accumulate, float clamp, void *stream)
{
    return b200_rms_norm_bwd_rows_h(x, dy, dy_ld, gamma, dx, rows, dim, eps, accumulate, clamp, nullptr, 1.0f, stream);
}

extern "C" int b200_qk_norm_rope(const float *qkv, long long ld, const float *q_gamma, const float *k_gamma,
                                 const float *inv_freq, int rows, int seq_len, int n_q, int n_kv, int hd, float eps,
                                 float *q_out, float *k_out, void *stream)
{
    if (!qkv || !q_gamma || !k_gamma || !inv_freq || !q_out || !k_out || rows <= 0 || seq_len <= 0) return B200_E_BADARG;
    const long long units = (long long)rows * (n_q + n_kv);
    const unsigned grid = (unsigned)((units + 7) / 8);
    cudaStream_t st = (cudaStream_t)stream;
    switch (hd) {
    case 64: qk_norm_rope_kernel<64><<<grid, 256, 0, st>>>(qkv, ld, q_gamma, k_gamma, inv_freq, rows, seq_len, n_q, n_kv, eps, q_out, k_out); break;
    case 128: qk_norm_rope_kernel<128><<<grid, 256, 0, st>>>(qkv, ld, q_gamma, k_gamma, inv_freq, rows, seq_len, n_q, n_kv, eps, q_out, k_out); break;
    case 256: qk_norm_rope_kernel<256><<<grid, 256, 0, st>>>(qkv, ld, q_gamma, k_gamma, inv_freq, rows, seq_len, n_q, n_kv, eps, q_out, k_out); break;
    default: return B200_E_BADARG;
    }
    return done();
}

extern "C" int b200_qk_norm_rope_bwd(float *dqkv, const float *qkv, long long ld, long long dld, const float *q_gamma,
                                     const float *k_gamma, const float *inv_freq, int rows, int seq_len, int n_q,
                                     int n_kv, int hd, float eps, void *stream)
{
    if (!dqkv || !qkv || !q_gamma || !k_gamma || !inv_freq || rows <= 0 || seq_len <= 0) return B200_E_BADARG;
    const long long units = (long long)rows * (n_q + n_kv);
    const unsigned grid = (unsigned)((units + 7) / 8);
    cudaStream_t st = (cudaStream_t)stream;
    switch (hd) {
    case 64: qk_norm_rope_bwd_kernel<64><<<grid, 256, 0, st>>>(dqkv, qkv, ld, dld, q_gamma, k_gamma, inv_freq, rows, seq_len, n_q, n_kv, eps); break;
    case 128: qk_norm_rope_bwd_kernel<128><<<grid, 256, 0, st>>>(dqkv, qkv, ld, dld, q_gamma, k_gamma, inv_freq, rows, seq_len, n_q, n_kv, eps); break;
    case 256: qk_norm_rope_bwd_kernel<256><<<grid, 256, 0, st>>>(dqkv, qkv, ld, dld, q_gamma, k_gamma, inv_freq, rows, seq_len, n_q, n_kv, eps); break;
    default: return B200_E_BADARG;
    }
    return done();
}

static bool attn_shape_ok(int n_seq, int seq_len, int n_q, int n_kv, int hd)
{
    return n_seq > 0 && seq_len > 0 && n_q > 0 && n_kv > 0 && n_q % n_kv == 0 && (hd == 64 || hd == 128 || hd == 256);
}

template <int HD>
static int attn_fwd_launch(const float *q, const float *k, const float *v, long long v_ld, int n_seq, int N, int n_q,
                           int n_kv, float scale, float *probs, float *out, __half *out_h, cudaStream_t st)
{
    if constexpr (HD <= 128) if (N <= AT) {                   // short sequences: one block per (sequence, head)
        const size_t tsm = ((size_t)2 * HD * ATP + (size_t)AT * ATP) * sizeof(float);
        int rc = opt_in_smem(attn_fwd_tile_kernel<HD>, tsm);
        if (rc) return rc;
        attn_fwd_tile_kernel<HD><<<n_seq * n_q, 256, tsm, st>>>(q, k, v, v_ld, N, n_q, n_kv, scale, probs, out, out_h);
        return done();
    }
    const size_t smem = (size_t)ATT_WARPS * (HD + N) * sizeof(float);
    int rc = opt_in_smem(attn_train_fwd_kernel<HD>, smem);
    if (rc) return rc;
    const long long units = (long long)n_seq * n_q * N;
    attn_train_fwd_kernel<HD><<<(unsigned)((units + ATT_WARPS - 1) / ATT_WARPS), ATT_WARPS * 32, smem, st>>>(
        q, k, v, v_ld, n_seq, N, n_q, n_kv, scale, probs, out, out_h);
    return done();
}

extern "C" int b200_attn_train_fwd_h(const float *q, const float *k, const float *v, long long v_ld, int n_seq,
                                     int seq_len, int n_q, int n_kv, int hd, float scale, float *probs, float *out,
                                     void *out_h, void *stream)
{
    if (!q || !k || !v || !probs || (!out && !out_h) || !attn_shape_ok(n_seq, seq_len, n_q, n_kv, hd)) return B200_E_BADARG;
    if ((v_ld & 3) || ((uintptr_t)v & 15) || ((uintptr_t)k & 15)) return B200_E_BADARG;     // 16-byte row loads
    cudaStream_t st = (cudaStream_t)stream;
    __half *oh = static_cast<__half *>(out_h);
    if (hd == 64) return attn_fwd_launch<64>(q, k, v, v_ld, n_seq, seq_len, n_q, n_kv, scale, probs, out, oh, st);
    if (hd == 128) return attn_fwd_launch<128>(q, k, v, v_ld, n_seq, seq_len, n_q, n_kv, scale, probs, out, oh, st);
    return attn_fwd_launch<256>(q, k, v, v_ld, n_seq, seq_len, n_q, n_kv, scale, probs, out, oh, st);
}

extern "C" int b200_attn_train_fwd(const float *q, const float *k, const float *v, long long v_ld, int n_seq,
                                   int seq_len, int n_q, int n_kv, int hd, float scale, float *probs, float *out,
                                   void *stream)
{
    if (!out) return B200_E_BADARG;
    return b200_attn_train_fwd_h(q, k, v, v_ld, n_seq, seq_len, n_q, n_kv, hd, scale, probs, out, nullptr, stream);
}

template <int HD>
static int attn_bwd_launch(const float *d_out, const float *probs, const float *q, const float *k, const float *v,
                           long long v_ld, int n_seq, int N, int n_q, int n_kv, float scale, float *d_score,
                           float *dqkv, long long ld, cudaStream_t st)
{
    if constexpr (HD <= 128) if (N <= AT) {
        // d_score is used as the per-head dK/dV scratch [S][n_q][N][2][HD] here
        const size_t tsm = ((size_t)2 * HD * ATP + (size_t)2 * AT * ATP) * sizeof(float);
        int rc = opt_in_smem(attn_bwd_tile_kernel<HD>, tsm);
        if (rc) return rc;
        attn_bwd_tile_kernel<HD><<<n_seq * n_q, 256, tsm, st>>>(d_out, probs, q, k, v, v_ld, N, n_q, n_kv, scale, dqkv, ld,
                                                                d_score);
        rc = done();
        if (rc) return rc;
        const size_t total = (size_t)n_seq * N * n_kv * 2 * HD;
        const unsigned grid = (unsigned)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
        attn_bwd_reduce_kernel<<<grid, 256, 0, st>>>(d_score, n_seq, N, n_q, n_kv, HD, dqkv, ld);
        return done();
    }
    const size_t smem = (size_t)ATT_WARPS * (HD + N) * sizeof(float);
    int rc = opt_in_smem(attn_bwd_dq_kernel<HD>, smem);
    if (rc) return rc;
    const long long uq = (long long)n_seq * n_q * N, uk = (long long)n_seq * n_kv * N;
    attn_bwd_dq_kernel<HD><<<(unsigned)((uq + ATT_WARPS - 1) / ATT_WARPS), ATT_WARPS * 32, smem, st>>>(
        d_out, probs, k, v, v_ld, n_seq, N, n_q, n_kv, scale, d_score, dqkv, ld);
    rc = done();
    if (rc) return rc;
    attn_bwd_dkv_kernel<HD><<<(unsigned)((uk + ATT_WARPS - 1) / ATT_WARPS), ATT_WARPS * 32, 0, st>>>(
        d_score, probs, q, d_out, n_seq, N, n_q, n_kv, dqkv, ld);
    return done();
}

extern "C" int b200_attn_train_bwd(const float *d_out, const float *probs, const float *q, const float *k,
                                   const float *v, long long v_ld, int n_seq, int seq_len, int n_q, int n_kv, int hd,
                                   float scale, float *d_score, float *dqkv, long long ld, void *stream)
{
    if (!d_out || !probs || !q || !k || !v || !d_score || !dqkv || !attn_shape_ok(n_seq, seq_len, n_q, n_kv, hd))
        return B200_E_BADARG;
    if ((v_ld & 3) || ((uintptr_t)v & 15)) return B200_E_BADARG;
    cudaStream_t st = (cudaStream_t)stream;
    if (hd == 64) return attn_bwd_launch<64>(d_out, probs, q, k, v, v_ld, n_seq, seq_len, n_q, n_kv, scale, d_score, dqkv, ld, st);
    if (hd == 128) return attn_bwd_launch<128>(d_out, probs, q, k, v, v_ld, n_seq, seq_len, n_q, n_kv, scale, d_score, dqkv, ld, st);
    return attn_bwd_launch<256>(d_out, probs, q, k, v, v_ld, n_seq, seq_len, n_q, n_kv, scale, d_score, dqkv, ld, st);
}

extern "C" int b200_silu_mul_rows_h(const float *gu, int rows, int inter, float *act, void *act_h, void *stream)
{
    if (!gu || (!act && !act_h) || rows <= 0 || inter <= 0) return B200_E_BADARG;
    const size_t total = (size_t)rows * inter;
    const unsigned grid = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    silu_mul_rows_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(gu, inter, act, static_cast<__half *>(act_h), total);
    return done();
}

extern "C" int b200_silu_mul_rows(const float *gu, int rows, int inter, float *act, void *stream)
{
    if (!act) return B200_E_BADARG;
    return b200_silu_mul_rows_h(gu, rows, inter, act, nullptr, stream);
}

extern "C" int b200_silu_mul_bwd_rows_h(const float *d_act, const float *gu, int rows, int inter, float *d_gu, void *d_gu_h,
                                        float h_scale, void *stream)
{
    if (!d_act || !gu || (!d_gu && !d_gu_h) || rows <= 0 || inter <= 0) return B200_E_BADARG;
    const size_t total = (size_t)rows * inter;
    const unsigned grid = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    silu_mul_bwd_rows_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(d_act, gu, inter, d_gu, static_cast<__half *>(d_gu_h),
                                                                    h_scale, total);
    return done();
}

extern "C" int b200_silu_mul_bwd_rows(const float *d_act, const float *gu, int rows, int inter, float *d_gu,
                                      void *stream)
{
    if (!d_gu) return B200_E_BADARG;
    return b200_silu_mul_bwd_rows_h(d_act, gu, rows, inter, d_gu, nullptr, 1.0f, stream);
}

extern "C" int b200_gelu_mul_rows(const float *gu, int rows, int inter, float *act, void *stream)
{
    if (!gu || !act || rows <= 0 || inter <= 0) return B200_E_BADARG;
    const size_t total = (size_t)rows * inter;
    const unsigned grid = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    gelu_mul_rows_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(gu, inter, act, total);
    return done();
}

extern "C" int b200_gelu_mul_bwd_rows(const float *d_act, const float *gu, int rows, int inter, float *d_gu, void *stream)
{
    if (!d_act || !gu || !d_gu || rows <= 0 || inter <= 0) return B200_E_BADARG;
    const size_t total = (size_t)rows * inter;
    const unsigned grid = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    gelu_mul_bwd_rows_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(d_act, gu, inter, d_gu, total);
    return done();
}

extern "C" int b200_add(const float *a, const float *b, float *out, size_t n, void *stream)
{
    if (!a || !b || !out) return B200_E_BADARG;
    if (n == 0) return 0;
    const unsigned grid = (unsigned)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    add_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(a, b, out, n);
    return done();
}

extern "C" int b200_lora_add(float *y, long long ld, int col0, int n_cols, const float *mid, long long mid_ld,
                             const float *B, int rank, float sc, int rows, void *stream)
{
    if (!y || !mid || !B || rank <= 0 || rank > 64 || rows <= 0 || n_cols <= 0 || mid_ld < rank) return B200_E_BADARG;
    if ((rows + LORA_ROWS - 1) / LORA_ROWS > 65535) return B200_E_TOOLARGE;
    dim3 grid((n_cols + 255) / 256, (rows + LORA_ROWS - 1) / LORA_ROWS);
    cudaStream_t st = (cudaStream_t)stream;
    if (rank <= 16) lora_add_kernel<16><<<grid, 256, 0, st>>>(y, ld, col0, n_cols, mid, mid_ld, B, rank, sc, rows);
    else lora_add_kernel<64><<<grid, 256, 0, st>>>(y, ld, col0, n_cols, mid, mid_ld, B, rank, sc, rows);
    return done();
}

extern "C" int b200_lora_pack(float *w_ext, float *wt_ext, const float *A_q, const float *B_q, const float *A_v,
                              const float *B_v, int d, int q_cols, int kv_cols, int rank, int xr, float sc, void *stream)
{
    if (!w_ext || !wt_ext || !A_q || !B_q || !A_v || !B_v || d <= 0 || q_cols <= 0 || kv_cols <= 0 || rank <= 0 ||
        xr < 2 * rank)
        return B200_E_BADARG;
    const int width = d > q_cols + 2 * kv_cols ? d : q_cols + 2 * kv_cols;
    dim3 grid((width + 255) / 256, xr);
    lora_pack_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>(w_ext, wt_ext, A_q, B_q, A_v, B_v, d, q_cols, kv_cols,
                                                                   rank, xr, sc);
    return done();
}

extern "C" int b200_lora_pack_f16(void *w_ext, void *wt_ext, const float *A_q, const float *B_q, const float *A_v,
                                  const float *B_v, int d, int q_cols, int kv_cols, int rank, int xr, float sc,
                                  void *stream)
{
    if (!w_ext || !wt_ext || !A_q || !B_q || !A_v || !B_v || d <= 0 || q_cols <= 0 || kv_cols <= 0 || rank <= 0 ||
        xr < 2 * rank)
        return B200_E_BADARG;
    const int width = d > q_cols + 2 * kv_cols ? d : q_cols + 2 * kv_cols;
    dim3 grid((width + 255) / 256, xr);
    lora_pack_kernel<__half><<<grid, 256, 0, (cudaStream_t)stream>>>(static_cast<__half *>(w_ext), static_cast<__half *>(wt_ext),
                                                                    A_q, B_q, A_v, B_v, d, q_cols, kv_cols, rank, xr, sc);
    return done();
}

extern "C" int b200_f32_to_f16(const float *src, size_t n, float scale, void *dst, void *stream)
{
    if (!src || !dst || n == 0 || ((uintptr_t)src & 15) || ((uintptr_t)dst & 7)) return B200_E_BADARG;
    const size_t n4 = (n + 3) / 4;
    const unsigned grid = (unsigned)((n4 + 255) / 256 < 148 * 16 ? (n4 + 255) / 256 : 148 * 16);
    f32_to_f16_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(src, n, scale, static_cast<__half *>(dst));
    return done();
}

extern "C" int b200_transpose_f16(const void *src, int rows, int cols, void *dst, void *stream)
{
    if (!src || !dst || rows <= 0 || cols <= 0 || (rows + 31) / 32 > 65535) return B200_E_BADARG;
    dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
    transpose_f16_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(static_cast<const __half *>(src), rows, cols,
                                                                  static_cast<__half *>(dst));
    return done();
}

extern "C" int b200_xty_skinny(const float *X, long long ld_x, const float *Y, long long ld_y, int rows, int P, int R,
                               float alpha, float *C, long long c_p, long long c_r, void *stream)
{
    if (!X || !Y || !C || rows <= 0 || P <= 0 || R <= 0 || ld_x < P || ld_y < R) return B200_E_BADARG;
    if (R > 16) return B200_E_UNSUPPORTED;               // wider ranks go through b200_gemm_f32
    xty_skinny_kernel<16><<<(unsigned)((P + 15) / 16), 256, 0, (cudaStream_t)stream>>>(X, ld_x, Y, ld_y, rows, P, R, alpha,
                                                                                        C, c_p, c_r);
    return done();
}

extern "C" int b200_softmax_ce_rows_h(const float *logits, const uint32_t *targets, int rows, int vocab,
                                      float grad_scale, float *losses, float *dlogits, void *dlogits_h, float h_scale,
                                      void *stream)
{
    if (!logits || !targets || !losses || !dlogits || rows <= 0 || vocab <= 0) return B200_E_BADARG;
    softmax_ce_rows_kernel<<<rows, 1024, 0, (cudaStream_t)stream>>>(logits, targets, vocab, grad_scale, losses, dlogits,
                                                                   static_cast<__half *>(dlogits_h), h_scale);
    return done();
}

extern "C" int b200_softmax_ce_rows(const float *logits, const uint32_t *targets, int rows, int vocab,
                                    float grad_scale, float *losses, float *dlogits, void *stream)
{
    return b200_softmax_ce_rows_h(logits, targets, rows, vocab, grad_scale, losses, dlogits, nullptr, 1.0f, stream);
}

extern "C" int b200_grpo_policy_grad(const float *logits, const uint32_t *actions, const float *old_logprobs,
                                     const float *advantages, float *new_logprobs, float *dlogits, int rows, int vocab,
                                     float clip_eps, void *stream)
{
    if (!logits || !actions || !old_logprobs || !advantages || !new_logprobs || !dlogits || rows <= 0 || vocab <= 0)
        return B200_E_BADARG;
    grpo_policy_grad_rows_kernel<<<rows, 1024, 0, (cudaStream_t)stream>>>(logits, actions, old_logprobs, advantages,
                                                                         new_logprobs, dlogits, vocab, clip_eps);
    return done();
}

extern "C" int b200_sgd_apply_f16(float *w, float *g, size_t n, float lr, void *stream)
{
    if (!w || !g) return B200_E_BADARG;
    if (n == 0) return 0;
    const size_t want = (n + 255) / 256;
    const unsigned grid = (unsigned)(want < 148 * 8 ? want : 148 * 8);
    sgd_apply_f16_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(w, g, n, lr);
    return done();
}

extern "C" int b200_scale(float *x, float alpha, size_t n, void *stream)
{
    if (!x) return B200_E_BADARG;
    if (n == 0) return 0;
    const size_t want = (n / 4 + 255) / 256;
    const unsigned grid = (unsigned)(want < 148 * 8 ? (want ? want : 1) : 148 * 8);
    scale_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(x, alpha, n);
    return done();
}

extern "C" int b200_sumsq_partials(const float *g, size_t n, double *partials, int n_partials, void *stream)
{
    if (!g || !partials || n == 0 || n_partials <= 0 || n_partials > 4096) return B200_E_BADARG;
    sumsq_partials_kernel<<<n_partials, 256, 0, (cudaStream_t)stream>>>(g, n, partials);
    return done();
}

extern "C" int b200_clip_adamw(float *p, float *g, float *m, float *v, size_t n, const double *partials,
                               int n_partials, float max_norm, float lr, float beta1, float beta2, float eps, float wd,
                               float bc1, float bc2, int apply_update, float *norm_out, void *stream)
{
    if (!g || !partials || n == 0 || n_partials <= 0) return B200_E_BADARG;
    if (apply_update && (!p || !m || !v)) return B200_E_BADARG;
    const unsigned grid = (unsigned)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
    clip_adamw_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(p, g, m, v, n, partials, n_partials, max_norm, lr, beta1,
                                                             beta2, eps, wd, bc1, bc2, apply_update, norm_out);
    return done();
}
