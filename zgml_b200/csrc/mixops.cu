// Sequence-model DeviceOps ZG_OP_TOKEN_SHIFT .. ZG_OP_POLY_NORM (parameter packs in include/zgml_cuda.h): the pieces of
// decoder stacks whose mixers attend over a per-sequence CACHE of keys and values (or of one latent that serves as both) —
// token shift, a learned average over the depth of the stack, rotary positions, the cache append, softmax attention over
// the cache with grouped heads / several score maps per head / causal, sliding and block masks, the differential
// combination of two maps, sigmoid gates, block-diagonal (per-head) products and the PolyNorm activation.
// Everything here is f32: positions and angles, scores and softmax weights, norms, gates and the sums.
#include "seq_common.cuh"

#include <math.h>

namespace {

// ── TOKEN_SHIFT ──────────────────────────────────────────────────────────────────────────────────────────────────
// Thread (0, c) alone touches state[c]: it reads the previous step's last row there and then replaces it.
template <typename WT>
__global__ void k_token_shift(float* __restrict__ dst, const float* __restrict__ src, const WT* __restrict__ mix, float* __restrict__ state,
                              const float* __restrict__ ctl, uint32_t T, uint32_t D) {
    pdl_enter();
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= (size_t)T * D) return;
    const uint32_t t = (uint32_t)(e / D), c = (uint32_t)(e % D);
    float* st = state + (size_t)ctl_word(ctl, ZG_CTL_SLOT) * D;
    const float h = src[e];
    const float prev = t ? src[e - D] : st[c];
    dst[e] = fmaf(prev - h, wld(mix, c), h);
    if (t == 0) st[c] = src[(size_t)(T - 1) * D + c];
}

// ── DEPTH_MIX ────────────────────────────────────────────────────────────────────────────────────────────────────
template <typename WT>
__global__ void k_depth_mix(float* __restrict__ dst, const float* __restrict__ hist, const WT* __restrict__ coeff, uint32_t n, uint32_t terms,
                            uint32_t stride) {
    pdl_enter();
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n) return;
    float acc = 0.0f;
    for (uint32_t j = 0; j < terms; j++) acc = fmaf(wld(coeff, j), hist[(size_t)j * stride + e], acc);
    dst[e] = acc;
}

// ── ROTARY ───────────────────────────────────────────────────────────────────────────────────────────────────────
// The frequency is the f32 rounding of base^(-2i / dims); the angle p * f and its sine and cosine are f32.
__device__ __forceinline__ void rotary_angle(uint32_t pos, uint32_t i, uint32_t dims, float base, float& sn, float& cs) {
    const float freq = (float)pow((double)base, -2.0 * (double)i / (double)dims);
    sincosf((float)pos * freq, &sn, &cs);
}
__global__ void k_rotary(float* x, const float* src, const float* __restrict__ ctl, uint32_t T, uint32_t heads, uint32_t head_stride,
                         uint32_t row_stride, uint32_t dims, uint32_t layout, uint32_t src_hs, uint32_t src_rs, float base) {
    pdl_enter();
    const uint32_t half = dims / 2;
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= (size_t)T * heads * half) return;
    const uint32_t i = (uint32_t)(e % half), hd = (uint32_t)((e / half) % heads), t = (uint32_t)(e / ((size_t)half * heads));
    float sn, cs;
    rotary_angle((uint32_t)ctl_word(ctl, ZG_CTL_POS) + t, i, dims, base, sn, cs);
    float* v = x + (size_t)t * row_stride + (size_t)hd * head_stride;
    const float* sv = src + (size_t)t * src_rs + (size_t)hd * src_hs;
    const uint32_t a = layout == 0 ? 2 * i : i, b = layout == 0 ? 2 * i + 1 : i + half;
    const float u = sv[a], w = sv[b];
    v[a] = u * cs - w * sn;
    v[b] = w * cs + u * sn;
}

// ── CACHE_APPEND: one CTA per token ──────────────────────────────────────────────────────────────────────────────
// A cache row is [normed | rotated | plain]: the first `normed` columns are divided by their root mean square and weighted
// (a latent), the next `rot` columns get the token's rotary position (a key part shared by the heads), the rest is copied.
template <typename WT>
__global__ void k_cache_append(float* __restrict__ cache, const float* __restrict__ src, const float* __restrict__ ctl, const WT* __restrict__ nw,
                               uint32_t cols, uint32_t src_rs, uint32_t width, uint32_t R, uint32_t normed, uint32_t rot, uint32_t layout, float eps,
                               float base) {
    pdl_enter();
    __shared__ float sh[32];
    const uint32_t t = blockIdx.x;
    const uint32_t pos = (uint32_t)ctl_word(ctl, ZG_CTL_POS) + t, slot = (uint32_t)ctl_word(ctl, ZG_CTL_SLOT);
    float* row = cache + ((size_t)slot * R + pos % R) * width;
    const float* s = src + (size_t)t * src_rs;
    if (normed) {
        float q = 0.0f;
        for (uint32_t c = threadIdx.x; c < normed; c += blockDim.x) q = fmaf(s[c], s[c], q);
        const float inv = 1.0f / sqrtf(block_sum(q, sh) / (float)normed + eps);
        for (uint32_t c = threadIdx.x; c < normed; c += blockDim.x) row[c] = s[c] * inv * wld(nw, c);
    }
    const uint32_t half = rot / 2;
    for (uint32_t i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        rotary_angle(pos, i, rot, base, sn, cs);
        const uint32_t a = normed + (layout == 0 ? 2 * i : i), b = normed + (layout == 0 ? 2 * i + 1 : i + half);
        const float u = s[a], w = s[b];
        row[a] = u * cs - w * sn;
        row[b] = w * cs + u * sn;
    }
    for (uint32_t c = normed + rot + threadIdx.x; c < cols; c += blockDim.x) row[c] = s[c];
}

// ── CACHED_ATTENTION ─────────────────────────────────────────────────────────────────────────────────────────────
// first position a query at p can see
__device__ __forceinline__ uint32_t mask_low(uint32_t p, uint32_t kind, uint32_t size) {
    if (kind == 1) return p + 1 >= size ? p + 1 - size : 0;
    if (kind == 2) return p - p % size;
    return 0;
}
struct CaArgs {
    float* dst; const float* q; const float* kc; const float* vc; const float* ctl;
    uint32_t T, H, G, maps, dk, dv, q_rs, q_off, kw, k_off, vw, v_off, R, kind, size;
    float scale;
};
constexpr int kCaMaxDv = 1024;   // 32 channels per lane in the per-query kernel
// Any shape: one warp per (token, head, map); 32 keys at a time, lane = key for the scores, lane = channel for the sum.
__global__ void k_cached_attention(CaArgs a) {
    pdl_enter();
    extern __shared__ float sq[];                      // [warps][dk]
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const uint32_t HM = a.H * a.maps;
    const uint32_t item = blockIdx.x * nw + warp;
    if (item >= a.T * HM) return;
    const uint32_t t = item / HM, hm = item % HM, h = hm / a.maps, m = hm % a.maps, g = h / (a.H / a.G);
    const uint32_t pos0 = (uint32_t)ctl_word(a.ctl, ZG_CTL_POS), slot = (uint32_t)ctl_word(a.ctl, ZG_CTL_SLOT);
    const uint32_t p = pos0 + t, lo = mask_low(p, a.kind, a.size);
    float* q = sq + warp * a.dk;
    const float* qrow = a.q + (size_t)t * a.q_rs + a.q_off + (size_t)hm * a.dk;
    for (uint32_t c = lane; c < a.dk; c += 32) q[c] = qrow[c];
    __syncwarp();
    const float* kbase = a.kc + (size_t)slot * a.R * a.kw + a.k_off + (size_t)(g * a.maps + m) * a.dk;
    const float* vbase = a.vc + (size_t)slot * a.R * a.vw + a.v_off + (size_t)g * a.dv;
    float mx = -INFINITY, l = 0.0f;
    float acc[kCaMaxDv / 32];
#pragma unroll
    for (int i = 0; i < kCaMaxDv / 32; i++) acc[i] = 0.0f;
    for (uint32_t j0 = lo; j0 <= p; j0 += 32) {
        const uint32_t j = j0 + lane;
        float s = -INFINITY;
        if (j <= p) {
            const float* k = kbase + (size_t)(j % a.R) * a.kw;
            float d = 0.0f;
            for (uint32_t c = 0; c < a.dk; c++) d = fmaf(q[c], k[c], d);
            s = d * a.scale;
        }
        const float m_new = fmaxf(mx, warp_max(s));    // finite: key j0 is visible
        const float corr = expf(mx - m_new);
        const float e = j <= p ? expf(s - m_new) : 0.0f;
        l = l * corr + warp_sum(e);
        mx = m_new;
        const uint32_t cnt = min(32u, p - j0 + 1);
#pragma unroll
        for (int i = 0; i < kCaMaxDv / 32; i++) acc[i] *= corr;
        for (uint32_t jj = 0; jj < cnt; jj++) {
            const float pj = __shfl_sync(0xffffffffu, e, jj);
            const float* v = vbase + (size_t)((j0 + jj) % a.R) * a.vw;
#pragma unroll
            for (int i = 0; i < kCaMaxDv / 32; i++) {
                const uint32_t c = lane + 32 * i;
                if (c < a.dv) acc[i] = fmaf(pj, v[c], acc[i]);
            }
        }
    }
    const float inv = 1.0f / l;
    float* out = a.dst + ((size_t)t * HM + hm) * a.dv;
#pragma unroll
    for (int i = 0; i < kCaMaxDv / 32; i++) {
        const uint32_t c = lane + 32 * i;
        if (c < a.dv) out[c] = acc[i] * inv;
    }
}

// ── MAP_COMBINE: one warp per (token, head) ──────────────────────────────────────────────────────────────────────
__global__ void k_map_combine(float* __restrict__ dst, const float* __restrict__ src, uint32_t rows, uint32_t dv, float lambda, float eps, float out_scale) {
    pdl_enter();
    const uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* a1 = src + (size_t)row * 2 * dv;
    const float* a2 = a1 + dv;
    float q = 0.0f;
    for (uint32_t c = lane; c < dv; c += 32) { const float o = fmaf(-lambda, a2[c], a1[c]); q = fmaf(o, o, q); }
    const float inv = out_scale / sqrtf(warp_sum(q) / (float)dv + eps);
    for (uint32_t c = lane; c < dv; c += 32) dst[(size_t)row * dv + c] = fmaf(-lambda, a2[c], a1[c]) * inv;
}

// ── GATE ─────────────────────────────────────────────────────────────────────────────────────────────────────────
__global__ void k_gate(float* __restrict__ dst, const float* __restrict__ gate, uint32_t T, uint32_t cols, uint32_t group, uint32_t gate_rs,
                       uint32_t gate_off, uint32_t dst_rs) {
    pdl_enter();
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= (size_t)T * cols) return;
    const uint32_t t = (uint32_t)(e / cols), c = (uint32_t)(e % cols);
    dst[(size_t)t * dst_rs + c] *= sigmoidf_(gate[(size_t)t * gate_rs + gate_off + c / group]);
}

// ── HEAD_LINEAR ──────────────────────────────────────────────────────────────────────────────────────────────────
struct HlArgs {
    float* dst; const float* src;
    uint32_t T, H, N, K, src_hs, src_rs, dst_hs, dst_rs;
};
constexpr int kHlRows = 8;
// few rows: one warp per (head, output), the weight row streamed once for all rows
template <typename WT>
__global__ void k_head_linear_rows(HlArgs a, const WT* __restrict__ W) {
    pdl_enter();
    const uint32_t n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31, h = blockIdx.y;
    if (n >= a.N) return;
    const WT* w = W + ((size_t)h * a.N + n) * a.K;
    const float* x = a.src + (size_t)h * a.src_hs;
    float acc[kHlRows];
#pragma unroll
    for (int m = 0; m < kHlRows; m++) acc[m] = 0.0f;
    for (uint32_t k = lane; k < a.K; k += 32) {
        const float wv = wld(w, k);
#pragma unroll
        for (int m = 0; m < kHlRows; m++)
            if (m < (int)a.T) acc[m] = fmaf(x[(size_t)m * a.src_rs + k], wv, acc[m]);
    }
#pragma unroll
    for (int m = 0; m < kHlRows; m++) {
        if (m < (int)a.T) {
            const float s = warp_sum(acc[m]);
            if (lane == 0) a.dst[(size_t)m * a.dst_rs + (size_t)h * a.dst_hs + n] = s;
        }
    }
}
// many rows, exact f32: 64 x 64 tile of one head, 16-deep k slices, 4 x 4 outputs per thread
constexpr int kHlTM = 64, kHlTN = 64, kHlTK = 16;
template <typename WT>
__global__ void __launch_bounds__(256) k_head_linear_tile(HlArgs a, const WT* __restrict__ W) {
    __shared__ float As[kHlTK][kHlTM + 4];
    __shared__ float Ws[kHlTK][kHlTN + 4];
    const uint32_t h = blockIdx.z, m0 = blockIdx.y * kHlTM, n0 = blockIdx.x * kHlTN;
    const uint32_t tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const float* src = a.src + (size_t)h * a.src_hs;
    const WT* Wh = W + (size_t)h * a.N * a.K;
    float acc[4][4] = {};
    for (uint32_t k0 = 0; k0 < a.K; k0 += kHlTK) {
        for (uint32_t e = threadIdx.x; e < kHlTM * kHlTK; e += 256) {
            const uint32_t r = e / kHlTK, kk = e % kHlTK;
            const uint32_t m = m0 + r, k = k0 + kk, n = n0 + r;
            As[kk][r] = (m < a.T && k < a.K) ? src[(size_t)m * a.src_rs + k] : 0.0f;
            Ws[kk][r] = (n < a.N && k < a.K) ? wld(Wh, (size_t)n * a.K + k) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kHlTK; kk++) {
            float x[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) { x[i] = As[kk][ty * 4 + i]; w[i] = Ws[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(x[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t m = m0 + ty * 4 + i;
        if (m >= a.T) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t n = n0 + tx * 4 + j;
            if (n < a.N) a.dst[(size_t)m * a.dst_rs + (size_t)h * a.dst_hs + n] = acc[i][j];
        }
    }
}

// ── POLY_NORM: one CTA per row ───────────────────────────────────────────────────────────────────────────────────
template <typename WT>
__global__ void k_poly_norm(float* dst, const float* src, const WT* __restrict__ coeff, uint32_t cols, float eps) {
    pdl_enter();
    __shared__ float sh[32];
    const float* z = src + (size_t)blockIdx.x * cols;
    float s2 = 0.0f, s4 = 0.0f, s6 = 0.0f;
    for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) {
        const float v = z[c], v2 = v * v, v3 = v2 * v;
        s2 = fmaf(v, v, s2); s4 = fmaf(v2, v2, s4); s6 = fmaf(v3, v3, s6);
    }
    const float n = (float)cols;
    const float i1 = wld(coeff, 0) / sqrtf(block_sum(s2, sh) / n + eps);
    const float i2 = wld(coeff, 1) / sqrtf(block_sum(s4, sh) / n + eps);
    const float i3 = wld(coeff, 2) / sqrtf(block_sum(s6, sh) / n + eps);
    const float e = wld(coeff, 3);
    float* out = dst + (size_t)blockIdx.x * cols;
    for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) {
        const float v = z[c], v2 = v * v;
        out[c] = fmaf(i1, v, fmaf(i2, v2, fmaf(i3, v2 * v, e)));
    }
}

}  // namespace

bool zg_mix_op_valid(const ZgOp& op, const size_t* elems, size_t n_bufs, char* why, size_t why_n) {
    const ZgSeqOp& s = op.u.seq;
    auto fail = [&](const char* m) { snprintf(why, why_n, "%s", m); return false; };
    auto have = [&](int i) { return s.buf[i] != ZG_NO_BUF && s.buf[i] < n_bufs; };
    auto fits = [&](int i, size_t off, size_t n) { return have(i) && off + n <= elems[s.buf[i]]; };
    auto wfits = [&](int i, uint32_t wdt, size_t off, size_t n) { return wdt <= ZG_W_BF16 && have(i) && (wdt == ZG_W_BF16 ? (off + n + 1) / 2 : off + n) <= elems[s.buf[i]]; };
    switch (op.tag) {
        case ZG_OP_TOKEN_SHIFT: {
            const size_t T = s.n[0], D = s.n[1];
            if (!T || !D) return fail("token_shift: shape");
            if (!fits(0, 0, T * D) || !fits(1, 0, T * D) || !wfits(2, s.n[2], s.off[0], D) || !have(3) || elems[s.buf[3]] < D || !fits(4, 0, ZG_CTL_IDS))
                return fail("token_shift: extent");
            if (s.buf[0] == s.buf[1]) return fail("token_shift: in place");
            return true;
        }
        case ZG_OP_DEPTH_MIX: {
            const size_t n = s.n[0], terms = s.n[1], stride = s.n[2];
            if (!n || !terms || stride < n) return fail("depth_mix: shape");
            if (!fits(0, 0, n) || !fits(1, 0, (terms - 1) * stride + n) || !wfits(2, s.n[3], s.off[0], terms)) return fail("depth_mix: extent");
            if (s.buf[0] == s.buf[1]) return fail("depth_mix: in place");
            return true;
        }
        case ZG_OP_ROTARY: {
            const size_t T = s.n[0], heads = s.n[1], hs = s.n[2], rs = s.n[3], dims = s.n[4];
            if (!T || !heads || !dims || dims % 2 || hs < dims || s.n[5] > 1 || !(s.f[0] > 0.0f)) return fail("rotary: shape");
            if (s.off[0] + (heads - 1) * hs + dims > rs) return fail("rotary: columns");
            if (!fits(0, 0, (T - 1) * rs + s.off[0] + (heads - 1) * hs + dims) || !fits(1, 0, ZG_CTL_IDS)) return fail("rotary: extent");
            if (s.buf[2] != ZG_NO_BUF) {
                const size_t shs = s.n[6], srs = s.n[7];
                if (shs < dims || s.off[1] + (heads - 1) * shs + dims > srs || !fits(2, 0, (T - 1) * srs + s.off[1] + (heads - 1) * shs + dims) || s.buf[2] == s.buf[0])
                    return fail("rotary: source");
            }
            return true;
        }
        case ZG_OP_CACHE_APPEND: {
            const size_t T = s.n[0], cols = s.n[1], srs = s.n[2], width = s.n[3], R = s.n[4];
            const size_t normed = s.n[5], rot = s.n[6];
            if (!T || !cols || R < T || s.off[0] + cols > srs || s.off[1] + cols > width || normed + rot > cols || rot % 2 || s.n[8] > 1) return fail("cache_append: shape");
            if (!have(0) || elems[s.buf[0]] < R * width || !fits(1, 0, (T - 1) * srs + s.off[0] + cols) || !fits(2, 0, ZG_CTL_IDS)) return fail("cache_append: extent");
            if (normed && !wfits(3, s.n[7], s.off[2], normed)) return fail("cache_append: norm weight");
            if (rot && !(s.f[1] > 0.0f)) return fail("cache_append: rotary base");
            return true;
        }
        case ZG_OP_CACHED_ATTENTION: {
            const size_t T = s.n[0], H = s.n[1], G = s.n[2], maps = s.n[3], dk = s.n[4], dv = s.n[5], qrs = s.n[6], kw = s.n[7], vw = s.n[8], R = s.n[9];
            const uint32_t kind = s.off[3], size = s.off[4];
            if (!T || !H || !G || H % G || !maps || !dk || !dv || dv > kCaMaxDv || kind > 2 || (kind && !size)) return fail("cached_attention: shape");
            if (R < T) return fail("cached_attention: cache rows");   // the caller sizes R for what the mask reaches and bounds the positions
            if (s.off[0] + H * maps * dk > qrs || s.off[1] + G * maps * dk > kw || s.off[2] + G * dv > vw) return fail("cached_attention: columns");
            if (!fits(0, 0, T * H * maps * dv) || !fits(1, 0, (T - 1) * qrs + s.off[0] + H * maps * dk) || !have(2) || elems[s.buf[2]] < R * kw || !have(3) ||
                elems[s.buf[3]] < R * vw || !fits(4, 0, ZG_CTL_IDS))
                return fail("cached_attention: extent");
            if (s.buf[0] == s.buf[1]) return fail("cached_attention: in place");
            return true;
        }
        case ZG_OP_MAP_COMBINE: {
            const size_t rows = s.n[0], dv = s.n[1];
            if (!rows || !dv) return fail("map_combine: shape");
            if (!fits(0, 0, rows * dv) || !fits(1, 0, rows * 2 * dv) || s.buf[0] == s.buf[1]) return fail("map_combine: extent");
            return true;
        }
        case ZG_OP_GATE: {
            const size_t T = s.n[0], cols = s.n[1], group = s.n[2], grs = s.n[3], drs = s.n[4];
            if (!T || !cols || !group || cols % group || drs < cols || s.off[0] + cols / group > grs) return fail("gate: shape");
            if (!fits(0, 0, (T - 1) * drs + cols) || !fits(1, 0, (T - 1) * grs + s.off[0] + cols / group)) return fail("gate: extent");
            return true;
        }
        case ZG_OP_HEAD_LINEAR: {
            const size_t T = s.n[0], H = s.n[1], N = s.n[2], K = s.n[3], shs = s.n[4], srs = s.n[5], dhs = s.n[6], drs = s.n[7];
            if (!T || !H || !N || !K || shs < K || dhs < N || s.off[1] + (H - 1) * shs + K > srs || s.off[2] + (H - 1) * dhs + N > drs) return fail("head_linear: shape");
            if (!fits(0, 0, (T - 1) * drs + s.off[2] + (H - 1) * dhs + N) || !fits(1, 0, (T - 1) * srs + s.off[1] + (H - 1) * shs + K) || !wfits(2, s.n[8], s.off[0], H * N * K))
                return fail("head_linear: extent");
            if (s.buf[0] == s.buf[1]) return fail("head_linear: in place");
            return true;
        }
        case ZG_OP_POLY_NORM: {
            const size_t n = (size_t)s.n[0] * s.n[1];
            if (!n) return fail("poly_norm: shape");
            if (!fits(0, 0, n) || !fits(1, 0, n) || !wfits(2, s.n[2], s.off[0], 4)) return fail("poly_norm: extent");
            return true;
        }
        default: return fail("not a sequence op");
    }
}

uint32_t zg_mix_op_writes(uint32_t tag) {
    return tag == ZG_OP_TOKEN_SHIFT ? (1u | (1u << 3)) : 1u;
}

size_t zg_mix_op_scratch_elems(const ZgOp& op) {
    (void)op;
    return 0;
}

bool zg_launch_mix_op(const ZgOp& op, float* const* bufs, float* scratch, cudaStream_t st) {
    (void)scratch;
    const ZgSeqOp& s = op.u.seq;
    switch (op.tag) {
        case ZG_OP_TOKEN_SHIFT: {
            const size_t n = (size_t)s.n[0] * s.n[1];
            ZG_SEQ_WDT(s.n[2], launch_pdl(k_token_shift<WT>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, bufs[s.buf[0]], bufs[s.buf[1]], wptr<WT>(bufs, s.buf[2], s.off[0]),
                                          bufs[s.buf[3]], bufs[s.buf[4]], s.n[0], s.n[1]));
            ZG_SEQ_CHECK();
            return true;
        }
        case ZG_OP_DEPTH_MIX:
            ZG_SEQ_WDT(s.n[3], launch_pdl(k_depth_mix<WT>, dim3((s.n[0] + 255) / 256), dim3(256), 0, st, bufs[s.buf[0]], bufs[s.buf[1]], wptr<WT>(bufs, s.buf[2], s.off[0]), s.n[0], s.n[1], s.n[2]));
            ZG_SEQ_CHECK();
            return true;
        case ZG_OP_ROTARY: {
            const size_t n = (size_t)s.n[0] * s.n[1] * (s.n[4] / 2);
            float* x = bufs[s.buf[0]] + s.off[0];
            const bool sep = s.buf[2] != ZG_NO_BUF;
            launch_pdl(k_rotary, dim3((unsigned)((n + 127) / 128)), dim3(128), 0, st, x, sep ? bufs[s.buf[2]] + s.off[1] : x, bufs[s.buf[1]], s.n[0], s.n[1], s.n[2], s.n[3], s.n[4], s.n[5],
                       sep ? s.n[6] : s.n[2], sep ? s.n[7] : s.n[3], s.f[0]);
            ZG_SEQ_CHECK();
            return true;
        }
        case ZG_OP_CACHE_APPEND:
            ZG_SEQ_WDT(s.n[5] ? s.n[7] : ZG_W_F32, launch_pdl(k_cache_append<WT>, dim3(s.n[0]), dim3(128), 0, st, bufs[s.buf[0]] + s.off[1], bufs[s.buf[1]] + s.off[0], bufs[s.buf[2]],
                                                             s.n[5] ? wptr<WT>(bufs, s.buf[3], s.off[2]) : nullptr, s.n[1], s.n[2], s.n[3], s.n[4], s.n[5], s.n[6], s.n[8], s.f[0], s.f[1]));
            ZG_SEQ_CHECK();
            return true;
        case ZG_OP_CACHED_ATTENTION: {
            CaArgs a;
            a.dst = bufs[s.buf[0]]; a.q = bufs[s.buf[1]]; a.kc = bufs[s.buf[2]]; a.vc = bufs[s.buf[3]]; a.ctl = bufs[s.buf[4]];
            a.T = s.n[0]; a.H = s.n[1]; a.G = s.n[2]; a.maps = s.n[3]; a.dk = s.n[4]; a.dv = s.n[5]; a.q_rs = s.n[6]; a.q_off = s.off[0];
            a.kw = s.n[7]; a.k_off = s.off[1]; a.vw = s.n[8]; a.v_off = s.off[2]; a.R = s.n[9]; a.kind = s.off[3]; a.size = s.off[4]; a.scale = s.f[0];
            const uint32_t warps = 4, items = a.T * a.H * a.maps;
            launch_pdl(k_cached_attention, dim3((items + warps - 1) / warps), dim3(warps * 32), warps * a.dk * sizeof(float), st, a);
            ZG_SEQ_CHECK();
            return true;
        }
        case ZG_OP_MAP_COMBINE:
            launch_pdl(k_map_combine, dim3((s.n[0] + 3) / 4), dim3(128), 0, st, bufs[s.buf[0]], bufs[s.buf[1]], s.n[0], s.n[1], s.f[0], s.f[1], s.f[2]);
            ZG_SEQ_CHECK();
            return true;
        case ZG_OP_GATE: {
            const size_t n = (size_t)s.n[0] * s.n[1];
            launch_pdl(k_gate, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, bufs[s.buf[0]], bufs[s.buf[1]], s.n[0], s.n[1], s.n[2], s.n[3], s.off[0], s.n[4]);
            ZG_SEQ_CHECK();
            return true;
        }
        case ZG_OP_HEAD_LINEAR: {
            HlArgs a;
            a.dst = bufs[s.buf[0]] + s.off[2]; a.src = bufs[s.buf[1]] + s.off[1];
            a.T = s.n[0]; a.H = s.n[1]; a.N = s.n[2]; a.K = s.n[3]; a.src_hs = s.n[4]; a.src_rs = s.n[5]; a.dst_hs = s.n[6]; a.dst_rs = s.n[7];
            ZG_SEQ_WDT(s.n[8], {
                const WT* W = wptr<WT>(bufs, s.buf[2], s.off[0]);
                if (a.T <= (uint32_t)kHlRows) launch_pdl(k_head_linear_rows<WT>, dim3((a.N + 7) / 8, a.H), dim3(256), 0, st, a, W);
                else k_head_linear_tile<WT><<<dim3((a.N + kHlTN - 1) / kHlTN, (a.T + kHlTM - 1) / kHlTM, a.H), 256, 0, st>>>(a, W);
            });
            ZG_SEQ_CHECK();
            return true;
        }
        case ZG_OP_POLY_NORM:
            ZG_SEQ_WDT(s.n[2], launch_pdl(k_poly_norm<WT>, dim3(s.n[0]), dim3(256), 0, st, bufs[s.buf[0]], bufs[s.buf[1]], wptr<WT>(bufs, s.buf[2], s.off[0]), s.n[1], s.f[0]));
            ZG_SEQ_CHECK();
            return true;
        default:
            zg_set_error("unsupported sequence op tag %u", op.tag);
            return false;
    }
}
