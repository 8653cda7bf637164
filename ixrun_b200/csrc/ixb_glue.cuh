// Per-token glue of a decode step around the packed linears: the work between two GEMVs that the reference leaves
// to HuggingFace eager code and to fla's Triton kernels (ixrun/fla_patch.py:23-72; 63 of 138 ms per token in its own
// breakdown).  Batch-1 (up to 8 rows) kernels, one launch each, all of them usable inside a captured CUDA graph:
// positions and context lengths are read from device memory.
//
//   k_add_rmsnorm   h += delta (bf16), xn = rmsnorm(h) * w          residual add + the norm in front of the next GEMVs
//   k_swiglu        y = silu(g) * u                                 (the GEMV can also do this in its epilogue)
//   k_rope_kv       per-head q/k norm (optional), rotary embedding, K and V written into the static cache
//   k_attn_decode   one query per head over the static KV cache (grouped-query), split over the context,
//   k_attn_combine  the splits joined; optional sigmoid output gate
//   k_conv_update   causal depth-wise conv1d over the last K inputs of every channel + SiLU, state shifted
//   k_gdn_step      gated delta rule, one recurrent step per value head: state decay, delta update, read-out,
//                   gated RMSNorm of the head's output
//
// Arithmetic follows the eager reference path: inputs bf16, sums and transcendental functions in fp32, every value
// that the eager code would hold in a bf16 tensor is rounded to bf16 at the same place.
#pragma once
#include "ixb_common.cuh"

namespace ixb {

__device__ __forceinline__ float bf2f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float bfround(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float silu_f(float v) { return v / (1.f + __expf(-v)); }
__device__ __forceinline__ float sigmoid_f(float v) { return 1.f / (1.f + __expf(-v)); }

// sum over the CTA (blockDim.x a multiple of 32, at most 1024); every thread gets the result
__device__ __forceinline__ float cta_sum(float v, float *red)
{
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    v = warp_sum(v);
    __syncthreads();                                   // red may still be read from an earlier call
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float t = lane < nw ? red[lane] : 0.f;
    return warp_sum(t);
}

// ---------------------------------------------------------------- residual add + RMSNorm
// One CTA per row.  h (bf16, in/out) += delta (bf16, may be null); xn = bf16(h * rsqrt(mean(h^2) + eps)) * w.
// Generic form (any hidden size): two passes of scalar accesses.
__global__ void __launch_bounds__(1024)
k_add_rmsnorm_any(__nv_bfloat16 *h, const __nv_bfloat16 *__restrict__ delta, const __nv_bfloat16 *__restrict__ w, float eps,
                  __nv_bfloat16 *xn, uint32_t hidden)
{
    __shared__ float red[32];
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const size_t base = (size_t)blockIdx.x * hidden;
    float ss = 0.f;
    for (uint32_t i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = bf2f(h[base + i]);
        if (delta) {
            v = bfround(v + bf2f(delta[base + i]));
            h[base + i] = __float2bfloat16_rn(v);
        }
        ss += v * v;
    }
    ss = cta_sum(ss, red);
    const float r = rsqrtf(ss / (float)hidden + eps);
    for (uint32_t i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = bf2f(h[base + i]);             // this thread wrote it: visible to itself
        xn[base + i] = __hmul(__float2bfloat16_rn(v * r), w[i]);
    }
}

__device__ __forceinline__ void unpack8(const uint4 &r, float (&f)[8])
{
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        f[2 * j] = __uint_as_float(w[j] << 16);
        f[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
    }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8])
{
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
        w[j] = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f[2 * j])) |
               ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f[2 * j + 1])) << 16);
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// Where the residual's increment comes from when the row-parallel linear before this norm was sharded: the ranks'
// fp32 partial sums lie as marked words in this rank's exchange buffer (see ixb_allreduce.cuh; stored there by the
// epilogue of every rank's GEMV).  world == 0: the increment is the bf16 vector `delta` (or nothing).
struct NormExchange {
    const uint2 *mine;            // this rank's slots [2 parities][world][n_max]
    uint32_t *epoch;              // this rank's call counters
    uint32_t *err;
    uint32_t world, n_max, counters, spin_limit;
};

// Vector form: hidden a multiple of 8 and at most 8192 (5120 with an exchange); thread t keeps elements 8 t .. 8 t + 7 in registers, so the
// row is read once, with all loads in flight together; the norm weights are requested before the dependency wait.
// With an exchange (W > 0) the kernel is also the second half of the all-reduce: it waits (bounded) for every
// rank's words of this call, adds them in rank order and rounds the sum to bf16 (the value a separate finishing
// kernel would have written), then goes on as above; the last step advances the call counters.
constexpr int kNormExchangeThreads = 640;           // the exchange variant holds more registers: hidden <= 5120
template <int W>
__global__ void __launch_bounds__(W > 0 ? kNormExchangeThreads : 1024)
k_add_rmsnorm(__nv_bfloat16 *h, const __nv_bfloat16 *__restrict__ delta, NormExchange ex, const __nv_bfloat16 *__restrict__ w,
              float eps, __nv_bfloat16 *xn, uint32_t hidden)
{
    __shared__ float red[32];
    __shared__ uint32_t e_s;
    asm volatile("griddepcontrol.launch_dependents;");
    const uint32_t t = threadIdx.x, i = 8u * t;
    const bool on = i < hidden;
    const size_t base = (size_t)blockIdx.x * hidden;
    uint4 wr = make_uint4(0, 0, 0, 0);
    if (on) wr = *(const uint4 *)(w + i);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    float v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = 0.f;
    uint32_t e = 0;
    if (W > 0) {
        if (t == 0) e_s = ex.epoch[blockIdx.x] + 1u;
        __syncthreads();
        e = e_s;
    }
    if (on) {
        const uint4 hr = *(const uint4 *)(h + base + i);
        unpack8(hr, v);
        if (W > 0) {
            const uint32_t limit = *(volatile uint32_t *)ex.err ? 64u : ex.spin_limit;
            const uint2 *src0 = ex.mine + (size_t)((e & 1u) * W) * ex.n_max + base + i;
            constexpr int GRP = W < 4 ? (W > 0 ? W : 1) : 4;       // senders polled together (their loads are in flight at once)
            float o[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) o[k] = 0.f;
#pragma unroll
            for (int s0 = 0; s0 < W; s0 += GRP) {
                uint32_t val[GRP][8], mark[GRP][8];
                for (uint32_t polls = 0;; ++polls) {
                    bool all = true;
#pragma unroll
                    for (int s = 0; s < GRP; ++s) {
                        const uint2 *src = src0 + (size_t)(s0 + s) * ex.n_max;
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                                         : "=r"(val[s][2 * q]), "=r"(mark[s][2 * q]), "=r"(val[s][2 * q + 1]), "=r"(mark[s][2 * q + 1])
                                         : "l"(src + 2 * q) : "memory");
                    }
#pragma unroll
                    for (int s = 0; s < GRP; ++s)
#pragma unroll
                        for (int k = 0; k < 8; ++k) all = all && mark[s][k] == e;
                    if (all) break;
                    if (polls > limit) {
#pragma unroll
                        for (int s = 0; s < GRP; ++s)
#pragma unroll
                            for (int k = 0; k < 8; ++k)
                                if (mark[s][k] != e) *ex.err = 1u + (uint32_t)(s0 + s);   // that sender never arrived: wrong result, no hang
                        break;
                    }
                    __nanosleep(20);
                }
#pragma unroll
                for (int s = 0; s < GRP; ++s)                      // in rank order: the same bits on every rank
#pragma unroll
                    for (int k = 0; k < 8; ++k) o[k] += __uint_as_float(val[s][k]);
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = bfround(v[k] + bfround(o[k]));
            *(uint4 *)(h + base + i) = pack8(v);
        } else if (delta) {
            float d[8];
            unpack8(*(const uint4 *)(delta + base + i), d);
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = bfround(v[k] + d[k]);
            *(uint4 *)(h + base + i) = pack8(v);
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) ss += v[k] * v[k];
    ss = cta_sum(ss, red);
    const float r = rsqrtf(ss / (float)hidden + eps);
    if (on) {
        float wf[8], o[8];
        unpack8(wr, wf);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = bfround(v[k] * r) * wf[k];
        *(uint4 *)(xn + base + i) = pack8(o);
    }
    if (W > 0 && t == 0)
        for (uint32_t k = blockIdx.x; k < ex.counters; k += gridDim.x) ex.epoch[k] = e;   // all counters advance together
}

// ---------------------------------------------------------------- SwiGLU
// y [rows][cols] = silu(g) * u; g and u may be column slices of a wider matrix (row pitch in_stride elements, e.g. the
// two halves of a fused gate|up output).  vec: cols and in_stride multiples of 8 and 16-byte aligned pointers: eight
// values per thread; otherwise one value per thread.
__global__ void __launch_bounds__(128)
k_swiglu(const __nv_bfloat16 *__restrict__ g, const __nv_bfloat16 *__restrict__ u, __nv_bfloat16 *y, uint32_t rows,
         uint32_t cols, uint32_t in_stride, int vec)
{
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (vec) {
        const uint32_t per_row = cols / 8u, r = t / per_row, c = (t - r * per_row) * 8u;
        if (r >= rows) return;
        float a[8], b[8], o[8];
        unpack8(*(const uint4 *)(g + (size_t)r * in_stride + c), a);
        unpack8(*(const uint4 *)(u + (size_t)r * in_stride + c), b);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = bfround(silu_f(a[k])) * b[k];
        *(uint4 *)(y + (size_t)r * cols + c) = pack8(o);
    } else {
        const uint32_t r = t / cols, c = t - r * cols;
        if (r >= rows) return;
        y[(size_t)r * cols + c] = __hmul(__float2bfloat16_rn(silu_f(bf2f(g[(size_t)r * in_stride + c]))), u[(size_t)r * in_stride + c]);
    }
}

// ---------------------------------------------------------------- q/k norm + RoPE + cache write
// grid (rows, q heads + kv heads), D / 2 threads.  Thread i of a head looks after the pair (i, i + D / 2) of the
// rotate-half convention; the first rot_dim elements are rotated with the caller's tables cos / sin [max_seq][rot_dim / 2]
// (the same fp32 tables as the eager path, so the results agree bit for bit), the rest pass through.
// q_norm / k_norm (per-head RMSNorm weights [D], may be null) are applied first.  q is rotated in place; k and v go
// into the caches [max_seq][kv heads][D].  batch_stride == 0: the rows are consecutive positions pos[0] + row of one
// sequence; batch_stride > 0: row r is the newest token of sequence r, at position pos[r] of the cache that starts
// batch_stride elements after the one before it.  Row pitches of q, k / v: q_stride, kv_stride elements.
__global__ void __launch_bounds__(128)
k_rope_kv(__nv_bfloat16 *q, const __nv_bfloat16 *__restrict__ k, const __nv_bfloat16 *__restrict__ v, const int32_t *pos,
          __nv_bfloat16 *k_cache, __nv_bfloat16 *v_cache, const __nv_bfloat16 *__restrict__ q_norm,
          const __nv_bfloat16 *__restrict__ k_norm, const float *__restrict__ cos_tab, const float *__restrict__ sin_tab,
          uint32_t hq, uint32_t hkv, uint32_t D, uint32_t rot_dim, float eps, uint32_t q_stride, uint32_t max_seq,
          uint32_t kv_stride, size_t batch_stride)
{
    __shared__ float red[32];
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t row = blockIdx.x, head = blockIdx.y, i = threadIdx.x, half = D / 2;
    const uint32_t p = batch_stride ? (uint32_t)pos[row] : (uint32_t)pos[0] + row;
    const bool is_q = head < hq;
    __nv_bfloat16 *src = is_q ? q + (size_t)row * q_stride + (size_t)head * D
                              : const_cast<__nv_bfloat16 *>(k) + (size_t)row * kv_stride + (size_t)(head - hq) * D;
    float a = bf2f(src[i]), b = bf2f(src[i + half]);
    const __nv_bfloat16 *nw = is_q ? q_norm : k_norm;
    if (nw) {
        const float ss = cta_sum(a * a + b * b, red);
        const float r = rsqrtf(ss / (float)D + eps);
        a = bf2f(__hmul(__float2bfloat16_rn(a * r), nw[i]));
        b = bf2f(__hmul(__float2bfloat16_rn(b * r), nw[i + half]));
    }
    __nv_bfloat16 *dst_a, *dst_b;
    if (is_q) {
        dst_a = src + i;
        dst_b = src + i + half;
    } else {
        const size_t at = (size_t)row * batch_stride + ((size_t)min(p, max_seq - 1u) * hkv + (head - hq)) * D;
        dst_a = k_cache + at + i;
        dst_b = k_cache + at + i + half;
        const __nv_bfloat16 *vs = v + (size_t)row * kv_stride + (size_t)(head - hq) * D;
        v_cache[at + i] = vs[i];
        v_cache[at + i + half] = vs[i + half];
    }
    // rotate-half over the first rot_dim dimensions: element j < rot_dim / 2 pairs with j + rot_dim / 2 (with
    // rot_dim == D that is this thread's own pair); the head's elements meet in shared memory
    __shared__ float buf[256];
    __syncthreads();
    buf[i] = a;
    buf[i + half] = b;
    __syncthreads();
    const uint32_t rh = rot_dim / 2;
    auto rot = [&](uint32_t e) -> float {              // rotated value of element e
        if (e >= rot_dim) return buf[e];
        const uint32_t j = e < rh ? e : e - rh;
        const size_t ti = (size_t)min(p, max_seq - 1u) * rh + j;
        const float c = cos_tab[ti], s = sin_tab[ti];
        return e < rh ? buf[e] * c - buf[e + rh] * s : buf[e] * c + buf[e - rh] * s;
    };
    const float oa = rot(i), ob = rot(i + half);
    *dst_a = __float2bfloat16_rn(oa);
    *dst_b = __float2bfloat16_rn(ob);
}

// ---------------------------------------------------------------- single-query attention over the static cache
// grid (groups, splits), 256 threads (8 warps).  A group is G consecutive query heads that share one KV head
// (G = query heads per KV head, or 1): the K and V rows of a position are loaded once and used for all G heads.
// The context [0, n_ctx) (n_ctx = pos[0] + 1) is cut into `splits` contiguous ranges; a warp walks its share of a range
// PPW positions at a time: D / 8 lanes hold 8 elements each of a position's K and V rows (one 16-byte load each, the
// next iteration's rows requested before this one's arithmetic), a shuffle tree gives the G scores, and every
// lane keeps a running maximum, denominator and weighted V sum per head (online softmax).  The CTA's warps are joined
// in shared memory; the split's (maximum, denominator, sum[D]) per head goes to `part`; k_attn_combine joins the splits.
template <int D, int G>
__global__ void __launch_bounds__(256)
k_attn_decode(const __nv_bfloat16 *__restrict__ q, const __nv_bfloat16 *__restrict__ k_cache,
              const __nv_bfloat16 *__restrict__ v_cache, const int32_t *pos, float *part, uint32_t hq, uint32_t hkv,
              float scale, uint32_t q_stride, size_t batch_stride)
{
    // blockIdx.z: the sequence (its query row, its caches batch_stride elements after the previous one's, its position)
    q += (size_t)blockIdx.z * q_stride;
    k_cache += (size_t)blockIdx.z * batch_stride;
    v_cache += (size_t)blockIdx.z * batch_stride;
    pos += blockIdx.z;
    part += (size_t)blockIdx.z * hq * gridDim.y * (D + 2);
    constexpr int LPP = D / 8;                         // lanes per position
    constexpr int PPW = 32 / LPP;                      // positions per warp iteration
    constexpr int NS = 8 * PPW;                        // partial states per head in the CTA
    __shared__ float sm_m[G][NS], sm_l[G][NS];
    __shared__ float sm_acc[NS][D];                    // one head at a time
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t head0 = blockIdx.x * G, split = blockIdx.y, splits = gridDim.y;
    const uint32_t kvh = head0 / (hq / hkv);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int sub = lane / LPP, li = lane % LPP;       // which of the warp's positions, which 8 elements
    const uint32_t n_ctx = (uint32_t)pos[0] + 1u;
    const uint32_t per = (n_ctx + splits - 1) / splits, p0 = split * per, p1 = min(p0 + per, n_ctx);
    float qv[G][8];
#pragma unroll
    for (int h = 0; h < G; ++h) {
        unpack8(*(const uint4 *)(q + (size_t)(head0 + h) * D + li * 8), qv[h]);
#pragma unroll
        for (int j = 0; j < 8; ++j) qv[h][j] *= scale;
    }
    float m[G], l[G], acc[G][8];
#pragma unroll
    for (int h = 0; h < G; ++h) {
        m[h] = -INFINITY;
        l[h] = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[h][j] = 0.f;
    }
    // the trip count is the same for all lanes of a warp (the shuffles below need every lane); a lane whose position
    // lies beyond the range reads position p1 - 1 and drops the result
    const size_t row_stride = (size_t)hkv * D;
    const __nv_bfloat16 *kb = k_cache + (size_t)kvh * D + li * 8, *vb = v_cache + (size_t)kvh * D + li * 8;
    // a ring of PF iterations' rows in registers: the loads of iteration i + PF are requested before the arithmetic
    // of iteration i, so a warp has PF round trips to memory in flight
    constexpr int PF = 4;
    constexpr uint32_t STR = 8 * PPW;                  // positions the CTA covers per iteration
    uint32_t pb = p0 + (uint32_t)(wid * PPW);
    uint4 kq[PF], vq[PF];
#pragma unroll
    for (int st = 0; st < PF; ++st) {
        kq[st] = make_uint4(0, 0, 0, 0);
        vq[st] = kq[st];
        const uint32_t cur = pb + st * STR;
        if (cur < p1) {                                // warp uniform
            const uint32_t p = min(cur + (uint32_t)sub, p1 - 1u);
            kq[st] = *(const uint4 *)(kb + p * row_stride);
            vq[st] = *(const uint4 *)(vb + p * row_stride);
        }
    }
    for (; pb < p1; pb += PF * STR) {
#pragma unroll
        for (int st = 0; st < PF; ++st) {
            const uint32_t cur = pb + st * STR;
            if (cur >= p1) break;                      // warp uniform
            const bool live = cur + (uint32_t)sub < p1;
            float kf[8], vf[8];
            unpack8(kq[st], kf);
            unpack8(vq[st], vf);
            const uint32_t nxt = cur + PF * STR;
            if (nxt < p1) {                            // warp uniform
                const uint32_t p = min(nxt + (uint32_t)sub, p1 - 1u);
                kq[st] = *(const uint4 *)(kb + p * row_stride);
                vq[st] = *(const uint4 *)(vb + p * row_stride);
            }
#pragma unroll
            for (int h = 0; h < G; ++h) {
                float s = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) s = fmaf(qv[h][j], kf[j], s);
#pragma unroll
                for (int d = LPP / 2; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
                if (live) {
                    const float mn = fmaxf(m[h], s), c = __expf(m[h] - mn), e = __expf(s - mn);
                    l[h] = l[h] * c + e;
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[h][j] = fmaf(acc[h][j], c, e * vf[j]);
                    m[h] = mn;
                }
            }
        }
    }
    // join the NS partial states of the CTA, head by head
    const int slot = wid * PPW + sub;
    if (li == 0) {
#pragma unroll
        for (int h = 0; h < G; ++h) {
            sm_m[h][slot] = m[h];
            sm_l[h][slot] = l[h];
        }
    }
#pragma unroll
    for (int h = 0; h < G; ++h) {
        __syncthreads();                               // sm_acc is free (and, first time, sm_m / sm_l are written)
#pragma unroll
        for (int j = 0; j < 8; ++j) sm_acc[slot][li * 8 + j] = acc[h][j];
        __syncthreads();
        float M = -INFINITY;
#pragma unroll
        for (int s2 = 0; s2 < NS; ++s2) M = fmaxf(M, sm_m[h][s2]);
        float *out = part + ((size_t)(head0 + h) * splits + split) * (D + 2);
        if (threadIdx.x < D) {
            float a = 0.f;
#pragma unroll
            for (int s2 = 0; s2 < NS; ++s2)
                if (sm_m[h][s2] != -INFINITY) a += sm_acc[s2][threadIdx.x] * __expf(sm_m[h][s2] - M);
            out[2 + threadIdx.x] = a;
        }
        if (threadIdx.x == 0) {
            float L = 0.f;
            for (int s2 = 0; s2 < NS; ++s2)
                if (sm_m[h][s2] != -INFINITY) L += sm_l[h][s2] * __expf(sm_m[h][s2] - M);
            out[0] = M;
            out[1] = L;
        }
    }
}

// grid q heads, D threads: out[head][d] = sum over the splits, optional sigmoid gate (gate[head][d], bf16).
// The splits' maxima and denominators are fetched by one thread each, the weighted sums with independent loads.
constexpr int kAttnMaxSplits = 256;
__global__ void __launch_bounds__(256)
k_attn_combine(const float *__restrict__ part, __nv_bfloat16 *out, const __nv_bfloat16 *__restrict__ gate, uint32_t splits,
               uint32_t D, uint32_t gate_stride, uint32_t gate_row_stride)
{
    __shared__ float wgt[kAttnMaxSplits], red[32];
    asm volatile("griddepcontrol.launch_dependents;");
    const uint32_t head = blockIdx.x, t = threadIdx.x;
    // blockIdx.y: the sequence
    part += (size_t)blockIdx.y * gridDim.x * splits * (D + 2);
    out += (size_t)blockIdx.y * gridDim.x * D;
    if (gate) gate += (size_t)blockIdx.y * gate_row_stride;
    float gv = 0.f;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (gate && t < D) gv = bf2f(gate[(size_t)head * gate_stride + t]);
    const float *p = part + (size_t)head * splits * (D + 2);
    float ms = -INFINITY, ls = 0.f;
    if (t < splits) {
        const float2 ml = *(const float2 *)(p + (size_t)t * (D + 2));
        ms = ml.x;
        ls = ml.y;
    }
    // CTA-wide maximum
    float M = ms;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, d));
    if ((t & 31u) == 0) red[t >> 5] = M;
    __syncthreads();
    M = red[0];
    for (uint32_t i = 1; i < (blockDim.x >> 5); ++i) M = fmaxf(M, red[i]);
    const float c = ms == -INFINITY ? 0.f : __expf(ms - M);
    if (t < splits) wgt[t] = c;
    const float L = cta_sum(ls * c, red);              // (its barriers also publish wgt)
    if (t >= D) return;
    float a0 = 0.f, a1 = 0.f;
    const float *pt = p + 2 + t;
    uint32_t s2 = 0;
    for (; s2 + 16 <= splits; s2 += 16) {              // sixteen independent loads in flight
        float v[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) v[k] = pt[(size_t)(s2 + k) * (D + 2)];
#pragma unroll
        for (int k = 0; k < 16; k += 2) {
            a0 = fmaf(v[k], wgt[s2 + k], a0);
            a1 = fmaf(v[k + 1], wgt[s2 + k + 1], a1);
        }
    }
    {
        float v[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) v[k] = s2 + k < splits ? pt[(size_t)(s2 + k) * (D + 2)] : 0.f;
#pragma unroll
        for (int k = 0; k < 16; ++k) a0 = fmaf(v[k], s2 + k < splits ? wgt[s2 + k] : 0.f, a0);
    }
    const float a = a0 + a1;
    float o = bfround(a / L);
    if (gate) o = bfround(o) * bfround(sigmoid_f(gv));
    out[(size_t)head * D + t] = __float2bfloat16_rn(o);
}

// ---------------------------------------------------------------- causal conv1d update (depth-wise)
// state [C][K - 1] (bf16, oldest first) holds the last K - 1 inputs of every channel;
// y_c = silu(sum_j w[c][j] * input_{t - K + 1 + j} + bias_c), then the state takes x in.
// K == 4 and C a multiple of 4: a thread looks after four channels with 8- and 16-byte accesses, everything
// requested at once (the weights before the dependency wait); other shapes take the scalar kernel.
__global__ void __launch_bounds__(64)
k_conv_update4(const __nv_bfloat16 *__restrict__ x, __nv_bfloat16 *state, const __nv_bfloat16 *__restrict__ w,
               const __nv_bfloat16 *__restrict__ bias, __nv_bfloat16 *y, uint32_t C)
{
    asm volatile("griddepcontrol.launch_dependents;");
    const uint32_t c = 4u * (blockIdx.x * blockDim.x + threadIdx.x);
    const bool on = c < C;
    uint4 w0 = make_uint4(0, 0, 0, 0), w1 = w0;
    uint2 bb = make_uint2(0, 0);
    if (on) {
        w0 = *(const uint4 *)(w + (size_t)c * 4);
        w1 = *(const uint4 *)(w + (size_t)c * 4 + 8);
        if (bias) bb = *(const uint2 *)(bias + c);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (!on) return;
    uint2 *sp = (uint2 *)(state + (size_t)c * 3);      // 12 state values of the four channels: 24 bytes
    const uint2 s0 = sp[0], s1 = sp[1], s2 = sp[2];
    const uint2 xr = *(const uint2 *)(x + c);
    const uint32_t sw[6] = {s0.x, s0.y, s1.x, s1.y, s2.x, s2.y}, ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
    const uint32_t xw[2] = {xr.x, xr.y}, bw[2] = {bb.x, bb.y};
    auto half = [](const uint32_t *a, int i) { return __uint_as_float((i & 1) ? (a[i >> 1] & 0xffff0000u) : (a[i >> 1] << 16)); };
    auto bits = [](const uint32_t *a, int i) { return (i & 1) ? (a[i >> 1] >> 16) : (a[i >> 1] & 0xffffu); };
    uint32_t ns[12], yo[4];
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
        float acc = half(bw, ch);
#pragma unroll
        for (int j = 0; j < 3; ++j) acc = fmaf(half(ww, 4 * ch + j), half(sw, 3 * ch + j), acc);
        acc = fmaf(half(ww, 4 * ch + 3), half(xw, ch), acc);
        yo[ch] = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(silu_f(acc)));
        ns[3 * ch] = bits(sw, 3 * ch + 1);
        ns[3 * ch + 1] = bits(sw, 3 * ch + 2);
        ns[3 * ch + 2] = bits(xw, ch);
    }
    sp[0] = make_uint2(ns[0] | ns[1] << 16, ns[2] | ns[3] << 16);
    sp[1] = make_uint2(ns[4] | ns[5] << 16, ns[6] | ns[7] << 16);
    sp[2] = make_uint2(ns[8] | ns[9] << 16, ns[10] | ns[11] << 16);
    *(uint2 *)(y + c) = make_uint2(yo[0] | yo[1] << 16, yo[2] | yo[3] << 16);
}

__global__ void __launch_bounds__(256)
k_conv_update(const __nv_bfloat16 *__restrict__ x, __nv_bfloat16 *state, const __nv_bfloat16 *__restrict__ w,
              const __nv_bfloat16 *__restrict__ bias, __nv_bfloat16 *y, uint32_t C, uint32_t K)
{
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    __nv_bfloat16 *st = state + (size_t)c * (K - 1);
    const __nv_bfloat16 *wc = w + (size_t)c * K;
    const float xv = bf2f(x[c]);
    float acc = bias ? bf2f(bias[c]) : 0.f;
    for (uint32_t j = 0; j + 1 < K; ++j) {
        const float s = bf2f(st[j]);
        acc = fmaf(bf2f(wc[j]), s, acc);
        if (j + 2 < K) st[j] = st[j + 1];
    }
    acc = fmaf(bf2f(wc[K - 1]), xv, acc);
    st[K - 2] = x[c];
    y[c] = __float2bfloat16_rn(silu_f(acc));
}

// ---------------------------------------------------------------- gated delta rule, one step
// One CTA per value head, 256 threads: thread (j = tid & 127, ih = tid >> 7) owns column j of the head's state
// S [DK = 128][DV = 128] (fp32, row i = key dimension) for rows [64 ih, 64 ih + 64), in registers.
//   q, k: the key head's vectors (value head / (hv / hk)), L2-normalised here; q scaled by DK^-0.5
//   g = exp(-exp(A_log) * softplus(a + dt_bias)),  beta = sigmoid(b)
//   S <- g S;  delta = (v - S^T k) beta;  S <- S + k delta^T;  o = S^T q
//   o <- rmsnorm(o) * norm_w * silu(z)                                  (the head's gated output norm)
// The state is read once and written once.
// CONV: the causal depth-wise conv (K = 4) + SiLU of the layer runs in the same kernel on the channels this head needs
// (its key head's q and k, its own v): qkv is then the raw projection, conv_state [2][C][3] holds the last three inputs
// of every channel twice -- the step at position p reads copy p & 1 and writes copy (p + 1) & 1, because the value heads
// that share a key head all read its q / k channels while one of them (the first) writes them.
template <bool CONV>
__global__ void __launch_bounds__(256)
k_gdn_step(const __nv_bfloat16 *__restrict__ qkv, const __nv_bfloat16 *__restrict__ z, const __nv_bfloat16 *__restrict__ a_in,
           const __nv_bfloat16 *__restrict__ b_in, const float *__restrict__ A_log, const float *__restrict__ dt_bias,
           const __nv_bfloat16 *__restrict__ norm_w, float *state, __nv_bfloat16 *out, uint32_t hk, uint32_t hv, float eps,
           __nv_bfloat16 *conv_state, const __nv_bfloat16 *__restrict__ conv_w, const int32_t *pos, uint32_t C)
{
    constexpr int DK = 128, DV = 128;
    __shared__ float red[32], qs[DK], ks[DK], vs[DV], part_k[2][DV], part_q[2][DV];
    asm volatile("griddepcontrol.launch_dependents;");
    const uint32_t vh = blockIdx.x, rep = hv / hk, kh = vh / rep;
    const uint32_t tid = threadIdx.x, j = tid & 127u, ih = tid >> 7;
    // the head's state was last written by this kernel one token ago and its parameters are constants: both are
    // requested before the dependency wait, so the longest loads overlap the tail of the kernel ahead
    float *S = state + (size_t)vh * DK * DV;
    float s[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) s[i] = S[(size_t)(64 * ih + i) * DV + j];
    const float a_log = A_log[vh], dtb = dt_bias[vh], nw = bf2f(norm_w[j]);
    // qkv = [q (hk * DK) | k (hk * DK) | v (hv * DV)]; channels of this head
    const uint32_t cq = kh * DK + j, ck = (hk + kh) * DK + j, cv = 2u * hk * DK + vh * DV + j;
    // conv: thread j < 128 looks after q channel j and v channel j, thread 128 + j after k channel j
    const uint32_t c0 = ih == 0 ? cq : ck, c1 = cv;
    float cw0[4] = {0.f, 0.f, 0.f, 0.f}, cw1[4] = {0.f, 0.f, 0.f, 0.f}, st0[3] = {0.f, 0.f, 0.f}, st1[3] = {0.f, 0.f, 0.f};
    uint32_t par = 0;
    if (CONV) {
        par = (uint32_t)pos[0] & 1u;                     // (written at the end of the token step before this one)
        const __nv_bfloat16 *rd = conv_state + (size_t)par * C * 3;
#pragma unroll
        for (int k = 0; k < 4; ++k) cw0[k] = bf2f(conv_w[(size_t)c0 * 4 + k]);
#pragma unroll
        for (int k = 0; k < 3; ++k) st0[k] = bf2f(rd[(size_t)c0 * 3 + k]);
        if (ih == 0) {
#pragma unroll
            for (int k = 0; k < 4; ++k) cw1[k] = bf2f(conv_w[(size_t)c1 * 4 + k]);
#pragma unroll
            for (int k = 0; k < 3; ++k) st1[k] = bf2f(rd[(size_t)c1 * 3 + k]);
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    float qe = 0.f, ke = 0.f;
    if (CONV) {
        auto conv = [&](uint32_t c, const float (&w)[4], const float (&st)[3], bool write) -> float {
            const __nv_bfloat16 xin = qkv[c];
            float acc = 0.f;
#pragma unroll
            for (int k = 0; k < 3; ++k) acc = fmaf(w[k], st[k], acc);
            acc = fmaf(w[3], bf2f(xin), acc);
            if (write) {
                __nv_bfloat16 *wr = conv_state + ((size_t)(par ^ 1u) * C + c) * 3;
                wr[0] = __float2bfloat16_rn(st[1]);
                wr[1] = __float2bfloat16_rn(st[2]);
                wr[2] = xin;
            }
            return bfround(silu_f(acc));                 // the conv's output is a bf16 tensor in the eager path
        };
        const float y0 = conv(c0, cw0, st0, vh % rep == 0);      // q or k: written by the key head's first value head
        if (ih == 0) {
            qe = y0;
            vs[j] = conv(c1, cw1, st1, true);
        } else {
            ke = y0;
        }
    } else {
        if (ih == 0) {
            qe = bf2f(qkv[cq]);
            vs[j] = bf2f(qkv[cv]);
        } else {
            ke = bf2f(qkv[ck]);
        }
    }
    const float qn = cta_sum(qe * qe, red), kn = cta_sum(ke * ke, red);     // (q lives in threads 0..127, k in 128..255)
    if (ih == 0) qs[j] = qe * rsqrtf(qn + 1e-6f) * rsqrtf((float)DK);
    else ks[j] = ke * rsqrtf(kn + 1e-6f);
    __syncthreads();
    const float av = bf2f(a_in[vh]) + dtb;
    const float sp = av > 20.f ? av : log1pf(__expf(av));
    const float g = __expf(-__expf(a_log) * sp), beta = sigmoid_f(bf2f(b_in[vh]));
    float sk = 0.f, sq = 0.f;
#pragma unroll
    for (int i = 0; i < 64; ++i) {
        s[i] *= g;
        sk = fmaf(s[i], ks[64 * ih + i], sk);
        sq = fmaf(s[i], qs[64 * ih + i], sq);
    }
    part_k[ih][j] = sk;
    part_q[ih][j] = sq;
    float kq = 0.f;
    if (tid < DK) kq = ks[tid] * qs[tid];
    kq = cta_sum(kq, red);                             // k . q (also the barrier for part_k / part_q)
    const float kv_mem = part_k[0][j] + part_k[1][j];
    const float delta = (vs[j] - kv_mem) * beta;
#pragma unroll
    for (int i = 0; i < 64; ++i) S[(size_t)(64 * ih + i) * DV + j] = fmaf(ks[64 * ih + i], delta, s[i]);
    // o_j = sum_i (S_ij + k_i delta_j) q_i = (S^T q)_j + delta_j (k . q)
    const float o = part_q[0][j] + part_q[1][j] + delta * kq;
    const float ob = bfround(o);                       // the recurrence's output is a bf16 tensor in the eager path
    const float ss = cta_sum(ih == 0 ? ob * ob : 0.f, red);
    if (ih == 0) {
        const float r = rsqrtf(ss / (float)DV + eps);
        const __nv_bfloat16 nv = __float2bfloat16_rn(bfround(ob * r) * nw);
        const float zg = silu_f(bf2f(z[(size_t)vh * DV + j]));
        out[(size_t)vh * DV + j] = __hmul(nv, __float2bfloat16_rn(zg));
    }
}

}  // namespace ixb
