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
__global__ void __launch_bounds__(1024)
k_add_rmsnorm(__nv_bfloat16 *h, const __nv_bfloat16 *__restrict__ delta, const __nv_bfloat16 *__restrict__ w, float eps,
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

// ---------------------------------------------------------------- SwiGLU
__global__ void __launch_bounds__(256)
k_swiglu(const __nv_bfloat16 *__restrict__ g, const __nv_bfloat16 *__restrict__ u, __nv_bfloat16 *y, uint32_t n)
{
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = __hmul(__float2bfloat16_rn(silu_f(bf2f(g[i]))), u[i]);
}

// ---------------------------------------------------------------- q/k norm + RoPE + cache write
// grid (rows, q heads + kv heads), D / 2 threads.  Thread i of a head looks after the pair (i, i + D / 2) of the
// rotate-half convention; the first rot_dim elements are rotated with the caller's tables cos / sin [max_seq][rot_dim / 2]
// (the same fp32 tables as the eager path, so the results agree bit for bit), the rest pass through.
// q_norm / k_norm (per-head RMSNorm weights [D], may be null) are applied first.  q is rotated in place; k and v go
// into the caches [max_seq][kv heads][D] at position pos[0] + row.
__global__ void __launch_bounds__(128)
k_rope_kv(__nv_bfloat16 *q, const __nv_bfloat16 *__restrict__ k, const __nv_bfloat16 *__restrict__ v, const int32_t *pos,
          __nv_bfloat16 *k_cache, __nv_bfloat16 *v_cache, const __nv_bfloat16 *__restrict__ q_norm,
          const __nv_bfloat16 *__restrict__ k_norm, const float *__restrict__ cos_tab, const float *__restrict__ sin_tab,
          uint32_t hq, uint32_t hkv, uint32_t D, uint32_t rot_dim, float eps, uint32_t q_stride, uint32_t max_seq)
{
    __shared__ float red[32];
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t row = blockIdx.x, head = blockIdx.y, i = threadIdx.x, half = D / 2;
    const uint32_t p = (uint32_t)pos[0] + row;
    const bool is_q = head < hq;
    __nv_bfloat16 *src = is_q ? q + (size_t)row * q_stride + (size_t)head * D
                              : const_cast<__nv_bfloat16 *>(k) + ((size_t)row * hkv + (head - hq)) * D;
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
        const size_t at = ((size_t)min(p, max_seq - 1u) * hkv + (head - hq)) * D;
        dst_a = k_cache + at + i;
        dst_b = k_cache + at + i + half;
        const __nv_bfloat16 *vs = v + ((size_t)row * hkv + (head - hq)) * D;
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
// grid (q heads, splits), 256 threads (8 warps).  The context [0, n_ctx) (n_ctx = pos[0] + 1) is cut into `splits`
// contiguous ranges; a warp walks its share of a range one position at a time: D / 8 lanes hold 8 elements each of
// the position's K row (one 16-byte load), a shuffle tree gives the score, the warp keeps a running maximum,
// denominator and weighted V sum (online softmax).  The eight warps are joined in shared memory, the split's
// (maximum, denominator, sum[D]) goes to `part`; k_attn_combine joins the splits.
template <int D>
__global__ void __launch_bounds__(256)
k_attn_decode(const __nv_bfloat16 *__restrict__ q, const __nv_bfloat16 *__restrict__ k_cache,
              const __nv_bfloat16 *__restrict__ v_cache, const int32_t *pos, float *part, uint32_t hq, uint32_t hkv,
              float scale)
{
    constexpr int LPP = D / 8;                         // lanes per position
    constexpr int PPW = 32 / LPP;                      // positions per warp iteration
    __shared__ float sm_m[8 * PPW], sm_l[8 * PPW], sm_acc[8 * PPW][D];
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t head = blockIdx.x, split = blockIdx.y, splits = gridDim.y;
    const uint32_t kvh = head / (hq / hkv);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int sub = lane / LPP, li = lane % LPP;       // which of the warp's positions, which 8 elements
    const uint32_t n_ctx = (uint32_t)pos[0] + 1u;
    const uint32_t per = (n_ctx + splits - 1) / splits, p0 = split * per, p1 = min(p0 + per, n_ctx);
    float qv[8];
    {
        const uint4 raw = *(const uint4 *)(q + (size_t)head * D + li * 8);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            qv[2 * j] = __uint_as_float(w[j] << 16) * scale;
            qv[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u) * scale;
        }
    }
    float m = -INFINITY, l = 0.f, acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    // the trip count is the same for all lanes of a warp (the shuffles below need every lane); a lane whose position
    // lies beyond the range reads position p1 - 1 and drops the result
    for (uint32_t pb = p0 + (uint32_t)(wid * PPW); pb < p1; pb += 8 * PPW) {
        const bool live = pb + (uint32_t)sub < p1;
        const uint32_t p = live ? pb + (uint32_t)sub : p1 - 1u;
        const size_t off = ((size_t)p * hkv + kvh) * D + li * 8;
        const uint4 kr = *(const uint4 *)(k_cache + off);
        const uint4 vr = *(const uint4 *)(v_cache + off);
        const uint32_t kw[4] = {kr.x, kr.y, kr.z, kr.w}, vw[4] = {vr.x, vr.y, vr.z, vr.w};
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            s = fmaf(qv[2 * j], __uint_as_float(kw[j] << 16), s);
            s = fmaf(qv[2 * j + 1], __uint_as_float(kw[j] & 0xffff0000u), s);
        }
#pragma unroll
        for (int d = LPP / 2; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
        if (live) {
            const float mn = fmaxf(m, s), c = __expf(m - mn), e = __expf(s - mn);
            l = l * c + e;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                acc[2 * j] = fmaf(acc[2 * j], c, e * __uint_as_float(vw[j] << 16));
                acc[2 * j + 1] = fmaf(acc[2 * j + 1], c, e * __uint_as_float(vw[j] & 0xffff0000u));
            }
            m = mn;
        }
    }
    // join the 8 * PPW partial states of the CTA
    const int slot = wid * PPW + sub;
    if (li == 0) {
        sm_m[slot] = m;
        sm_l[slot] = l;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) sm_acc[slot][li * 8 + j] = acc[j];
    __syncthreads();
    float M = -INFINITY;
    for (int s2 = 0; s2 < 8 * PPW; ++s2) M = fmaxf(M, sm_m[s2]);
    float *out = part + ((size_t)head * splits + split) * (D + 2);
    if (threadIdx.x < D) {
        float a = 0.f;
        for (int s2 = 0; s2 < 8 * PPW; ++s2)
            if (sm_m[s2] != -INFINITY) a += sm_acc[s2][threadIdx.x] * __expf(sm_m[s2] - M);
        out[2 + threadIdx.x] = a;
    }
    if (threadIdx.x == 0) {
        float L = 0.f;
        for (int s2 = 0; s2 < 8 * PPW; ++s2)
            if (sm_m[s2] != -INFINITY) L += sm_l[s2] * __expf(sm_m[s2] - M);
        out[0] = M;
        out[1] = L;
    }
}

// grid q heads, D threads: out[head][d] = sum over the splits, optional sigmoid gate (gate[head][d], bf16)
__global__ void __launch_bounds__(256)
k_attn_combine(const float *__restrict__ part, __nv_bfloat16 *out, const __nv_bfloat16 *__restrict__ gate, uint32_t splits,
               uint32_t D, uint32_t gate_stride)
{
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t head = blockIdx.x, d = threadIdx.x;
    if (d >= D) return;
    const float *p = part + (size_t)head * splits * (D + 2);
    float M = -INFINITY;
    for (uint32_t s = 0; s < splits; ++s) M = fmaxf(M, p[s * (D + 2)]);
    float L = 0.f, a = 0.f;
    for (uint32_t s = 0; s < splits; ++s) {
        const float ms = p[s * (D + 2)];
        if (ms == -INFINITY) continue;
        const float c = __expf(ms - M);
        L += p[s * (D + 2) + 1] * c;
        a += p[s * (D + 2) + 2 + d] * c;
    }
    float o = bfround(a / L);
    if (gate) o = bf2f(__hmul(__float2bfloat16_rn(o), __float2bfloat16_rn(sigmoid_f(bf2f(gate[(size_t)head * gate_stride + d])))));
    out[(size_t)head * D + d] = __float2bfloat16_rn(o);
}

// ---------------------------------------------------------------- causal conv1d update (depth-wise, kernel K <= 8)
// state [C][K - 1] (bf16, oldest first) holds the last K - 1 inputs of every channel;
// y_c = silu(sum_j w[c][j] * input_{t - K + 1 + j} + bias_c), then the state takes x in.
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
__global__ void __launch_bounds__(256)
k_gdn_step(const __nv_bfloat16 *__restrict__ qkv, const __nv_bfloat16 *__restrict__ z, const __nv_bfloat16 *__restrict__ a_in,
           const __nv_bfloat16 *__restrict__ b_in, const float *__restrict__ A_log, const float *__restrict__ dt_bias,
           const __nv_bfloat16 *__restrict__ norm_w, float *state, __nv_bfloat16 *out, uint32_t hk, uint32_t hv, float eps)
{
    constexpr int DK = 128, DV = 128;
    __shared__ float red[32], qs[DK], ks[DK], part_k[2][DV], part_q[2][DV];
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t vh = blockIdx.x, kh = vh / (hv / hk);
    const uint32_t tid = threadIdx.x, j = tid & 127u, ih = tid >> 7;
    // qkv = [q (hk * DK) | k (hk * DK) | v (hv * DV)]
    const __nv_bfloat16 *qp = qkv + (size_t)kh * DK, *kp = qkv + (size_t)(hk + kh) * DK;
    const __nv_bfloat16 *vp = qkv + (size_t)2 * hk * DK + (size_t)vh * DV;
    float qe = 0.f, ke = 0.f;
    if (tid < DK) {
        qe = bf2f(qp[tid]);
        ke = bf2f(kp[tid]);
    }
    const float qn = cta_sum(qe * qe, red), kn = cta_sum(ke * ke, red);
    if (tid < DK) {
        qs[tid] = qe * rsqrtf(qn + 1e-6f) * rsqrtf((float)DK);
        ks[tid] = ke * rsqrtf(kn + 1e-6f);
    }
    __syncthreads();
    const float av = bf2f(a_in[vh]) + dt_bias[vh];
    const float sp = av > 20.f ? av : log1pf(__expf(av));
    const float g = __expf(-__expf(A_log[vh]) * sp), beta = sigmoid_f(bf2f(b_in[vh]));
    float *S = state + (size_t)vh * DK * DV;
    float s[64];
    float sk = 0.f, sq = 0.f;
#pragma unroll
    for (int i = 0; i < 64; ++i) {
        s[i] = S[(size_t)(64 * ih + i) * DV + j] * g;
        sk = fmaf(s[i], ks[64 * ih + i], sk);
        sq = fmaf(s[i], qs[64 * ih + i], sq);
    }
    part_k[ih][j] = sk;
    part_q[ih][j] = sq;
    float kq = 0.f;
    if (tid < DK) kq = ks[tid] * qs[tid];
    kq = cta_sum(kq, red);                             // k . q (also the barrier for part_k / part_q)
    const float kv_mem = part_k[0][j] + part_k[1][j];
    const float delta = (bf2f(vp[j]) - kv_mem) * beta;
#pragma unroll
    for (int i = 0; i < 64; ++i) S[(size_t)(64 * ih + i) * DV + j] = fmaf(ks[64 * ih + i], delta, s[i]);
    // o_j = sum_i (S_ij + k_i delta_j) q_i = (S^T q)_j + delta_j (k . q)
    const float o = part_q[0][j] + part_q[1][j] + delta * kq;
    const float ob = bfround(o);                       // the recurrence's output is a bf16 tensor in the eager path
    const float ss = cta_sum(ih == 0 ? ob * ob : 0.f, red);
    if (ih == 0) {
        const float r = rsqrtf(ss / (float)DV + eps);
        const __nv_bfloat16 nv = __hmul(__float2bfloat16_rn(ob * r), norm_w[j]);
        const float zg = silu_f(bf2f(z[(size_t)vh * DV + j]));
        out[(size_t)vh * DV + j] = __hmul(nv, __float2bfloat16_rn(zg));
    }
}

}  // namespace ixb
